// Picking the next token from a row of logits, on the device.
//
// Order of operations (reference: src/sample.rs:80-140): repeat penalty on the
// recent history (l > 0 ? l / p : l * p, once per occurrence); temperature <= 0 is
// an argmax whose first maximum wins; otherwise top-k, p_i = exp((l_i - max) / temp)
// normalised, top-p keeps the shortest prefix of the descending order whose
// cumulative probability reaches top_p, and the draw takes the first element of
// that order whose cumulative probability exceeds r.  A single candidate consumes
// no random number.  The generator is xorshift64* (src/sample.rs:4-19).
//
// The descending order is never materialised: a cut "the first element where the
// cumulative weight reaches u" is found by a 32-step descent over the bits of an
// order-preserving integer key of the logit.  Logits that are exactly equal at a
// cut are kept (or dropped) together, and a draw that lands on equal logits takes
// the lowest index; the reference leaves the order of equal logits unspecified.
//
// Three kernels.  Greedy: every row is cut into chunks, one block each; a block folds its chunk's
// maximum into one 64-bit word per row (key, then lowest index) and the row's last block writes
// the token.  Sampling: a thread-block cluster per row keeps the row's keys and weights in its
// CTAs' shared memory and descends four bits a pass (a 16-bin histogram per pass, summed over
// the cluster through distributed shared memory in a fixed order, so a draw is reproducible).
// A vocabulary too large for the cluster's shared memory takes the third kernel, one block per
// row over global memory, one bit a pass.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

// Order-preserving integer key of a logit.  -0 counts as +0 and a NaN as -inf.
__device__ __forceinline__ unsigned key_of(float v) {
    if (v != v) v = -INFINITY;
    const unsigned b = __float_as_uint(v + 0.f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float logit_of(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct RowCtx {
    const float* logits;
    int vocab;
    float max_logit, inv_temp;
    float* red;
};

// sum over i of weight(i) for key(i) >= k and key(i) >= floor_key; weight = 1 (count) or exp((l - max) / temp)
template <bool MASS>
__device__ float mass_ge(const RowCtx& c, unsigned k, unsigned floor_key) {
    float s = 0.f;
    const unsigned lim = k > floor_key ? k : floor_key;
    for (int i = threadIdx.x; i < c.vocab; i += blockDim.x) {
        const unsigned kk = key_of(c.logits[i]);
        if (kk >= lim) s += MASS ? expf((logit_of(kk) - c.max_logit) * c.inv_temp) : 1.f;
    }
    return block_sum(s, c.red);
}

// largest key K with mass_ge(K) >= target (strict: > target); 0 if none
template <bool MASS>
__device__ unsigned descend(const RowCtx& c, float target, bool strict, unsigned floor_key) {
    unsigned K = 0;
    for (int b = 31; b >= 0; b--) {
        const unsigned cand = K | (1u << b);
        const float s = mass_ge<MASS>(c, cand, floor_key);
        if (strict ? (s > target) : (s >= target)) K = cand;
    }
    return K;
}

__device__ __forceinline__ float next_f32(unsigned long long* state) {
    unsigned long long x = *state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    *state = x;
    return (float)((x * 0x2545f4914f6cdd1dull) >> 40) / 16777216.0f;
}

// One block per row, over global memory: any vocabulary.
__global__ void __launch_bounds__(THREADS)
sample_global_kernel(float* __restrict__ logits_all, int vocab, const int* __restrict__ slots,
              unsigned long long* __restrict__ rng_states, const int* __restrict__ history, int history_len,
              float temp, int top_k, float top_p, float repeat_penalty, int* __restrict__ out_tokens,
              int* __restrict__ last_token) {
    __shared__ float red[32];
    __shared__ int s_best;
    __shared__ float s_r;
    const int row = blockIdx.x;
    float* logits = logits_all + (size_t)row * vocab;

    if (repeat_penalty != 1.0f && history) {
        if (threadIdx.x == 0) {
            const int* h = history + (size_t)row * history_len;   // most recent first, -1 padded
            for (int i = 0; i < history_len; i++) {
                const int t = h[i];
                if (t < 0 || t >= vocab) continue;
                const float l = logits[t];
                logits[t] = l > 0.f ? l / repeat_penalty : l * repeat_penalty;
            }
        }
        __syncthreads();
    }

    // maximum and its first index
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = logits[i];
        if (v > best) best = v, bi = i;
    }
    const float mx = block_max(best, red);
    if (threadIdx.x == 0) s_best = 0x7fffffff;
    __syncthreads();
    if (best == mx && bi != 0x7fffffff) atomicMin(&s_best, bi);
    __syncthreads();
    int arg = s_best;
    if (arg == 0x7fffffff) arg = 0;   // all NaN or -inf: as the reference's loop, index 0

    if (temp <= 0.f) {
        if (threadIdx.x == 0) {
            out_tokens[row] = arg;
            if (last_token) last_token[slots[row]] = arg;
        }
        return;
    }

    RowCtx c{logits, vocab, mx, 1.0f / temp, red};
    unsigned floor_key = 0;
    const int k = (top_k <= 0 || top_k > vocab) ? vocab : top_k;
    if (k < vocab) floor_key = descend<false>(c, (float)k, false, 0);
    float z = mass_ge<true>(c, 0, floor_key);
    if (top_p > 0.f && top_p < 1.f) {
        const unsigned kp = descend<true>(c, top_p * z, false, floor_key);
        if (kp > floor_key) floor_key = kp;
        z = mass_ge<true>(c, 0, floor_key);
    }
    const float count = mass_ge<false>(c, 0, floor_key);
    unsigned pick_key;
    if (count <= 1.5f) {
        pick_key = floor_key;   // one candidate: no random number is consumed
        if (count < 0.5f) pick_key = key_of(mx);
    } else {
        if (threadIdx.x == 0) s_r = next_f32(&rng_states[slots[row]]);
        __syncthreads();
        pick_key = descend<true>(c, s_r * z, true, floor_key);
        if (pick_key < floor_key) pick_key = floor_key;   // rounding left r beyond the sum: the last candidate
    }
    // lowest index carrying pick_key (the smallest kept key may be absent when it came
    // from the fallback above: then the smallest key >= it is taken)
    __syncthreads();
    if (threadIdx.x == 0) s_best = 0x7fffffff;
    __syncthreads();
    {
        int mine = 0x7fffffff;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            if (key_of(logits[i]) == pick_key) {
                mine = i;
                break;
            }
        if (mine != 0x7fffffff) atomicMin(&s_best, mine);
    }
    __syncthreads();
    if (s_best == 0x7fffffff) {
        // no element has exactly this key: take the smallest key >= pick_key (lowest index)
        unsigned bk = 0xffffffffu;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned kk = key_of(logits[i]);
            if (kk >= pick_key && kk < bk) bk = kk;
        }
        // block minimum of bk via float-free reduction
        __shared__ unsigned s_bk;
        if (threadIdx.x == 0) s_bk = 0xffffffffu;
        __syncthreads();
        atomicMin(&s_bk, bk);
        __syncthreads();
        const unsigned target = s_bk;
        int mine = 0x7fffffff;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            if (key_of(logits[i]) == target) {
                mine = i;
                break;
            }
        if (mine != 0x7fffffff) atomicMin(&s_best, mine);
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int tok = s_best == 0x7fffffff ? arg : s_best;
        out_tokens[row] = tok;
        if (last_token) last_token[slots[row]] = tok;      // the sequence's next input, kept on the device
    }
}

// ---- repeat penalty (ahead of the greedy and the cluster kernels) --------------------------------
__global__ void repeat_penalty_kernel(float* __restrict__ logits_all, int vocab, const int* __restrict__ history,
                                      int history_len, float repeat_penalty, int rows) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    float* logits = logits_all + (size_t)row * vocab;
    const int* h = history + (size_t)row * history_len;   // most recent first, -1 padded
    for (int i = 0; i < history_len; i++) {
        const int t = h[i];
        if (t < 0 || t >= vocab) continue;
        const float l = logits[t];
        logits[t] = l > 0.f ? l / repeat_penalty : l * repeat_penalty;
    }
}

// ---- greedy ----------------------------------------------------------------------------------------
constexpr int ARG_THREADS = 256;

// grid (chunks, rows).  best[row] is (key << 32) | ~index, so that the 64-bit maximum is the largest
// logit at its lowest index; it and tickets[row] are zero between launches.
__global__ void __launch_bounds__(ARG_THREADS)
argmax_kernel(const float* __restrict__ logits_all, int vocab, int chunk, const int* __restrict__ slots,
              unsigned long long* __restrict__ best, int* __restrict__ tickets, int* __restrict__ out_tokens,
              int* __restrict__ last_token) {
    __shared__ unsigned long long s_part[ARG_THREADS / 32];
    pdl_sync();
    const int row = blockIdx.y;
    const float* logits = logits_all + (size_t)row * vocab;
    const int lo = blockIdx.x * chunk, hi = min(vocab, lo + chunk);
    unsigned long long mine = 0;
#pragma unroll 4
    for (int i = lo + threadIdx.x; i < hi; i += ARG_THREADS) {
        const unsigned long long c = ((unsigned long long)key_of(logits[i]) << 32) | (unsigned)~i;
        mine = c > mine ? c : mine;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long c = __shfl_xor_sync(0xffffffffu, mine, o);
        mine = c > mine ? c : mine;
    }
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < ARG_THREADS / 32; w++) mine = s_part[w] > mine ? s_part[w] : mine;
        atomicMax(&best[row], mine);
        __threadfence();
        if (atomicAdd(&tickets[row], 1) == (int)gridDim.x - 1) {
            __threadfence();
            const unsigned long long top = atomicExch(&best[row], 0ull);
            tickets[row] = 0;
            const int tok = (int)~(unsigned)(top & 0xffffffffull);
            out_tokens[row] = tok;
            if (last_token) last_token[slots[row]] = tok;
        }
    }
}

// ---- sampling by a cluster per row -------------------------------------------------------------------
constexpr int ST = 512;       // threads of a CTA: 16 warps, one per bin of a pass
constexpr int NBIN = 16;      // four bits a pass
constexpr int MAILS = 32;

namespace cl {
__device__ __forceinline__ unsigned rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned size() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the 32-bit word at the same shared-memory address in CTA r of the cluster
__device__ __forceinline__ unsigned peer_u32(const void* local, unsigned r) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(local);
    unsigned pa, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(pa) : "r"(a), "r"(r));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(pa) : "memory");
    return v;
}
}  // namespace cl

enum { OP_SUM = 0, OP_MINU = 1, OP_MAXF = 2 };

// What a CTA of the cluster works with.
struct Row {
    unsigned* keys;     // [n] keys of this CTA's part of the row
    float* wt;          // [n] exp((l - max) / temp)
    float* col;         // [NBIN][ST] one column per thread: a pass adds without atomics, in a fixed order
    unsigned* mail;     // [2][MAILS] this CTA's values of the exchange under way (two, by parity)
    unsigned* res;      // [MAILS] the exchange's result
    float* red;         // [32] block reductions
    int n, lo;
    unsigned phase, ctas;
};

// Threads t < nv have put their CTA's value t into r.mail[(phase & 1) * MAILS + t]; afterwards
// r.res[t] holds the value reduced over the CTAs of the cluster, in rank order.  One cluster barrier
// an exchange: a CTA can overwrite a mail buffer only two exchanges later, by when every CTA has
// passed the barrier in between and so has read it.
template <int OP>
__device__ void exchange(Row& r, int nv) {
    cl::sync();
    if ((int)threadIdx.x < nv) {
        const unsigned* slot = r.mail + (r.phase & 1) * MAILS + threadIdx.x;
        unsigned acc = cl::peer_u32(slot, 0);
        for (unsigned c = 1; c < r.ctas; c++) {
            const unsigned v = cl::peer_u32(slot, c);
            if (OP == OP_SUM) acc = __float_as_uint(__uint_as_float(acc) + __uint_as_float(v));
            if (OP == OP_MINU) acc = v < acc ? v : acc;
            if (OP == OP_MAXF) acc = __float_as_uint(fmaxf(__uint_as_float(acc), __uint_as_float(v)));
        }
        r.res[threadIdx.x] = acc;
    }
    __syncthreads();
    r.phase++;
}

// mass and number of the candidates (keys >= floor_key) over the whole row
__device__ void totals(Row& r, unsigned floor_key, float* mass, float* count) {
    float m = 0.f, c = 0.f;
    for (int i = threadIdx.x; i < r.n; i += ST)
        if (r.keys[i] >= floor_key) m += r.wt[i], c += 1.f;
    m = block_sum(m, r.red);
    c = block_sum(c, r.red);
    if (threadIdx.x == 0) {
        r.mail[(r.phase & 1) * MAILS + 0] = __float_as_uint(m);
        r.mail[(r.phase & 1) * MAILS + 1] = __float_as_uint(c);
    }
    exchange<OP_SUM>(r, 2);
    *mass = __uint_as_float(r.res[0]);
    *count = __uint_as_float(r.res[1]);
}

// Largest key K such that the weight of the candidates with key >= K reaches `target` (strict:
// exceeds it); 0 if none does.  weight = exp((l - max) / temp), or 1 with MASS false.  Four bits a
// pass: the candidates that share K's bits so far fall into 16 bins by their next four bits.
template <bool MASS>
__device__ unsigned select_key(Row& r, float target, bool strict, unsigned floor_key) {
    unsigned K = 0;
    float above = 0.f;      // weight of the candidates whose key lies above every key that starts like K
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
        for (int b = 0; b < NBIN; b++) r.col[b * ST + threadIdx.x] = 0.f;
        for (int i = threadIdx.x; i < r.n; i += ST) {
            const unsigned k = r.keys[i];
            if (k >= floor_key && (shift == 28 || (k >> (shift + 4)) == (K >> (shift + 4))))
                r.col[((k >> shift) & 15u) * ST + threadIdx.x] += MASS ? r.wt[i] : 1.f;
        }
        __syncthreads();
        {   // warp b sums bin b over the threads
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < ST / 32; j++) s += r.col[warp * ST + lane + 32 * j];
            s = warp_sum(s);
            if (lane == 0) r.mail[(r.phase & 1) * MAILS + warp] = __float_as_uint(s);
        }
        exchange<OP_SUM>(r, NBIN);
        float cum = above;
        unsigned sel = 0;
        for (int b = NBIN - 1; b >= 1; b--) {
            const float next = cum + __uint_as_float(r.res[b]);
            if (strict ? (next > target) : (next >= target)) {
                sel = (unsigned)b;
                break;
            }
            cum = next;
        }
        if (shift == 28 && sel == 0) {
            // not even the whole of bin 0 may reach the target: then no key does
            const float all = cum + __uint_as_float(r.res[0]);
            if (!(strict ? (all > target) : (all >= target))) return 0u;      // the same in every thread and CTA
        }
        above = cum;
        K |= sel << shift;
    }
    return K;
}

// lowest index of the row whose key is `key`; 0x7fffffff if there is none
__device__ int first_index_of(Row& r, unsigned key, int* s_idx) {
    __syncthreads();
    if (threadIdx.x == 0) *s_idx = 0x7fffffff;
    __syncthreads();
    for (int i = threadIdx.x; i < r.n; i += ST)
        if (r.keys[i] == key) {
            atomicMin(s_idx, r.lo + i);
            break;
        }
    __syncthreads();
    if (threadIdx.x == 0) r.mail[(r.phase & 1) * MAILS] = (unsigned)*s_idx;
    exchange<OP_MINU>(r, 1);
    return (int)r.res[0];
}

// grid (1, rows, ctas) in clusters of `ctas` along z; CTA c holds elements [c * per_cta, ...) of its row.
__global__ void __launch_bounds__(ST)
sample_cluster_kernel(const float* __restrict__ logits_all, int vocab, int per_cta, const int* __restrict__ slots,
                      unsigned long long* __restrict__ rng_states, float temp, int top_k, float top_p,
                      int* __restrict__ out_tokens, int* __restrict__ last_token) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_idx;
    __shared__ unsigned s_key;
    Row r;
    r.keys = reinterpret_cast<unsigned*>(smem_raw);
    r.wt = reinterpret_cast<float*>(r.keys + per_cta);
    r.col = r.wt + per_cta;
    r.mail = reinterpret_cast<unsigned*>(r.col + NBIN * ST);
    r.res = r.mail + 2 * MAILS;
    r.red = reinterpret_cast<float*>(r.res + MAILS);
    r.phase = 0;
    r.ctas = cl::size();
    const unsigned rank = cl::rank();
    const int row = blockIdx.y;
    r.lo = (int)rank * per_cta;
    r.n = max(0, min(per_cta, vocab - r.lo));
    pdl_sync();
    const float* logits = logits_all + (size_t)row * vocab + r.lo;
    // every CTA reads the generator's state now; CTA 0 writes the next state at the very end,
    // after barriers that every CTA has passed
    unsigned long long rng = 0;
    if (threadIdx.x == 0) rng = rng_states[slots[row]];

    // keys into shared memory; the row's maximum and its first index
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < r.n; i += ST) {
        const unsigned k = key_of(logits[i]);
        r.keys[i] = k;
        const float v = logit_of(k);
        if (v > best) best = v, bi = r.lo + i;
    }
    const float mxl = block_max(best, r.red);
    if (threadIdx.x == 0) r.mail[0] = __float_as_uint(mxl);
    exchange<OP_MAXF>(r, 1);
    const float mx = __uint_as_float(r.res[0]);
    if (threadIdx.x == 0) s_idx = 0x7fffffff;
    __syncthreads();
    if (best == mx && bi != 0x7fffffff) atomicMin(&s_idx, bi);
    __syncthreads();
    if (threadIdx.x == 0) r.mail[(r.phase & 1) * MAILS] = (unsigned)s_idx;
    exchange<OP_MINU>(r, 1);
    int arg = (int)r.res[0];
    if (arg == 0x7fffffff) arg = 0;   // nothing above -inf: as the reference's loop, index 0

    int tok = arg;
    bool drew = false;
    if (mx > -INFINITY) {
        const float inv_temp = 1.0f / temp;
        for (int i = threadIdx.x; i < r.n; i += ST) r.wt[i] = expf((logit_of(r.keys[i]) - mx) * inv_temp);
        __syncthreads();
        unsigned floor_key = 0;
        const int k = (top_k <= 0 || top_k > vocab) ? vocab : top_k;
        if (k < vocab) floor_key = select_key<false>(r, (float)k, false, 0);
        float z, count;
        if (top_p > 0.f && top_p < 1.f) {
            totals(r, floor_key, &z, &count);
            const unsigned kp = select_key<true>(r, top_p * z, false, floor_key);
            if (kp > floor_key) floor_key = kp;
        }
        totals(r, floor_key, &z, &count);
        unsigned pick_key;
        if (count <= 1.5f) {
            pick_key = floor_key;   // one candidate: no random number is consumed
            if (count < 0.5f) pick_key = key_of(mx);
        } else {
            // every CTA draws the same number from its copy of the state
            float u = 0.f;
            if (threadIdx.x == 0) u = next_f32(&rng);
            if (threadIdx.x == 0) s_key = __float_as_uint(u);
            __syncthreads();
            u = __uint_as_float(s_key);
            drew = true;
            pick_key = select_key<true>(r, u * z, true, floor_key);
            if (pick_key < floor_key) pick_key = floor_key;   // rounding left r beyond the sum: the last candidate
        }
        int found = first_index_of(r, pick_key, &s_idx);
        if (found == 0x7fffffff) {
            // no element has exactly this key: the smallest key >= pick_key, at its lowest index
            __syncthreads();
            if (threadIdx.x == 0) s_key = 0xffffffffu;
            __syncthreads();
            unsigned bk = 0xffffffffu;
            for (int i = threadIdx.x; i < r.n; i += ST) {
                const unsigned kk = r.keys[i];
                if (kk >= pick_key && kk < bk) bk = kk;
            }
            atomicMin(&s_key, bk);
            __syncthreads();
            if (threadIdx.x == 0) r.mail[(r.phase & 1) * MAILS] = s_key;
            exchange<OP_MINU>(r, 1);
            found = first_index_of(r, r.res[0], &s_idx);
        }
        if (found != 0x7fffffff) tok = found;
    }
    cl::sync();      // no CTA leaves while another may still read its shared memory (or the generator's state)
    if (rank == 0 && threadIdx.x == 0) {
        out_tokens[row] = tok;
        if (last_token) last_token[slots[row]] = tok;
        if (drew) rng_states[slots[row]] = rng;
    }
}

__global__ void seed_rng_kernel(unsigned long long* states, const int* slots, const unsigned long long* seeds, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) states[slots[i]] = (seeds[i] * 0x9e3779b97f4a7c15ull) | 1ull;
}

// What the model thought of a token it committed (reference: src/generate.rs:78-105, `probe`):
// from the RAW logits of a row, logprob = logit[token] - logsumexp(row), and the `top` most likely
// tokens with their logprobs, strongest first (of equal logits the lower id first).  One block a row.
__global__ void __launch_bounds__(1024)
logprob_kernel(const float* __restrict__ logits_all, int vocab, const int* __restrict__ tokens, int top,
               float* __restrict__ out_lp, int* __restrict__ top_ids, float* __restrict__ top_lps) {
    __shared__ float red[32];
    __shared__ unsigned long long best[32];
    __shared__ unsigned long long s_prev;
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* logits = logits_all + (size_t)row * vocab;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, logits[i]);
    mx = block_max(mx, red);
    float sum = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = logits[i];
        if (v == v) sum += expf(v - mx);             // (a NaN counts for nothing, as in the samplers)
    }
    sum = block_sum(sum, red);
    const float lse = mx + logf(sum);
    if (threadIdx.x == 0) {
        const int t = tokens[row];
        out_lp[row] = (t >= 0 && t < vocab) ? logits[t] - lse : -INFINITY;
    }
    // A key that orders (logit descending, id ascending) as one unsigned number, larger = better:
    // the float's bits made monotone in the high word, the complement of the id in the low word.
    auto key_of = [](float v, int i) {
        unsigned u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        return ((unsigned long long)u << 32) | (unsigned)(0x7fffffff - i);
    };
    unsigned long long prev = ~0ull;                 // the key picked last: the next pick lies below it
    for (int k = 0; k < top; k++) {
        unsigned long long b = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = logits[i];
            if (v != v) continue;                    // (a NaN is no candidate)
            const unsigned long long key = key_of(v, i);
            if (key < prev && key > b) b = key;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
            b = other > b ? other : b;
        }
        if (lane == 0) best[warp] = b;
        __syncthreads();
        if (warp == 0) {
            b = lane < (int)(blockDim.x >> 5) ? best[lane] : 0;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
                b = other > b ? other : b;
            }
            if (lane == 0) {
                s_prev = b;
                const int id = b ? 0x7fffffff - (int)(unsigned)(b & 0xffffffffu) : -1;
                top_ids[(size_t)row * top + k] = id;
                top_lps[(size_t)row * top + k] = id >= 0 ? logits[id] - lse : -INFINITY;
            }
        }
        __syncthreads();
        prev = s_prev;                               // (0: fewer candidates than asked for, the rest stay -1)
    }
}

}  // namespace

// logits: [rows, vocab] float32, raw (before any penalty or temperature); tokens: [rows] the
// committed tokens.  out_lp [rows]; top_ids, top_lps [rows, top] (top may be 0, at most 64).
MOE_API int moe_logprobs(const float* logits, int rows, int vocab, const int* tokens, int top, float* out_lp,
                         int* top_ids, float* top_lps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || top < 0 || top > 64 || !tokens || !out_lp || (top && (!top_ids || !top_lps)))
        return (int)cudaErrorInvalidValue;
    logprob_kernel<<<rows, 1024, 0, stream>>>(logits, vocab, tokens, top, out_lp, top_ids, top_lps);
    return launch_status();
}

static size_t cluster_smem(int per_cta) {
    return (size_t)per_cta * 8 + (size_t)NBIN * ST * 4 + (size_t)(3 * MAILS + 32) * 4;
}

// Bytes of zeroed workspace that moe_sample wants for `rows` rows (the kernels leave it zeroed).
MOE_API long long moe_sample_workspace_bytes(int rows) { return (long long)rows * 16; }

// logits: [rows, vocab] 32-bit, modified in place by the repeat penalty.  history
// (may be null): [rows, history_len] most recent first, -1 padded.  last_token (may be null):
// per-slot table that also receives each row's token (the embedding reads it for a token id of -1,
// so that the next step can be launched before the host has seen this one's tokens).
// workspace: zeroed, moe_sample_workspace_bytes(rows) bytes, 8-byte aligned.  force_global: take the
// kernel that works over global memory whatever the vocabulary (for comparison).
MOE_API int moe_sample(float* logits, int rows, int vocab, const int* slots, unsigned long long* rng_states,
                       const int* history, int history_len, float temp, int top_k, float top_p,
                       float repeat_penalty, int* out_tokens, int* last_token, void* workspace,
                       long long workspace_bytes, int force_global, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return (int)cudaErrorInvalidValue;
    int ctas = vocab <= 4096 ? 1 : vocab <= 16384 ? 2 : vocab <= 65536 ? 4 : 8;
    const int per_cta = (((vocab + ctas - 1) / ctas) + 3) & ~3;
    const size_t smem = cluster_smem(per_cta);
    const bool greedy = temp <= 0.f;
    const size_t smem_max = 227 * 1024 - 256;      // the kernel has a few static words besides
    const bool fits = smem <= smem_max && vocab < (1 << 24) && rows <= 65535;
    if (force_global || (!greedy && !fits) || (greedy && (workspace_bytes < (long long)rows * 16 || rows > 65535))) {
        sample_global_kernel<<<rows, THREADS, 0, stream>>>(logits, vocab, slots, rng_states, history, history_len, temp,
                                                          top_k, top_p, repeat_penalty, out_tokens, last_token);
        return launch_status();
    }
    if (repeat_penalty != 1.0f && history) {
        repeat_penalty_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(logits, vocab, history, history_len,
                                                                     repeat_penalty, rows);
        const int e = launch_status();
        if (e) return e;
    }
    if (greedy) {
        int chunk = 2048;
        while ((vocab + chunk - 1) / chunk > 128) chunk *= 2;
        unsigned long long* best = (unsigned long long*)workspace;
        int* tickets = (int*)(best + rows);
        return launch_pdl(argmax_kernel, dim3((vocab + chunk - 1) / chunk, rows), dim3(ARG_THREADS), 0, stream,
                          (const float*)logits, vocab, chunk, slots, best, tickets, out_tokens, last_token);
    }
    static bool attr_set = false;
    if (!attr_set) {
        const int e = (int)cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)smem_max);
        if (e) return e;
        attr_set = true;
    }
    return launch_pdl_cluster(sample_cluster_kernel, dim3(1, rows, ctas), dim3(ST), smem, stream, ctas,
                              (const float*)logits, vocab, per_cta, slots, rng_states, temp, top_k, top_p, out_tokens,
                              last_token);
}

// state = seed * 0x9e3779b97f4a7c15 | 1 (src/sample.rs:7-9)
MOE_API int moe_seed_rng(unsigned long long* states, const int* slots, const unsigned long long* seeds, int n,
                         cudaStream_t stream) {
    if (n <= 0) return 0;
    seed_rng_kernel<<<(n + 127) / 128, 128, 0, stream>>>(states, slots, seeds, n);
    return launch_status();
}
