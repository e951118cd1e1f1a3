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
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned key_of(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
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
        const float l = c.logits[i];
        if (key_of(l) >= lim) s += MASS ? expf((l - c.max_logit) * c.inv_temp) : 1.f;
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

// One block per row.
__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits_all, int vocab, const int* __restrict__ slots,
              unsigned long long* __restrict__ rng_states, const int* __restrict__ history, int history_len,
              float temp, int top_k, float top_p, float repeat_penalty, int* __restrict__ out_tokens) {
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
        if (threadIdx.x == 0) out_tokens[row] = arg;
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
    if (threadIdx.x == 0) out_tokens[row] = s_best == 0x7fffffff ? arg : s_best;
}

__global__ void seed_rng_kernel(unsigned long long* states, const int* slots, const unsigned long long* seeds, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) states[slots[i]] = (seeds[i] * 0x9e3779b97f4a7c15ull) | 1ull;
}

}  // namespace

// logits: [rows, vocab] 32-bit, modified in place by the repeat penalty.  history
// (may be null): [rows, history_len] most recent first, -1 padded.
MOE_API int moe_sample(float* logits, int rows, int vocab, const int* slots, unsigned long long* rng_states,
                       const int* history, int history_len, float temp, int top_k, float top_p,
                       float repeat_penalty, int* out_tokens, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return (int)cudaErrorInvalidValue;
    sample_kernel<<<rows, THREADS, 0, stream>>>(logits, vocab, slots, rng_states, history, history_len, temp, top_k,
                                               top_p, repeat_penalty, out_tokens);
    return launch_status();
}

// state = seed * 0x9e3779b97f4a7c15 | 1 (src/sample.rs:7-9)
MOE_API int moe_seed_rng(unsigned long long* states, const int* slots, const unsigned long long* seeds, int n,
                         cudaStream_t stream) {
    if (n <= 0) return 0;
    seed_rng_kernel<<<(n + 127) / 128, 128, 0, stream>>>(states, slots, seeds, n);
    return launch_status();
}
