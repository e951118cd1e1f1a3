// Routing and the glue of the expert feed-forward.
//
// Router (reference: src/model.rs:844-897): logits = Wr n; sc = softmax over ALL
// experts; the top k by descending sc (a tie goes to the lower expert index, as in
// scripts/oracle.py:323); w = max(sc, 0); if norm_topk: w /= max(sum w, 1e-20);
// w *= routed_scaling_factor.  Logits, softmax and the pick are 32-bit.
// Shared-expert gate (src/model.rs:959-966): g = sigmoid(Wsg . n), one scalar a token.
//
// Dispatch (src/model.rs:902-942) inverts the (token, expert) table so that an
// expert's weights are read once for all of its tokens; the combine step sums a
// token's k expert outputs in pick order, then adds the gated shared expert.
#include "common.cuh"

namespace {

constexpr int TOK_TILE = 8;         // tokens per block: a weight row is read once for all of them

template <typename WT>
__device__ __forceinline__ void w_load8(const WT* p, float* out);
template <>
__device__ __forceinline__ void w_load8<float>(const float* p, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x, out[1] = a.y, out[2] = a.z, out[3] = a.w, out[4] = b.x, out[5] = b.y, out[6] = b.z, out[7] = b.w;
}
template <>
__device__ __forceinline__ void w_load8<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// logits[t, r] = h[t, :] . W[r, :] for r < rows; row `num_experts` (if wsg) is the shared gate.
// 32-bit products and sums in a fixed order.  A block has ROWS x KSPLIT warps: warp (r, ks) takes
// router row r and the ks-th slice of the hidden dimension for 8 tokens; the slices are added in
// order.  Few tokens: many small blocks (ROWS 2, KSPLIT 4); many tokens: ROWS 8, KSPLIT 1, so that
// the activations are re-read 8 times less.  Grid: (ceil(rows / ROWS), ceil(T / 8)).
template <typename WT, int ROWS, int KSPLIT>
__global__ void __launch_bounds__(ROWS * KSPLIT * 32)
router_logits_kernel(const float* __restrict__ h, const WT* __restrict__ wr, const WT* __restrict__ wsg,
                     int num_tokens, int hidden, int num_experts, int rows, int vec_ok,
                     float* __restrict__ logits) {
    __shared__ float part[ROWS][KSPLIT][TOK_TILE];
    pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rr = warp / KSPLIT, ks = warp % KSPLIT;
    const int r = blockIdx.x * ROWS + rr;
    const int t0 = blockIdx.y * TOK_TILE;
    const int nt = min(TOK_TILE, num_tokens - t0);
    float acc[TOK_TILE];
#pragma unroll
    for (int i = 0; i < TOK_TILE; i++) acc[i] = 0.f;
    if (r < rows) {
        const WT* w = r < num_experts ? wr + (size_t)r * hidden : wsg;
        // slice of the hidden dimension of this warp, in whole groups of 8 elements
        const int groups = vec_ok ? hidden / 8 : 0;
        const int gper = (groups + KSPLIT - 1) / KSPLIT;
        const int g0 = ks * gper, g1 = min(groups, g0 + gper);
#pragma unroll 2
        for (int gi = g0 + lane; gi < g1; gi += 32) {
            const int c = gi * 8;
            float wv[8];
            w_load8<WT>(w + c, wv);
#pragma unroll
            for (int i = 0; i < TOK_TILE; i++) {
                if (i < nt) {
                    const float* x = h + (size_t)(t0 + i) * hidden + c;
                    const float4 a = *reinterpret_cast<const float4*>(x), b = *reinterpret_cast<const float4*>(x + 4);
                    float s = acc[i];
                    s = fmaf(a.x, wv[0], s), s = fmaf(a.y, wv[1], s), s = fmaf(a.z, wv[2], s), s = fmaf(a.w, wv[3], s);
                    s = fmaf(b.x, wv[4], s), s = fmaf(b.y, wv[5], s), s = fmaf(b.z, wv[6], s), s = fmaf(b.w, wv[7], s);
                    acc[i] = s;
                }
            }
        }
        if (ks == KSPLIT - 1) {   // the elements past the last whole group
            for (int c = groups * 8 + lane; c < hidden; c += 32) {
                const float wv = ld_f(w + c);
#pragma unroll
                for (int i = 0; i < TOK_TILE; i++)
                    if (i < nt) acc[i] = fmaf(h[(size_t)(t0 + i) * hidden + c], wv, acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TOK_TILE; i++) {
        const float s = warp_sum(acc[i]);
        if (lane == 0) part[rr][ks][i] = s;
    }
    __syncthreads();
    if (ks == 0 && lane < nt && r < rows) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < KSPLIT; k++) s += part[rr][k][lane];
        logits[(size_t)(t0 + lane) * rows + r] = s;
    }
}

// The same product for many tokens (a prompt): a block takes 8 router rows (one per warp) and 16
// tokens, and walks the hidden dimension in chunks of 512 that are staged in shared memory, so
// that an activation is read from global memory once per 8 rows and a weight once per 16 tokens.
// hidden must be a multiple of 8.  Grid: (ceil(rows / 8), ceil(T / 16)).
constexpr int PT = 16, PKC = 512;
template <typename WT>
__global__ void __launch_bounds__(256)
router_logits_tiled_kernel(const float* __restrict__ h, const WT* __restrict__ wr, const WT* __restrict__ wsg,
                           int num_tokens, int hidden, int num_experts, int rows, float* __restrict__ logits) {
    __shared__ __align__(16) float xs[PT][PKC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * PT;
    const int nt = min(PT, num_tokens - t0);
    const WT* w = r < num_experts ? wr + (size_t)r * hidden : wsg;
    float acc[PT];
#pragma unroll
    for (int i = 0; i < PT; i++) acc[i] = 0.f;
    for (int c0 = 0; c0 < hidden; c0 += PKC) {
        const int kc = min(PKC, hidden - c0);            // a multiple of 8
        __syncthreads();
        for (int idx = threadIdx.x; idx < PT * (PKC / 4); idx += blockDim.x) {
            const int i = idx / (PKC / 4), c = (idx % (PKC / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < nt && c < kc) v = *reinterpret_cast<const float4*>(h + (size_t)(t0 + i) * hidden + c0 + c);
            *reinterpret_cast<float4*>(&xs[i][c]) = v;
        }
        __syncthreads();
        if (r < rows) {
            for (int c = lane * 8; c < kc; c += 256) {
                float wv[8];
                w_load8<WT>(w + c0 + c, wv);
#pragma unroll
                for (int i = 0; i < PT; i++) {
                    const float4 a = *reinterpret_cast<const float4*>(&xs[i][c]);
                    const float4 b = *reinterpret_cast<const float4*>(&xs[i][c + 4]);
                    float s = acc[i];
                    s = fmaf(a.x, wv[0], s), s = fmaf(a.y, wv[1], s), s = fmaf(a.z, wv[2], s), s = fmaf(a.w, wv[3], s);
                    s = fmaf(b.x, wv[4], s), s = fmaf(b.y, wv[5], s), s = fmaf(b.z, wv[6], s), s = fmaf(b.w, wv[7], s);
                    acc[i] = s;
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < PT; i++) {
        const float s = warp_sum(acc[i]);
        if (lane == 0 && i < nt && r < rows) logits[(size_t)(t0 + i) * rows + r] = s;
    }
}

// The product for a whole prompt, register-tiled: a block of 128 threads takes 128 tokens x 64
// router rows and a slice of the hidden dimension; a thread holds 8 x 8 sums and walks its slice
// in order, so that every operand fetched from shared memory feeds 8 multiply-adds.  The slices'
// partial sums go to part[slice][token][row]; sum_slices_kernel adds them in slice order.
// hidden must be a multiple of 8 and the slice length of 16.
constexpr int ST = 128, SR = 64, SK = 16;
template <typename WT>
__global__ void __launch_bounds__(128)
router_logits_sgemm_kernel(const float* __restrict__ h, const WT* __restrict__ wr, const WT* __restrict__ wsg,
                           int num_tokens, int hidden, int num_experts, int rows, int kper,
                           float* __restrict__ part) {
    __shared__ __align__(16) float Xs[SK][ST + 4];
    __shared__ __align__(16) float Ws[SK][SR + 4];
    pdl_sync();
    const int tid = threadIdx.x, tg = tid % 16, rg = tid / 16;
    const int t0 = blockIdx.x * ST, r0 = blockIdx.z * SR;
    const int k0 = blockIdx.y * kper, k1 = min(hidden, k0 + kper);
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
    const int xt = t0 + tid;                         // the token whose activations this thread stages
    const int wrow = r0 + tid / 2, whalf = tid % 2;   // the router row and the half of the chunk it stages
    const WT* wp = wrow < num_experts ? wr + (size_t)wrow * hidden : wsg;
    for (int kk = k0; kk < k1; kk += SK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (xt < num_tokens && kk + 4 * j < k1) v = *reinterpret_cast<const float4*>(h + (size_t)xt * hidden + kk + 4 * j);
            Xs[4 * j + 0][tid] = v.x, Xs[4 * j + 1][tid] = v.y, Xs[4 * j + 2][tid] = v.z, Xs[4 * j + 3][tid] = v.w;
        }
        {
            float wv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (wrow < rows && kk + whalf * 8 < k1) w_load8<WT>(wp + kk + whalf * 8, wv);
#pragma unroll
            for (int i = 0; i < 8; i++) Ws[whalf * 8 + i][tid / 2] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SK; k++) {
            const float4 a0 = *reinterpret_cast<const float4*>(&Xs[k][tg * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&Xs[k][64 + tg * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Ws[k][rg * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Ws[k][32 + rg * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* out = part + (size_t)blockIdx.y * num_tokens * rows;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int t = t0 + (i < 4 ? tg * 4 + i : 64 + tg * 4 + i - 4);
        if (t >= num_tokens) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int r = r0 + (j < 4 ? rg * 4 + j : 32 + rg * 4 + j - 4);
            if (r < rows) out[(size_t)t * rows + r] = acc[i][j];
        }
    }
}

__global__ void sum_slices_kernel(const float* __restrict__ part, float* __restrict__ out, size_t n, int slices) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int k = 0; k < slices; k++) s += part[(size_t)k * n + i];
    out[i] = s;
}

// Softmax over all experts, top-k and weights of ONE token, by one warp.  `sc` is shared memory
// of num_experts floats owned by the warp.
__device__ __forceinline__ void route_token(const float* __restrict__ lg, float* sc, int lane, bool padding,
                                            int num_experts, int rows, int top_k, int norm_topk, float scale,
                                            int* __restrict__ idx_out, float* __restrict__ w_out,
                                            float* __restrict__ gate_out, float* wk = nullptr) {
    // wk: top_k floats of shared memory for the picked weights before scaling (else they are
    // staged in w_out itself, which costs round trips to global memory)
    if (!wk) wk = w_out;
    if (padding) {   // a row that belongs to no sequence: no expert
        for (int j = lane; j < top_k; j += 32) idx_out[j] = -1, w_out[j] = 0.f;
        if (gate_out && lane == 0) *gate_out = 0.f;
        return;
    }
    if (gate_out && rows > num_experts && lane == 0) *gate_out = 1.0f / (1.0f + expf(-lg[num_experts]));
    float m = -INFINITY;
    for (int e = lane; e < num_experts; e += 32) m = fmaxf(m, lg[e]);
    m = warp_max(m);
    float z = 0.f;
    for (int e = lane; e < num_experts; e += 32) {
        const float v = expf(lg[e] - m);
        sc[e] = v;
        z += v;
    }
    z = warp_sum(z);
    for (int e = lane; e < num_experts; e += 32) sc[e] = sc[e] / z;
    __syncwarp();
    float wsum = 0.f;
    for (int j = 0; j < top_k; j++) {
        float best = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < num_experts; e += 32) {
            const float v = sc[e];
            if (v > best) best = v, bi = e;   // ascending e: first maximum kept
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
        }
        if (bi < 0 || bi >= num_experts) bi = j % num_experts;   // only with NaN scores
        const float w = fmaxf(best, 0.f);
        wsum += w;
        if (lane == 0) {
            sc[bi] = -2.f;   // taken
            idx_out[j] = bi;
            wk[j] = w;
        }
        __syncwarp();
    }
    const float zz = norm_topk ? fmaxf(wsum, 1e-20f) : 1.0f;   // wsum is the same in every lane
    if (wk != w_out) {
        for (int j = lane; j < top_k; j += 32) {
            float w = wk[j];
            if (norm_topk) w = w / zz;
            w_out[j] = w * scale;
        }
    } else if (lane == 0) {
        for (int j = 0; j < top_k; j++) {
            float w = w_out[j];
            if (norm_topk) w = w / zz;
            w_out[j] = w * scale;
        }
    }
}

// One warp per token.  With `part` (the partial sums of router_logits_sgemm_kernel, `slices` of
// them) the warp first adds its token's slices in slice order and writes the logits, which spares
// the launch of sum_slices_kernel.
__global__ void __launch_bounds__(128)
router_topk_kernel(float* __restrict__ logits, const float* __restrict__ part, int slices,
                   const int* __restrict__ seq_of_token, int num_tokens, int num_experts, int rows, int top_k,
                   int norm_topk, float scale, int* __restrict__ topk_idx, float* __restrict__ topk_w,
                   float* __restrict__ shared_gate) {
    extern __shared__ float sc_all[];   // per warp: rows logits, num_experts scores, top_k weights
    pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= num_tokens) return;
    float* lg = sc_all + (size_t)warp * (rows + num_experts + top_k);
    const size_t n = (size_t)num_tokens * rows;
    for (int r = lane; r < rows; r += 32) {
        float s;
        if (part) {
            s = 0.f;
            for (int k = 0; k < slices; k++) s += part[(size_t)k * n + (size_t)t * rows + r];
            logits[(size_t)t * rows + r] = s;
        } else {
            s = logits[(size_t)t * rows + r];
        }
        lg[r] = s;
    }
    __syncwarp();
    route_token(lg, lg + rows, lane, seq_of_token && seq_of_token[t] < 0, num_experts, rows, top_k, norm_topk, scale,
                topk_idx + (size_t)t * top_k, topk_w + (size_t)t * top_k, shared_gate ? shared_gate + t : nullptr,
                lg + rows + num_experts);
}

// Inverting the (token, expert) table, by one block.  pairs = tokens * top_k entries of topk_idx
// (expert id, or -1).  counts and cursor are shared memory of num_experts ints each.
__device__ __forceinline__ void align_block(const int* __restrict__ topk_idx, int pairs, int top_k, int num_experts,
                                            int* counts, int* cursor, int* __restrict__ offsets,
                                            int* __restrict__ sorted_token, int* __restrict__ pos_of_pair,
                                            int* status) {
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = topk_idx[i];
        if (e >= 0 && e < num_experts)
            atomicAdd(&counts[e], 1);
        else if (e != -1)
            atomicOr(status, ST_BAD_EXPERT);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < num_experts; e++) {
            offsets[e] = run;
            cursor[e] = run;
            run += counts[e];
        }
        offsets[num_experts] = run;
        counts[0] = run;
    }
    __syncthreads();
    const int total = counts[0];
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = topk_idx[i];
        if (e >= 0 && e < num_experts) {
            const int p = atomicAdd(&cursor[e], 1);
            sorted_token[p] = i / top_k;
            pos_of_pair[i] = p;
        } else {
            pos_of_pair[i] = -1;
        }
    }
    // positions past the last routed pair (padding rows dropped out): a valid row index, never used
    for (int i = total + threadIdx.x; i < pairs; i += blockDim.x) sorted_token[i] = 0;
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_idx, int pairs, int top_k, int num_experts, int* __restrict__ offsets,
                 int* __restrict__ sorted_token, int* __restrict__ pos_of_pair, int* status) {
    extern __shared__ int sm[];   // counts[E], cursor[E]
    pdl_sync();
    align_block(topk_idx, pairs, top_k, num_experts, sm, sm + num_experts, offsets, sorted_token, pos_of_pair, status);
}

// Few tokens (a decode step): pick, inversion and the gather of the picked tokens' activations in
// ONE block, to spare two launches.  xs[p, :] = x[sorted_token[p], :] for 16-byte units.
__global__ void __launch_bounds__(1024)
route_dispatch_kernel(const float* __restrict__ logits, const int* __restrict__ seq_of_token, int num_tokens,
                      int num_experts, int rows, int top_k, int norm_topk, float scale, int* __restrict__ topk_idx,
                      float* __restrict__ topk_w, float* __restrict__ shared_gate, int* __restrict__ offsets,
                      int* __restrict__ sorted_token, int* __restrict__ pos_of_pair, const uint4* __restrict__ x,
                      uint4* __restrict__ xs, int row_units, int* status) {
    extern __shared__ float dyn[];   // 32 warps x num_experts floats, then counts[E], cursor[E]
    pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < num_tokens; t += 32)
        route_token(logits + (size_t)t * rows, dyn + (size_t)warp * num_experts, lane,
                    seq_of_token && seq_of_token[t] < 0, num_experts, rows, top_k, norm_topk, scale,
                    topk_idx + (size_t)t * top_k, topk_w + (size_t)t * top_k, shared_gate ? shared_gate + t : nullptr);
    __syncthreads();   // the picks were written by this block: visible to it after the barrier
    int* counts = reinterpret_cast<int*>(dyn + (size_t)32 * num_experts);
    const int pairs = num_tokens * top_k;
    align_block(topk_idx, pairs, top_k, num_experts, counts, counts + num_experts, offsets, sorted_token, pos_of_pair,
                status);
    __syncthreads();
    if (x) {
        const int total = offsets[num_experts];
        for (int i = threadIdx.x; i < total * row_units; i += blockDim.x) {
            const int p = i / row_units, c = i % row_units;
            xs[(size_t)p * row_units + c] = x[(size_t)sorted_token[p] * row_units + c];
        }
    }
}

// act[m, j] = silu(gu[m, j]) * gu[m, inter + j], silu(a) = a / (1 + exp(-a))
// (reference: src/model.rs:31-33).
template <typename OT>
__global__ void swiglu_kernel(const float* __restrict__ gu, OT* __restrict__ act, long long total, int inter) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long m = i / inter;
    const int j = (int)(i % inter);
    const float a = gu[m * 2 * inter + j], b = gu[m * 2 * inter + inter + j];
    st_f(act + i, (a / (1.0f + expf(-a))) * b);
}

// One block per token: out[t] = sum_j w[t, j] * y[pos_of_pair[t k + j]] + g[t] * shared[t]
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of_pair,
                                   const float* __restrict__ topk_w, int top_k, const float* __restrict__ shared,
                                   const float* __restrict__ shared_gate, float* __restrict__ out, int hidden,
                                   int vec) {
    extern __shared__ int pick[];   // pos[top_k], then weight[top_k]
    pdl_sync();
    const int t = blockIdx.x;
    int* sp = pick;
    float* sw = reinterpret_cast<float*>(pick + top_k);
    for (int j = threadIdx.x; j < top_k; j += blockDim.x) {
        sp[j] = pos_of_pair[(size_t)t * top_k + j];
        sw[j] = topk_w[(size_t)t * top_k + j];
    }
    const float g = shared_gate ? shared_gate[t] : 1.0f;
    __syncthreads();
    const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
    if (vec) {   // four columns per thread, 16-byte accesses
#pragma unroll 2
        for (int c4 = first; c4 < hidden / 4; c4 += step) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int j = 0; j < top_k; j++) {
                const int p = sp[j];
                if (p >= 0) {
                    const float4 v = *reinterpret_cast<const float4*>(y + (size_t)p * hidden + 4 * c4);
                    const float w = sw[j];
                    acc.x = fmaf(w, v.x, acc.x), acc.y = fmaf(w, v.y, acc.y);
                    acc.z = fmaf(w, v.z, acc.z), acc.w = fmaf(w, v.w, acc.w);
                }
            }
            if (shared) {
                const float4 s = *reinterpret_cast<const float4*>(shared + (size_t)t * hidden + 4 * c4);
                if (shared_gate)
                    acc.x += g * s.x, acc.y += g * s.y, acc.z += g * s.z, acc.w += g * s.w;
                else
                    acc.x += s.x, acc.y += s.y, acc.z += s.z, acc.w += s.w;
            }
            *reinterpret_cast<float4*>(out + (size_t)t * hidden + 4 * c4) = acc;
        }
        return;
    }
    for (int c = first; c < hidden; c += step) {
        float acc = 0.f;
        for (int j = 0; j < top_k; j++) {
            const int p = sp[j];
            if (p >= 0) acc = fmaf(sw[j], y[(size_t)p * hidden + c], acc);
        }
        if (shared) {
            const float s = shared[(size_t)t * hidden + c];
            acc += shared_gate ? g * s : s;
        }
        out[(size_t)t * hidden + c] = acc;
    }
}

// Few tokens (a decode step): the norm before the feed-forward, the router and the dispatch in
// ONE launch.  A block per token adds the pending delta to the stream, normalises the row
// (as rmsnorm_kernel), forms the token's router logits from the 32-bit normalised row in shared
// memory (one warp per router row) and picks its experts; the block that finishes last inverts
// the table and gathers the picked tokens' activations (as route_dispatch_kernel).
int g_norm_route_cluster = 1;

struct NormRouteParams {
    float* x;                 // [T, hidden] stream, updated in place if delta
    const float* delta;       // pending sum or null
    const float* norm_w;
    float eps;
    int hidden, num_tokens;
    float* out32;             // normalised rows, 32-bit (or null)
    __nv_bfloat16* out16;     // normalised rows, bfloat16 (or null)
    const void* wr;           // [E, hidden]
    const void* wsg;          // [hidden] or null
    int num_experts, rows, top_k, norm_topk;
    float scale;
    const int* seq_of_token;
    int* topk_idx;
    float* topk_w;
    float* shared_gate;
    int* offsets;
    int* sorted_token;
    int* pos_of_pair;
    uint4* xs;                // gathered bfloat16 rows or null
    int row_units;            // 16-byte units per bfloat16 row
    int* ticket;              // one int, zero before and after
    int* status;
    int vec_ok;
    int cluster;              // 1: the tokens' blocks are one cluster (at most 8 tokens), see the kernel
};

template <typename WT>
__global__ void __launch_bounds__(1024) norm_route_kernel(const NormRouteParams p) {
    extern __shared__ __align__(16) float nr_smem[];
    __shared__ float red[32];
    __shared__ int s_last;
    __shared__ int s_mine[64];                         // this token's picks, for the other blocks of a cluster
    const int t = blockIdx.x + blockIdx.z, H = p.hidden, E = p.num_experts;      // (a cluster lies along z)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    {
        // the weights do not depend on the predecessor: they are asked into L2 before the wait
        // (the blocks share the router's lines among them)
        const size_t line = 128, w_bytes = (size_t)E * H * sizeof(WT);
        for (size_t off = ((size_t)t * blockDim.x + threadIdx.x) * line; off < w_bytes;
             off += (size_t)p.num_tokens * blockDim.x * line)
            prefetch_l2((const char*)p.wr + off);
        for (size_t off = threadIdx.x * line; off < (size_t)H * sizeof(float); off += blockDim.x * line)
            prefetch_l2((const char*)p.norm_w + off);
        if (p.wsg)
            for (size_t off = threadIdx.x * line; off < (size_t)H * sizeof(WT); off += blockDim.x * line)
                prefetch_l2((const char*)p.wsg + off);
    }
    pdl_sync();
    float* row = nr_smem;                              // [H] (H rounded up to 4)
    float* logit = row + ((H + 3) & ~3);               // [rows]
    float* sc = logit + p.rows;                        // [E]
    float* wk = sc + E;                                // [top_k]
    int* picks = reinterpret_cast<int*>(wk + p.top_k); // [pairs]
    const int pairs = p.num_tokens * p.top_k;
    int* sorted = picks + pairs;                       // [pairs]
    int* counts = sorted + pairs;                      // [E], then cursor [E]

    // ---- the norm --------------------------------------------------------------------------
    float* xr = p.x + (size_t)t * H;
    const float* dr = p.delta ? p.delta + (size_t)t * H : nullptr;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = xr[j];
        if (dr) {
            v += dr[j];
            xr[j] = v;
        }
        row[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)H + p.eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float y = row[j] * rs * p.norm_w[j];
        row[j] = y;
        if (p.out32) p.out32[(size_t)t * H + j] = y;
        if (p.out16) p.out16[(size_t)t * H + j] = __float2bfloat16_rn(y);
    }
    __syncthreads();

    // ---- router logits: one warp per router row, 32-bit products and sums in a fixed order ----
    // (a warp takes two rows at a time, so that the loads of both are in flight together)
    const int groups = p.vec_ok ? H / 8 : 0;
    for (int r = warp; r < p.rows; r += 2 * nwarps) {
        const int r2 = r + nwarps;
        const bool two = r2 < p.rows;
        const WT* w = r < E ? (const WT*)p.wr + (size_t)r * H : (const WT*)p.wsg;
        const WT* w2 = !two ? w : (r2 < E ? (const WT*)p.wr + (size_t)r2 * H : (const WT*)p.wsg);
        float acc = 0.f, acc2 = 0.f;
#pragma unroll 4
        for (int gi = lane; gi < groups; gi += 32) {
            float wv[8], wv2[8];
            w_load8<WT>(w + gi * 8, wv);
            w_load8<WT>(w2 + gi * 8, wv2);
            const float4 a = *reinterpret_cast<const float4*>(row + gi * 8);
            const float4 b = *reinterpret_cast<const float4*>(row + gi * 8 + 4);
            acc = fmaf(a.x, wv[0], acc), acc = fmaf(a.y, wv[1], acc), acc = fmaf(a.z, wv[2], acc);
            acc = fmaf(a.w, wv[3], acc), acc = fmaf(b.x, wv[4], acc), acc = fmaf(b.y, wv[5], acc);
            acc = fmaf(b.z, wv[6], acc), acc = fmaf(b.w, wv[7], acc);
            acc2 = fmaf(a.x, wv2[0], acc2), acc2 = fmaf(a.y, wv2[1], acc2), acc2 = fmaf(a.z, wv2[2], acc2);
            acc2 = fmaf(a.w, wv2[3], acc2), acc2 = fmaf(b.x, wv2[4], acc2), acc2 = fmaf(b.y, wv2[5], acc2);
            acc2 = fmaf(b.z, wv2[6], acc2), acc2 = fmaf(b.w, wv2[7], acc2);
        }
        for (int c = groups * 8 + lane; c < H; c += 32) {
            acc = fmaf(row[c], ld_f(w + c), acc);
            acc2 = fmaf(row[c], ld_f(w2 + c), acc2);
        }
        acc = warp_sum(acc);
        acc2 = warp_sum(acc2);
        if (lane == 0) {
            logit[r] = acc;
            if (two) logit[r2] = acc2;
        }
    }
    __syncthreads();

    // ---- this token's experts ------------------------------------------------------------------
    if (warp == 0)
        route_token(logit, sc, lane, p.seq_of_token && p.seq_of_token[t] < 0, E, p.rows, p.top_k, p.norm_topk, p.scale,
                    p.topk_idx + (size_t)t * p.top_k, p.topk_w + (size_t)t * p.top_k,
                    p.shared_gate ? p.shared_gate + t : nullptr, wk);

    if (p.cluster) {
        // ---- one cluster: every block learns all picks through distributed shared memory, inverts
        // the table for itself (in pair order, so the result does not depend on timing) and writes
        // the gathered rows of ITS token from the row it still holds; block 0 writes the tables
        __syncthreads();
        for (int j = threadIdx.x; j < p.top_k; j += blockDim.x) s_mine[j] = p.topk_idx[(size_t)t * p.top_k + j];
        cl_sync();
        for (int i = threadIdx.x; i < pairs; i += blockDim.x)
            picks[i] = (int)cl_peer_u32(&s_mine[i % p.top_k], (unsigned)(i / p.top_k));
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            int c = 0;
            for (int i = 0; i < pairs; i++) c += picks[i] == e;
            counts[e] = c;
        }
        for (int i = threadIdx.x; i < pairs; i += blockDim.x)
            if (picks[i] != -1 && (picks[i] < 0 || picks[i] >= E)) atomicOr(p.status, ST_BAD_EXPERT);
        __syncthreads();
        int* start = counts + E;
        if (warp == 0) {   // exclusive scan of the counts, 32 experts at a time
            int run = 0;
            for (int e0 = 0; e0 < E; e0 += 32) {
                const int e = e0 + lane;
                const int c = e < E ? counts[e] : 0;
                int inc = c;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int n = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += n;
                }
                if (e < E) {
                    start[e] = run + inc - c;
                    if (t == 0) p.offsets[e] = run + inc - c;
                }
                run += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (lane == 0) {
                if (t == 0) p.offsets[E] = run;
                s_last = run;
            }
        }
        __syncthreads();
        const int total = s_last;
        for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
            const int e = picks[i];
            int q = -1;
            if (e >= 0 && e < E) {
                q = start[e];
                for (int j = 0; j < i; j++) q += picks[j] == e;      // pairs of the same expert before this one
                if (t == 0) p.sorted_token[q] = i / p.top_k;
            }
            sorted[i] = q;                                          // here: the place of pair i
            if (t == 0) p.pos_of_pair[i] = q;
        }
        if (t == 0)
            for (int i = total + threadIdx.x; i < pairs; i += blockDim.x) p.sorted_token[i] = 0;
        __syncthreads();
        if (p.xs) {
            for (int j = 0; j < p.top_k; j++) {
                const int q = sorted[t * p.top_k + j];
                if (q < 0) continue;
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.xs) + (size_t)q * H;
                for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2)
                    *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(row[c], row[c + 1]);
            }
        }
        cl_sync();      // no block leaves while another may still read its picks
        return;
    }

    // ---- the block that finishes last inverts the table and gathers ----------------------------
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int last = atomicAdd(p.ticket, 1) == p.num_tokens - 1;
        if (last) *p.ticket = 0;
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    int* cursor = counts + E;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) picks[i] = __ldcg(p.topk_idx + i);
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = picks[i];
        if (e >= 0 && e < E)
            atomicAdd(&counts[e], 1);
        else if (e != -1)
            atomicOr(p.status, ST_BAD_EXPERT);
    }
    __syncthreads();
    if (warp == 0) {   // exclusive scan of the counts, 32 experts at a time
        int run = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < E ? counts[e] : 0;
            int inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += n;
            }
            if (e < E) {
                p.offsets[e] = run + inc - c;
                cursor[e] = run + inc - c;
            }
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) {
            p.offsets[E] = run;
            s_last = run;          // total, for the whole block
        }
    }
    __syncthreads();
    const int total = s_last;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = picks[i];
        if (e >= 0 && e < E) {
            const int q = atomicAdd(&cursor[e], 1);
            sorted[q] = i / p.top_k;
            p.sorted_token[q] = i / p.top_k;
            p.pos_of_pair[i] = q;
        } else {
            p.pos_of_pair[i] = -1;
        }
    }
    for (int i = total + threadIdx.x; i < pairs; i += blockDim.x) p.sorted_token[i] = 0;
    __syncthreads();
    if (p.xs) {
        const uint4* src = reinterpret_cast<const uint4*>(p.out16);
        const int n = total * p.row_units;
#pragma unroll 8
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int q = i / p.row_units, c = i % p.row_units;
            p.xs[i] = __ldcg(src + (size_t)sorted[q] * p.row_units + c);
        }
    }
}

}  // namespace

// The cluster form of norm_route_kernel (up to 8 tokens) on or off (on by default).
MOE_API void moe_set_norm_route_cluster(int enabled) { g_norm_route_cluster = enabled ? 1 : 0; }

// The norm before a routed feed-forward, the router and the dispatch of a step of few tokens, one
// launch (see norm_route_kernel).  Returns -1, with nothing launched, for sizes it does not take
// (more than 64 tokens, 256 experts or 4096 (token, expert) pairs, or a row too long for shared
// memory): the caller then runs the separate kernels.
MOE_API int moe_norm_route(float* x, const float* delta, const float* norm_w, float eps, int hidden, int num_tokens,
                           float* out32, void* out16, const void* wr, const void* wsg, int w_dt, int num_experts,
                           int top_k, int norm_topk, float scale, const int* seq_of_token, int* topk_idx,
                           float* topk_w, float* shared_gate, int* offsets, int* sorted_token, int* pos_of_pair,
                           void* xs, int* ticket, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (top_k <= 0 || top_k > num_experts || hidden <= 0 || !ticket || (wsg && !shared_gate) || (xs && !out16))
        return (int)cudaErrorInvalidValue;
    const int pairs = num_tokens * top_k;
    if (num_tokens > 64 || num_experts > 256 || pairs > 4096) return -1;
    NormRouteParams p;
    p.x = x, p.delta = delta, p.norm_w = norm_w, p.eps = eps, p.hidden = hidden, p.num_tokens = num_tokens;
    p.out32 = out32, p.out16 = (__nv_bfloat16*)out16, p.wr = wr, p.wsg = wsg, p.num_experts = num_experts;
    p.rows = num_experts + (wsg ? 1 : 0), p.top_k = top_k, p.norm_topk = norm_topk, p.scale = scale;
    p.seq_of_token = seq_of_token, p.topk_idx = topk_idx, p.topk_w = topk_w, p.shared_gate = shared_gate;
    p.offsets = offsets, p.sorted_token = sorted_token, p.pos_of_pair = pos_of_pair;
    p.xs = (uint4*)xs, p.row_units = hidden * 2 / 16, p.ticket = ticket, p.status = status;
    if (xs && ((hidden * 2) % 16 || (uintptr_t)xs % 16 || (uintptr_t)out16 % 16)) return -1;
    const size_t elt = w_dt == DT_F32 ? 4 : 2;
    p.vec_ok = (hidden % 8 == 0) && ((uintptr_t)wr % 16 == 0) && (!wsg || (uintptr_t)wsg % 16 == 0) &&
               ((hidden * elt) % 16 == 0);
    const size_t smem = ((size_t)((hidden + 3) & ~3) + p.rows + num_experts + top_k) * sizeof(float) +
                        ((size_t)2 * pairs + 2 * num_experts) * sizeof(int);
    if (smem > 200 * 1024) return -1;
    auto kernel = w_dt == DT_F32 ? norm_route_kernel<float> : norm_route_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // up to 8 tokens: one cluster, no ticket, no second reading of what other blocks wrote
    p.cluster = (num_tokens <= 8 && top_k <= 64 && hidden % 2 == 0 && g_norm_route_cluster) ? 1 : 0;
    if (p.cluster) return launch_pdl_cluster(kernel, dim3(1, 1, num_tokens), 1024, smem, stream, num_tokens, p);
    return launch_pdl(kernel, num_tokens, 1024, smem, stream, p);
}

// Slices of the hidden dimension the register-tiled kernel would use for this size (0: the size
// goes to another kernel); it then wants slices * num_tokens * rows floats of scratch.
static int router_slices(int num_tokens, int hidden, int rows, int* kper) {
    if (num_tokens <= 256 || hidden % 8) return 0;
    const long long blocks = (long long)((num_tokens + ST - 1) / ST) * ((rows + SR - 1) / SR);
    int want = (int)((2 * 148 + blocks - 1) / blocks);
    if (want < 1) want = 1;
    if (want > hidden / 64) want = hidden / 64 > 0 ? hidden / 64 : 1;
    int per = (hidden + want - 1) / want;
    per = (per + SK - 1) / SK * SK;
    *kper = per;
    return (hidden + per - 1) / per;
}

MOE_API long long moe_router_scratch_floats(int num_tokens, int hidden, int num_experts, int has_gate_row) {
    int kper = 0;
    const int rows = num_experts + (has_gate_row ? 1 : 0);
    return (long long)router_slices(num_tokens, hidden, rows, &kper) * num_tokens * rows;
}

// logits[t, r] = h[t] . W[r] for the router rows (and the shared-gate row, if wsg): num_tokens *
// (num_experts + (wsg ? 1 : 0)) floats.  scratch: moe_router_scratch_floats floats (may be null:
// a prompt then takes the slower kernel).
// *left_in_slices (if given): the sgemm kernel's partial sums are left in scratch, to be added by the
// caller's next kernel; set to the number of slices, or to 0 if the logits are complete.
static int router_logits_impl(const float* h, const void* wr, const void* wsg, int w_dt, int num_tokens, int hidden,
                              int num_experts, float* logits, float* scratch, long long scratch_floats,
                              int* left_in_slices, cudaStream_t stream) {
    if (left_in_slices) *left_in_slices = 0;
    if (num_tokens <= 0) return 0;
    if (num_experts <= 0 || !logits) return (int)cudaErrorInvalidValue;
    const int rows = num_experts + (wsg ? 1 : 0);
    const size_t elt = w_dt == DT_F32 ? 4 : 2;
    const int vec_ok = (hidden % 8 == 0) && ((uintptr_t)h % 16 == 0) && ((uintptr_t)wr % 16 == 0) &&
                       (!wsg || (uintptr_t)wsg % 16 == 0) && ((hidden * elt) % 16 == 0);
    const int ty = (num_tokens + TOK_TILE - 1) / TOK_TILE;
    if (ty > 65535) return (int)cudaErrorInvalidValue;
#define LOGITS(WT, ROWS, KSPLIT)                                                                          \
    launch_pdl(router_logits_kernel<WT, ROWS, KSPLIT>, dim3((rows + ROWS - 1) / ROWS, ty), ROWS * KSPLIT * 32, 0,   \
               stream, h, (const WT*)wr, (const WT*)wsg, num_tokens, hidden, num_experts, rows, vec_ok, logits)
    int kper = 0;
    const int slices = vec_ok ? router_slices(num_tokens, hidden, rows, &kper) : 0;
    if (slices > 0 && scratch && scratch_floats >= (long long)slices * num_tokens * rows &&
        (num_tokens + ST - 1) / ST <= 0x7fffffff && slices <= 65535 && (rows + SR - 1) / SR <= 65535) {
        const dim3 g((num_tokens + ST - 1) / ST, slices, (rows + SR - 1) / SR);
        int e;
        if (w_dt == DT_F32)
            e = launch_pdl(router_logits_sgemm_kernel<float>, g, 128, 0, stream, h, (const float*)wr, (const float*)wsg,
                           num_tokens, hidden, num_experts, rows, kper, scratch);
        else
            e = launch_pdl(router_logits_sgemm_kernel<__nv_bfloat16>, g, 128, 0, stream, h, (const __nv_bfloat16*)wr,
                           (const __nv_bfloat16*)wsg, num_tokens, hidden, num_experts, rows, kper, scratch);
        if (e) return e;
        if (left_in_slices) {
            *left_in_slices = slices;
            return 0;
        }
        const size_t n = (size_t)num_tokens * rows;
        sum_slices_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(scratch, logits, n, slices);
    } else if (num_tokens <= 64) {
        if (w_dt == DT_F32) LOGITS(float, 2, 4); else LOGITS(__nv_bfloat16, 2, 4);
    } else if (vec_ok && (num_tokens + PT - 1) / PT <= 65535) {
        const dim3 tg((rows + 7) / 8, (num_tokens + PT - 1) / PT);
        if (w_dt == DT_F32)
            router_logits_tiled_kernel<float><<<tg, 256, 0, stream>>>(h, (const float*)wr, (const float*)wsg,
                                                                      num_tokens, hidden, num_experts, rows, logits);
        else
            router_logits_tiled_kernel<__nv_bfloat16><<<tg, 256, 0, stream>>>(
                h, (const __nv_bfloat16*)wr, (const __nv_bfloat16*)wsg, num_tokens, hidden, num_experts, rows, logits);
    } else {
        if (w_dt == DT_F32) LOGITS(float, 8, 1); else LOGITS(__nv_bfloat16, 8, 1);
    }
#undef LOGITS
    return launch_status();
}

MOE_API int moe_router_logits(const float* h, const void* wr, const void* wsg, int w_dt, int num_tokens, int hidden,
                              int num_experts, float* logits, float* scratch, long long scratch_floats,
                              cudaStream_t stream) {
    return router_logits_impl(h, wr, wsg, w_dt, num_tokens, hidden, num_experts, logits, scratch, scratch_floats,
                              nullptr, stream);
}

// logits: scratch of num_tokens * (num_experts + (wsg ? 1 : 0)) floats.
MOE_API int moe_router(const float* h, const void* wr, const void* wsg, int w_dt, const int* seq_of_token,
                       int num_tokens, int hidden, int num_experts, int top_k, int norm_topk, float scale,
                       float* logits, int* topk_idx, float* topk_w, float* shared_gate, float* scratch,
                       long long scratch_floats, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (top_k <= 0 || top_k > num_experts || num_experts > 2048 || !logits) return (int)cudaErrorInvalidValue;
    if (wsg && !shared_gate) return (int)cudaErrorInvalidValue;
    int slices = 0;
    const int rc = router_logits_impl(h, wr, wsg, w_dt, num_tokens, hidden, num_experts, logits, scratch,
                                      scratch_floats, &slices, stream);
    if (rc) return rc;
    const int rows = num_experts + (wsg ? 1 : 0);
    const size_t smem = (size_t)4 * (rows + num_experts + top_k) * sizeof(float);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(router_topk_kernel, (num_tokens + 3) / 4, 128, smem, stream, logits,
                      (const float*)(slices ? scratch : nullptr), slices, seq_of_token, num_tokens, num_experts, rows,
                      top_k, norm_topk, scale, topk_idx, topk_w, shared_gate);
}

// Picks, weights and shared gate from logits that are already there ([T, rows] float32).
MOE_API int moe_router_topk(float* logits, const int* seq_of_token, int num_tokens, int num_experts, int has_gate_row,
                            int top_k, int norm_topk, float scale, int* topk_idx, float* topk_w, float* shared_gate,
                            cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (top_k <= 0 || top_k > num_experts || num_experts > 2048 || !logits || (has_gate_row && !shared_gate))
        return (int)cudaErrorInvalidValue;
    const int rows = num_experts + (has_gate_row ? 1 : 0);
    const size_t smem = (size_t)4 * (rows + num_experts + top_k) * sizeof(float);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(router_topk_kernel, (num_tokens + 3) / 4, 128, smem, stream, logits, (const float*)nullptr, 0,
                      seq_of_token, num_tokens, num_experts, rows, top_k, norm_topk, scale, topk_idx, topk_w, shared_gate);
}

// A float32 row as three bfloat16 terms, x = p0 + p1 + p2 exactly (8 + 8 + 8 bits of mantissa):
// out[t] = [p0 (hidden) | p1 (hidden) | p2 (hidden)].  A product of these with bfloat16 weights on
// the tensor cores, accumulated in float32, is a float32-accurate product of x: every partial
// product is exact.  (The router's logits for a prompt.)  hidden a multiple of 4.
__global__ void split3_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n4, int hidden) {
    pdl_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const long long t = (i * 4) / hidden;
    const int c = (int)((i * 4) % hidden);
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const float in[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat16 p[3][4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        float r = in[e];
#pragma unroll
        for (int k = 0; k < 3; k++) {
            p[k][e] = __float2bfloat16_rn(r);
            r -= __bfloat162float(p[k][e]);          // exact: the difference fits in float32
        }
    }
    __nv_bfloat16* o = out + t * 3 * hidden + c;
#pragma unroll
    for (int k = 0; k < 3; k++) *reinterpret_cast<uint2*>(o + (size_t)k * hidden) = *reinterpret_cast<const uint2*>(p[k]);
}
MOE_API int moe_split3(const float* x, void* out, long long num_tokens, int hidden, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hidden <= 0 || hidden % 4 || ((uintptr_t)x & 15) || ((uintptr_t)out & 7)) return (int)cudaErrorInvalidValue;
    const long long n4 = num_tokens * hidden / 4;
    if ((n4 + 255) / 256 > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    return launch_pdl(split3_kernel, (unsigned)((n4 + 255) / 256), 256, 0, stream, x, (__nv_bfloat16*)out, n4, hidden);
}

MOE_API int moe_align(const int* topk_idx, int num_tokens, int top_k, int num_experts, int* offsets,
                      int* sorted_token, int* pos_of_pair, int* status, cudaStream_t stream) {
    if (num_experts > 4096) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)num_experts * 2 * sizeof(int);
    return launch_pdl(moe_align_kernel, 1, 1024, smem, stream, topk_idx, num_tokens * top_k, top_k, num_experts,
                      offsets, sorted_token, pos_of_pair, status);
}

// logits -> picks, weights, shared gate, inverted table and (optionally) gathered activations, one
// launch.  For at most 64 tokens and 256 experts.  x / xs: rows of row_bytes bytes (a multiple of 16).
MOE_API int moe_route_dispatch(const float* logits, const int* seq_of_token, int num_tokens, int num_experts,
                               int has_gate_row, int top_k, int norm_topk, float scale, int* topk_idx, float* topk_w,
                               float* shared_gate, int* offsets, int* sorted_token, int* pos_of_pair, const void* x,
                               void* xs, int row_bytes, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (num_tokens > 64 || num_experts > 256 || top_k <= 0 || top_k > num_experts || row_bytes % 16)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)32 * num_experts * sizeof(float) + (size_t)2 * num_experts * sizeof(int);
    return launch_pdl(route_dispatch_kernel, 1, 1024, smem, stream, logits, seq_of_token, num_tokens, num_experts,
                      num_experts + (has_gate_row ? 1 : 0), top_k, norm_topk, scale, topk_idx, topk_w, shared_gate,
                      offsets, sorted_token, pos_of_pair, (const uint4*)x, (uint4*)xs, row_bytes / 16, status);
}

MOE_API int moe_swiglu(const float* gu, void* act, int out_dt, long long rows, int inter, cudaStream_t stream) {
    const long long total = rows * inter;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dt == DT_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>(gu, (float*)act, total, inter);
    else
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(gu, (__nv_bfloat16*)act, total, inter);
    return launch_status();
}

MOE_API int moe_combine(const float* y, const int* pos_of_pair, const float* topk_w, int top_k, const float* shared,
                        const float* shared_gate, float* out, int num_tokens, int hidden, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (top_k < 0 || top_k > 4096) return (int)cudaErrorInvalidValue;
    const int vec = hidden % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                    (!shared || (uintptr_t)shared % 16 == 0);
    const int units = vec ? hidden / 4 : hidden;
    // few tokens: several small blocks a token, for parallelism; many: one block a token, whose
    // threads each keep the loads of two columns in flight
    const int threads = num_tokens >= 512 ? 256 : 128;
    const int by = num_tokens >= 512 ? 1 : max(1, min(64, (units + 127) / 128));
    return launch_pdl(moe_combine_kernel, dim3(num_tokens, by), threads, (size_t)top_k * 8, stream, y, pos_of_pair,
                      topk_w, top_k, shared, shared_gate, out, hidden, vec);
}
