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

template <typename WT>
__device__ __forceinline__ float row_dot(const float* __restrict__ x, const WT* __restrict__ w, int n, int lane) {
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s = fmaf(x[i], ld_f(w + i), s);
    return warp_sum(s);
}

// One block (4 warps) per token.
template <typename WT>
__global__ void __launch_bounds__(128)
router_kernel(const float* __restrict__ h, const WT* __restrict__ wr, const WT* __restrict__ wsg,
              const int* __restrict__ seq_of_token, int hidden, int num_experts, int top_k, int norm_topk,
              float scale, int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ shared_gate) {
    extern __shared__ float sc[];   // num_experts scores
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (seq_of_token && seq_of_token[t] < 0) {   // padding row: no expert
        for (int j = threadIdx.x; j < top_k; j += blockDim.x) {
            topk_idx[(size_t)t * top_k + j] = -1;
            topk_w[(size_t)t * top_k + j] = 0.f;
        }
        if (shared_gate && threadIdx.x == 0) shared_gate[t] = 0.f;
        return;
    }
    const float* x = h + (size_t)t * hidden;
    for (int e = warp; e < num_experts + (wsg ? 1 : 0); e += 4) {
        if (e < num_experts) {
            const float d = row_dot(x, wr + (size_t)e * hidden, hidden, lane);
            if (lane == 0) sc[e] = d;
        } else {
            const float d = row_dot(x, wsg, hidden, lane);
            if (lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-d));
        }
    }
    __syncthreads();
    if (warp != 0) return;
    // softmax over all experts
    float m = -INFINITY;
    for (int e = lane; e < num_experts; e += 32) m = fmaxf(m, sc[e]);
    m = warp_max(m);
    float z = 0.f;
    for (int e = lane; e < num_experts; e += 32) {
        const float v = expf(sc[e] - m);
        sc[e] = v;
        z += v;
    }
    z = warp_sum(z);
    for (int e = lane; e < num_experts; e += 32) sc[e] = sc[e] / z;
    __syncwarp();
    // top-k by repeated argmax; a tie goes to the lower index
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
            topk_idx[(size_t)t * top_k + j] = bi;
            topk_w[(size_t)t * top_k + j] = w;
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float zz = norm_topk ? fmaxf(wsum, 1e-20f) : 1.0f;
        for (int j = 0; j < top_k; j++) {
            float w = topk_w[(size_t)t * top_k + j];
            if (norm_topk) w = w / zz;
            topk_w[(size_t)t * top_k + j] = w * scale;
        }
    }
}

// Single block.  pairs = tokens * top_k entries of topk_idx (expert id, or -1).
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_idx, int pairs, int top_k, int num_experts, int* __restrict__ offsets,
                 int* __restrict__ sorted_token, int* __restrict__ pos_of_pair, int* status) {
    extern __shared__ int sm[];   // counts[E], cursor[E]
    int* counts = sm;
    int* cursor = sm + num_experts;
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
    }
    __syncthreads();
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
    for (int i = offsets[num_experts] + threadIdx.x; i < pairs; i += blockDim.x) sorted_token[i] = 0;
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
                                   const float* __restrict__ shared_gate, float* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top_k; j++) {
            const int p = pos_of_pair[(size_t)t * top_k + j];
            if (p >= 0) acc = fmaf(topk_w[(size_t)t * top_k + j], y[(size_t)p * hidden + c], acc);
        }
        if (shared) {
            const float s = shared[(size_t)t * hidden + c];
            acc += shared_gate ? shared_gate[t] * s : s;
        }
        out[(size_t)t * hidden + c] = acc;
    }
}

}  // namespace

MOE_API int moe_router(const float* h, const void* wr, const void* wsg, int w_dt, const int* seq_of_token,
                       int num_tokens, int hidden, int num_experts, int top_k, int norm_topk, float scale,
                       int* topk_idx, float* topk_w, float* shared_gate, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (top_k <= 0 || top_k > num_experts || num_experts > 8192) return (int)cudaErrorInvalidValue;
    if (wsg && !shared_gate) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)num_experts * sizeof(float);
    if (w_dt == DT_F32)
        router_kernel<float><<<num_tokens, 128, smem, stream>>>(h, (const float*)wr, (const float*)wsg, seq_of_token,
                                                               hidden, num_experts, top_k, norm_topk, scale, topk_idx,
                                                               topk_w, shared_gate);
    else
        router_kernel<__nv_bfloat16><<<num_tokens, 128, smem, stream>>>(
            h, (const __nv_bfloat16*)wr, (const __nv_bfloat16*)wsg, seq_of_token, hidden, num_experts, top_k,
            norm_topk, scale, topk_idx, topk_w, shared_gate);
    return launch_status();
}

MOE_API int moe_align(const int* topk_idx, int num_tokens, int top_k, int num_experts, int* offsets,
                      int* sorted_token, int* pos_of_pair, int* status, cudaStream_t stream) {
    if (num_experts > 4096) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)num_experts * 2 * sizeof(int);
    moe_align_kernel<<<1, 1024, smem, stream>>>(topk_idx, num_tokens * top_k, top_k, num_experts, offsets,
                                               sorted_token, pos_of_pair, status);
    return launch_status();
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
    moe_combine_kernel<<<num_tokens, 256, 0, stream>>>(y, pos_of_pair, topk_w, top_k, shared, shared_gate, out,
                                                      hidden);
    return launch_status();
}
