// Token embedding gather and RMSNorm (with the residual add fused in front of it).
//
// RMSNorm: s = 1/sqrt(mean(x^2) + eps); out = x * s * w, the weight multiplying
// directly and eps inside the square root (reference: src/model.rs:211-216).
// Statistics, the residual sum and the product are 32-bit; only the optional
// second output is rounded to bfloat16 for the matrix products that follow.
#include "common.cuh"

// x[t, :] = table[token[t], :]; a token id outside [0, vocab) sets ST_BAD_TOKEN
// and reads row 0 (the reference wraps modulo the vocabulary, src/model.rs:664).
// A token id of -1 stands for "the token sampled last for this row's sequence": it is read from
// last_token[slot of the sequence] (written by the sampling kernel), so a decode step can be
// launched before the host knows the previous step's tokens.
template <typename WT>
__global__ void embed_kernel(const WT* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x,
                             int hidden, int vocab, int* status, const int* __restrict__ last_token,
                             const int* __restrict__ seq_of_token, const int* __restrict__ slots) {
    pdl_sync();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok == -1 && last_token) {
        const int s = seq_of_token[t];
        tok = s >= 0 ? last_token[slots[s]] : 0;      // a padding row: any valid row
    }
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, ST_BAD_TOKEN);
        tok = 0;
    }
    const WT* row = table + (size_t)tok * hidden;
    float* out = x + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = ld_f(row + i);
}

MOE_API int moe_embed(const void* table, int table_dt, const int* tokens, float* x, int num_tokens, int hidden,
                      int vocab, int* status, const int* last_token, const int* seq_of_token, const int* slots,
                      cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (last_token && (!seq_of_token || !slots)) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dt == DT_F32)
        return launch_pdl(embed_kernel<float>, num_tokens, threads, 0, stream, (const float*)table, tokens, x, hidden,
                          vocab, status, last_token, seq_of_token, slots);
    return launch_pdl(embed_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (const __nv_bfloat16*)table, tokens,
                      x, hidden, vocab, status, last_token, seq_of_token, slots);
}

// A delta that is still the output of routed experts, not yet combined: for token t,
//   delta[t] = sum_j w[t, j] * y[pos[t, j]] + gate[t] * shared[t]
// with the arithmetic (and its order) of moe_combine_kernel in moe.cu.  The norm that follows the
// feed-forward forms it on the fly, which spares one pass over the stream.
struct CombineSrc {
    const float* y;        // null: no such delta
    const int* pos;        // [T, top_k], -1: no expert
    const float* w;        // [T, top_k]
    int top_k;
    const float* shared;   // [T, hidden] or null
    const float* gate;     // [T] or null
};

// One block per output row i.  Source row r = rows ? rows[i] : i.
//   v = x[r] (+ delta[r]);  if write_back: x[r] = v
//   y = v * rsqrt(mean(v^2) + eps) * w;  out32[i] = y;  out16[i] = bf16(y)
// The row is held in shared memory so that x is read once.
// MINB: blocks of 512 threads that must fit an SM.  4 for many rows (a prompt: the kernel is bound by
// how many loads are in flight, and 32 registers a thread cost a few spills that do not matter there:
// 26.7 -> 20.5 us for 2,048 rows of 2,048), 1 for few rows (a decode step: every instruction counts).
template <int MINB>
__global__ void __launch_bounds__(512, MINB) rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ w,
                               const int* __restrict__ rows, float* __restrict__ out32,
                               __nv_bfloat16* __restrict__ out16, int hidden, float eps, int write_back,
                               int num_src_rows, int* status, int vec, const CombineSrc cs) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int i = blockIdx.x;
    // The experts' combine with one 16-byte unit a thread: what does not come from the predecessor
    // (the stream, the picks' places and weights, the gate and the norm's weight were all written
    // at least two kernels ago) is read before the wait, so that only the experts' rows are left.
    if (cs.y && !rows && hidden / 4 <= (int)blockDim.x && cs.top_k <= 8) {
        const int j = threadIdx.x;
        const bool mine = j < hidden / 4;
        int pq[8];
        float wq[8];
#pragma unroll
        for (int q = 0; q < 8; q++) {
            pq[q] = q < cs.top_k ? cs.pos[(size_t)i * cs.top_k + q] : -1;
            wq[q] = q < cs.top_k ? cs.w[(size_t)i * cs.top_k + q] : 0.f;
        }
        const float g = cs.gate ? cs.gate[i] : 1.0f;
        float* xr = x + (size_t)i * hidden;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f), nw = v;
        if (mine) v = reinterpret_cast<const float4*>(xr)[j], nw = reinterpret_cast<const float4*>(w)[j];
        pdl_sync();
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mine) {
#pragma unroll
            for (int q = 0; q < 8; q++)
                if (pq[q] >= 0) {
                    const float4 yv = *reinterpret_cast<const float4*>(cs.y + (size_t)pq[q] * hidden + 4 * j);
                    acc.x = fmaf(wq[q], yv.x, acc.x), acc.y = fmaf(wq[q], yv.y, acc.y);
                    acc.z = fmaf(wq[q], yv.z, acc.z), acc.w = fmaf(wq[q], yv.w, acc.w);
                }
            if (cs.shared) {
                const float4 sv = *reinterpret_cast<const float4*>(cs.shared + (size_t)i * hidden + 4 * j);
                if (cs.gate)
                    acc.x += g * sv.x, acc.y += g * sv.y, acc.z += g * sv.z, acc.w += g * sv.w;
                else
                    acc.x += sv.x, acc.y += sv.y, acc.z += sv.z, acc.w += sv.w;
            }
            v.x += acc.x, v.y += acc.y, v.z += acc.z, v.w += acc.w;
            if (write_back) reinterpret_cast<float4*>(xr)[j] = v;
        }
        const float ss1 = block_sum(mine ? v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w : 0.f, red);
        const float scale = 1.0f / sqrtf(ss1 / (float)hidden + eps);
        if (mine) {
            const float4 y = make_float4(v.x * scale * nw.x, v.y * scale * nw.y, v.z * scale * nw.z, v.w * scale * nw.w);
            if (out32) reinterpret_cast<float4*>(out32 + (size_t)i * hidden)[j] = y;
            if (out16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
                reinterpret_cast<uint2*>(out16 + (size_t)i * hidden)[j] = u;
            }
        }
        return;
    }
    pdl_sync();
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= num_src_rows) {
        if (threadIdx.x == 0) atomicOr(status, ST_BAD_ROW);
        r = 0;
    }
    float* xr = x + (size_t)r * hidden;
    const float* dr = delta ? delta + (size_t)r * hidden : nullptr;
    float ss = 0.f;
    if (cs.y) {   // (vec is set: the host refuses this form otherwise)
        const float g = cs.gate ? cs.gate[r] : 1.0f;
        for (int j = threadIdx.x; j < hidden / 4; j += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int q = 0; q < cs.top_k; q++) {
                const int p = cs.pos[(size_t)r * cs.top_k + q];
                if (p >= 0) {
                    const float4 yv = *reinterpret_cast<const float4*>(cs.y + (size_t)p * hidden + 4 * j);
                    const float wq = cs.w[(size_t)r * cs.top_k + q];
                    acc.x = fmaf(wq, yv.x, acc.x), acc.y = fmaf(wq, yv.y, acc.y);
                    acc.z = fmaf(wq, yv.z, acc.z), acc.w = fmaf(wq, yv.w, acc.w);
                }
            }
            if (cs.shared) {
                const float4 sv = *reinterpret_cast<const float4*>(cs.shared + (size_t)r * hidden + 4 * j);
                if (cs.gate)
                    acc.x += g * sv.x, acc.y += g * sv.y, acc.z += g * sv.z, acc.w += g * sv.w;
                else
                    acc.x += sv.x, acc.y += sv.y, acc.z += sv.z, acc.w += sv.w;
            }
            float4 v = reinterpret_cast<const float4*>(xr)[j];
            v.x += acc.x, v.y += acc.y, v.z += acc.z, v.w += acc.w;
            if (write_back) reinterpret_cast<float4*>(xr)[j] = v;
            reinterpret_cast<float4*>(row)[j] = v;
            ss += v.x * v.x, ss += v.y * v.y, ss += v.z * v.z, ss += v.w * v.w;
        }
    } else if (vec) {   // rows of whole 16-byte units: four elements per access
        for (int j = threadIdx.x; j < hidden / 4; j += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(xr)[j];
            if (dr) {
                const float4 d = reinterpret_cast<const float4*>(dr)[j];
                v.x += d.x, v.y += d.y, v.z += d.z, v.w += d.w;
                if (write_back) reinterpret_cast<float4*>(xr)[j] = v;
            }
            reinterpret_cast<float4*>(row)[j] = v;
            ss += v.x * v.x, ss += v.y * v.y, ss += v.z * v.z, ss += v.w * v.w;
        }
    }
    if (vec) {
        ss = block_sum(ss, red);
        const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int j = threadIdx.x; j < hidden / 4; j += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(row)[j], g = reinterpret_cast<const float4*>(w)[j];
            const float4 y = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
            if (out32) reinterpret_cast<float4*>(out32 + (size_t)i * hidden)[j] = y;
            if (out16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
                reinterpret_cast<uint2*>(out16 + (size_t)i * hidden)[j] = u;
            }
        }
        return;
    }
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = xr[j];
        if (dr) {
            v += dr[j];
            if (write_back) xr[j] = v;
        }
        row[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float y = row[j] * scale * w[j];
        if (out32) out32[(size_t)i * hidden + j] = y;
        if (out16) out16[(size_t)i * hidden + j] = __float2bfloat16_rn(y);
    }
}

static int rmsnorm_launch(float* x, const float* delta, const float* w, const int* rows, float* out32, void* out16,
                          int num_out_rows, int num_src_rows, int hidden, float eps, int write_back, int* status,
                          const CombineSrc& cs, cudaStream_t stream) {
    if (num_out_rows <= 0) return 0;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const bool many = num_out_rows >= 256;
    if (smem > 48 * 1024) {
        cudaError_t e = many ? cudaFuncSetAttribute(rmsnorm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                             : cudaFuncSetAttribute(rmsnorm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int vec = hidden % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                    (uintptr_t)out32 % 16 == 0 && (uintptr_t)out16 % 8 == 0;
    if (cs.y && (!vec || delta || (uintptr_t)cs.y % 16 || (uintptr_t)cs.shared % 16 || cs.top_k < 0)) return -1;
    if (many)
        return launch_pdl(rmsnorm_kernel<4>, num_out_rows, threads, smem, stream, x, delta, w, rows, out32,
                          (__nv_bfloat16*)out16, hidden, eps, write_back, num_src_rows, status, vec, cs);
    return launch_pdl(rmsnorm_kernel<1>, num_out_rows, threads, smem, stream, x, delta, w, rows, out32,
                      (__nv_bfloat16*)out16, hidden, eps, write_back, num_src_rows, status, vec, cs);
}

MOE_API int moe_rmsnorm(float* x, const float* delta, const float* w, const int* rows, float* out32, void* out16,
                        int num_out_rows, int num_src_rows, int hidden, float eps, int write_back, int* status,
                        cudaStream_t stream) {
    CombineSrc none = {};
    return rmsnorm_launch(x, delta, w, rows, out32, out16, num_out_rows, num_src_rows, hidden, eps, write_back, status,
                          none, stream);
}

// The same with the delta still uncombined (see CombineSrc).  Returns -1, with nothing launched, if
// the rows are not whole 16-byte units: the caller then combines first.
MOE_API int moe_rmsnorm_combine(float* x, const float* y, const int* pos_of_pair, const float* topk_w, int top_k,
                                const float* shared, const float* shared_gate, const float* w, const int* rows,
                                float* out32, void* out16, int num_out_rows, int num_src_rows, int hidden, float eps,
                                int write_back, int* status, cudaStream_t stream) {
    if (!y || !pos_of_pair || !topk_w) return (int)cudaErrorInvalidValue;
    CombineSrc cs;
    cs.y = y, cs.pos = pos_of_pair, cs.w = topk_w, cs.top_k = top_k, cs.shared = shared, cs.gate = shared_gate;
    return rmsnorm_launch(x, nullptr, w, rows, out32, out16, num_out_rows, num_src_rows, hidden, eps, write_back,
                          status, cs, stream);
}

// Programmatic dependent launch on or off for every kernel of this library (on by default).
MOE_API void moe_set_pdl(int enabled) { g_pdl_enabled = enabled ? 1 : 0; }

// out[i] = a[i] + b[i] (32-bit residual sum where no norm follows).
__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}
MOE_API int moe_add_inplace(float* a, const float* b, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(a, b, (size_t)n);
    return launch_status();
}
