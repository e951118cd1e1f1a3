// Attention of single new tokens over the paged cache, split along the keys.
//
// A decode step has few queries and long caches, so one CTA per (key split, kv head,
// token) reads its share of the keys and values ONCE for all query heads of the group
// and leaves a partial softmax (running maximum m, sum l, weighted values) in scratch;
// a second kernel merges the splits.  Formulas as in attention_generic.cu
// (reference: src/model.rs:794-827); scores, softmax and sums are 32-bit.
//
// Every key comes from the cache: the step's own keys must have been appended before
// the call.  That is only safe for steps of ONE token per sequence (a ring then never
// overwrites a key the same step still needs), which is what the caller guarantees.
//
// The number of splits is fixed at launch (so the launch can live in a CUDA graph);
// the keys per split follow each sequence's length on the device.
#include "common.cuh"

namespace {

constexpr int MAX_HD = 256;
constexpr int GH = 4;          // query heads handled together (registers)
constexpr int WARPS = 4;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* out);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* out) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x, out[1] = a.y, out[2] = a.z, out[3] = a.w, out[4] = b.x, out[5] = b.y, out[6] = b.z, out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// partial layout: [token][head][split] records of (hd + 2) floats: acc[hd], m, l
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_partial_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                           float* __restrict__ partial, const int* __restrict__ seq_of_token,
                           const int* __restrict__ pos, const int* __restrict__ slots,
                           const int* __restrict__ tables, int table_stride, int ring, int page_size, int num_pages,
                           int nh, int nkv, int hd, int window, float scale, int* status) {
    extern __shared__ float sm[];
    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = nh / nkv;
    const int rec = hd + 2;
    const int s = seq_of_token[t];
    if (s < 0) return;                                   // padding row: the merge kernel writes zeros
    const int p = pos[t];
    const int lo = window > 0 ? max(0, p + 1 - window) : 0;
    const int n_keys = p + 1 - lo;
    int per = (n_keys + nsplit - 1) / nsplit;
    per = (per + 31) & ~31;                              // whole tiles of 32 keys per split
    const int k_begin = lo + split * per;
    const int k_end = min(p + 1, k_begin + per);
    const int* table = tables + (size_t)slots[s] * table_stride;

    float* qs = sm;                                      // [GH][hd]
    float* red = sm + GH * hd;                           // [WARPS][GH][hd + 2]
    const int dpl = (hd + 31) / 32;                      // dims per lane

    for (int h0 = 0; h0 < group; h0 += GH) {
        const int gh = min(GH, group - h0);
        __syncthreads();
        for (int i = threadIdx.x; i < gh * hd; i += blockDim.x)
            qs[i] = ld_f(q + ((size_t)t * nh + kvh * group + h0 + i / hd) * hd + i % hd);
        __syncthreads();

        float m[GH], l[GH], acc[GH][MAX_HD / 32];
#pragma unroll
        for (int g = 0; g < GH; g++) {
            m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; i++) acc[g][i] = 0.f;
        }
        for (int j0 = k_begin + warp * 32; j0 < k_end; j0 += WARPS * 32) {
            const int j = j0 + lane;
            const bool valid = j < k_end;
            const T* kp = nullptr;
            const T* vp = nullptr;
            float sc[GH];
#pragma unroll
            for (int g = 0; g < GH; g++) sc[g] = 0.f;
            if (valid) {
                const CachePos cp = cache_pos(j, ring, table, page_size, num_pages, status);
                const size_t r = cache_index(cp, kvh, nkv, page_size, hd);
                kp = k_cache + r, vp = v_cache + r;
#pragma unroll 4
                for (int d = 0; d < hd; d += 8) {
                    float kv[8];
                    load8<T>(kp + d, kv);
#pragma unroll
                    for (int g = 0; g < GH; g++) {
                        if (g < gh) {
                            const float* qg = qs + g * hd + d;
#pragma unroll
                            for (int e = 0; e < 8; e++) sc[g] = fmaf(kv[e], qg[e], sc[g]);
                        }
                    }
                }
            }
            const int n_valid = min(32, k_end - j0);
            float pr[GH];
#pragma unroll
            for (int g = 0; g < GH; g++) {
                if (g < gh) {
                    const float x = valid ? sc[g] * scale : -INFINITY;
                    const float m_new = fmaxf(m[g], warp_max(x));
                    const float alpha = (m[g] == -INFINITY) ? 0.f : expf(m[g] - m_new);
                    pr[g] = valid ? expf(x - m_new) : 0.f;
                    l[g] = l[g] * alpha + warp_sum(pr[g]);
                    m[g] = m_new;
#pragma unroll
                    for (int i = 0; i < MAX_HD / 32; i++) acc[g][i] *= alpha;
                } else {
                    pr[g] = 0.f;
                }
            }
#pragma unroll 4
            for (int jj = 0; jj < n_valid; jj++) {
                const T* vj = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vp, jj);
                float vv[MAX_HD / 32];
#pragma unroll
                for (int i = 0; i < MAX_HD / 32; i++) {
                    const int d = lane + 32 * i;
                    vv[i] = (i < dpl && d < hd) ? ld_f(vj + d) : 0.f;
                }
#pragma unroll
                for (int g = 0; g < GH; g++) {
                    if (g < gh) {
                        const float pj = __shfl_sync(0xffffffffu, pr[g], jj);
#pragma unroll
                        for (int i = 0; i < MAX_HD / 32; i++) acc[g][i] = fmaf(pj, vv[i], acc[g][i]);
                    }
                }
            }
        }
        // merge the warps of this CTA (fixed order), then write the split's record
#pragma unroll
        for (int g = 0; g < GH; g++) {
            if (g < gh) {
                float* r = red + ((size_t)warp * GH + g) * rec;
#pragma unroll
                for (int i = 0; i < MAX_HD / 32; i++) {
                    const int d = lane + 32 * i;
                    if (d < hd) r[d] = acc[g][i];
                }
                if (lane == 0) r[hd] = m[g], r[hd + 1] = l[g];
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < gh * hd; idx += blockDim.x) {
            const int g = idx / hd, d = idx % hd;
            float mm = -INFINITY;
            for (int w = 0; w < WARPS; w++) mm = fmaxf(mm, red[((size_t)w * GH + g) * rec + hd]);
            float a = 0.f, ll = 0.f;
            for (int w = 0; w < WARPS; w++) {
                const float* r = red + ((size_t)w * GH + g) * rec;
                const float f = (r[hd] == -INFINITY) ? 0.f : expf(r[hd] - mm);
                a += f * r[d];
                ll += f * r[hd + 1];
            }
            float* out = partial + (((size_t)t * nh + kvh * group + h0 + g) * nsplit + split) * rec;
            out[d] = a;
            if (d == 0) out[hd] = mm, out[hd + 1] = ll;
        }
    }
}

// one block per (token, head): merge the splits in order and normalise
template <typename T>
__global__ void attn_decode_merge_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                         const int* __restrict__ seq_of_token, int nh, int hd, int nsplit) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int rec = hd + 2;
    T* o = out + ((size_t)t * nh + h) * hd;
    if (seq_of_token[t] < 0) {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) st_f(o + d, 0.f);
        return;
    }
    const float* base = partial + ((size_t)t * nh + h) * nsplit * rec;
    float mm = -INFINITY;
    for (int s = 0; s < nsplit; s++) mm = fmaxf(mm, base[(size_t)s * rec + hd]);
    float ll = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ms = base[(size_t)s * rec + hd];
        ll += (ms == -INFINITY) ? 0.f : expf(ms - mm) * base[(size_t)s * rec + hd + 1];
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < nsplit; s++) {
            const float ms = base[(size_t)s * rec + hd];
            if (ms != -INFINITY) a += expf(ms - mm) * base[(size_t)s * rec + d];
        }
        st_f(o + d, a / ll);
    }
}

}  // namespace

// q: [T, nh, hd]; out: [T, nh * hd]; partial: T * nh * nsplit * (hd + 2) floats of scratch.
MOE_API int moe_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* partial,
                                 int dt, const int* seq_of_token, const int* pos, const int* slots,
                                 const int* tables, int table_stride, int ring, int page_size, int num_pages,
                                 int num_tokens, int nh, int nkv, int hd, int window, float scale, int nsplit,
                                 int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hd % 16 != 0 || hd > MAX_HD || hd <= 0 || nkv <= 0 || nh % nkv != 0 || nsplit < 1 || nsplit > 65535 ||
        nkv > 65535 || num_tokens > 65535)
        return (int)cudaErrorInvalidValue;
    dim3 grid(nsplit, nkv, num_tokens);
    const size_t smem = ((size_t)GH * hd + (size_t)WARPS * GH * (hd + 2)) * sizeof(float);
    dim3 mgrid(num_tokens, nh);
    if (dt == DT_F32) {
        attn_decode_partial_kernel<float><<<grid, WARPS * 32, smem, stream>>>(
            (const float*)q, (const float*)k_cache, (const float*)v_cache, partial, seq_of_token, pos, slots, tables,
            table_stride, ring, page_size, num_pages, nh, nkv, hd, window, scale, status);
        attn_decode_merge_kernel<float><<<mgrid, 128, 0, stream>>>(partial, (float*)out, seq_of_token, nh, hd, nsplit);
    } else {
        attn_decode_partial_kernel<__nv_bfloat16><<<grid, WARPS * 32, smem, stream>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, partial,
            seq_of_token, pos, slots, tables, table_stride, ring, page_size, num_pages, nh, nkv, hd, window, scale,
            status);
        attn_decode_merge_kernel<__nv_bfloat16>
            <<<mgrid, 128, 0, stream>>>(partial, (__nv_bfloat16*)out, seq_of_token, nh, hd, nsplit);
    }
    return launch_status();
}
