// Attention of this step's queries over the cache: the plain kernel.
//
// For the query at position p of a sequence (reference: src/model.rs:794-827):
//   lo = window ? max(0, p + 1 - window) : 0
//   s_j = (q . k_j) * scale for j in [lo, p];  softmax (subtract max, exp, divide
//   by the sum);  o = sum_j s_j v_j;  kv head = head / (heads / kv_heads).
// Scores, the softmax and the weighted sum are 32-bit whatever the storage type.
//
// Keys and values at positions before the step (j < seq_start) come from the
// paged cache; those of the step itself come from k_new / v_new, so the kernel
// does not depend on whether the step has been appended to the cache yet.  With
// use_local == 0 every key comes from the cache (a layer that reads another
// layer's cache).
//
// One warp per (token, head): lanes take one key each for the scores and one
// slice of the head dimension each for the weighted sum.  Any number of heads
// and groups; head_dim a multiple of 16 up to 256.
#include "common.cuh"

namespace {

constexpr int MAX_HD = 256;

__device__ __forceinline__ float dot_row(const float* kp, const float* qs, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kp + d);
        s = fmaf(kv.x, qs[d], s);
        s = fmaf(kv.y, qs[d + 1], s);
        s = fmaf(kv.z, qs[d + 2], s);
        s = fmaf(kv.w, qs[d + 3], s);
    }
    return s;
}
__device__ __forceinline__ float dot_row(const __nv_bfloat16* kp, const float* qs, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 8) {
        const uint4 kv = *reinterpret_cast<const uint4*>(kp + d);
        const unsigned w[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s = fmaf(__uint_as_float(w[i] << 16), qs[d + 2 * i], s);
            s = fmaf(__uint_as_float(w[i] & 0xffff0000u), qs[d + 2 * i + 1], s);
        }
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(32)
attn_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_new, const T* __restrict__ v_new,
                    const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
                    const int* __restrict__ seq_of_token, const int* __restrict__ pos,
                    const int* __restrict__ seq_start, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ slots, const int* __restrict__ tables, int table_stride, int ring,
                    int page_size, int num_pages, int nh, int nkv, int hd, int window, float scale, int use_local,
                    int* status) {
    __shared__ __align__(16) float qs[MAX_HD];
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int s = seq_of_token[t];
    T* o = out + ((size_t)t * nh + h) * hd;
    if (s < 0) {   // padding row
        for (int d = lane; d < hd; d += 32) st_f(o + d, 0.f);
        return;
    }
    const int p = pos[t];
    const int p0 = use_local ? seq_start[s] : p + 1;
    const int lo = window > 0 ? max(0, p + 1 - window) : 0;
    const int kvh = h / (nh / nkv);
    const int tok0 = cu_seqlens[s];
    const int* table = tables + (size_t)slots[s] * table_stride;
    for (int d = lane; d < hd; d += 32) qs[d] = ld_f(q + ((size_t)t * nh + h) * hd + d);
    __syncwarp();

    float acc[MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; i++) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= p;
        const T* kp = nullptr;
        const T* vp = nullptr;
        if (valid) {
            if (j >= p0) {
                const size_t r = ((size_t)(tok0 + (j - p0)) * nkv + kvh) * hd;
                kp = k_new + r, vp = v_new + r;
            } else {
                const CachePos cp = cache_pos(j, ring, table, page_size, num_pages, status);
                const size_t r = cache_index(cp, kvh, nkv, page_size, hd);
                kp = k_cache + r, vp = v_cache + r;
            }
        }
        const float sc = valid ? dot_row(kp, qs, hd) * scale : -INFINITY;
        const float m_new = fmaxf(m, warp_max(sc));
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pr = valid ? expf(sc - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < MAX_HD / 32; i++) acc[i] *= alpha;
        const int n_valid = min(32, p - j0 + 1);
        for (int jj = 0; jj < n_valid; jj++) {
            const float pj = __shfl_sync(0xffffffffu, pr, jj);
            const T* vj = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vp, jj);
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; i++) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, ld_f(vj + d), acc[i]);
            }
        }
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; i++) {
        const int d = lane + 32 * i;
        if (d < hd) st_f(o + d, acc[i] * inv);
    }
}

}  // namespace

MOE_API int moe_attention_generic(const void* q, const void* k_new, const void* v_new, const void* k_cache,
                                  const void* v_cache, void* out, int dt, const int* seq_of_token, const int* pos,
                                  const int* seq_start, const int* cu_seqlens, const int* slots, const int* tables,
                                  int table_stride, int ring, int page_size, int num_pages, int num_tokens, int nh,
                                  int nkv, int hd, int window, float scale, int use_local, int* status,
                                  cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hd % 16 != 0 || hd > MAX_HD || hd <= 0 || nkv <= 0 || nh % nkv != 0 || nh > 65535)
        return (int)cudaErrorInvalidValue;
    dim3 grid(num_tokens, nh);
    if (dt == DT_F32)
        attn_generic_kernel<float><<<grid, 32, 0, stream>>>(
            (const float*)q, (const float*)k_new, (const float*)v_new, (const float*)k_cache, (const float*)v_cache,
            (float*)out, seq_of_token, pos, seq_start, cu_seqlens, slots, tables, table_stride, ring, page_size,
            num_pages, nh, nkv, hd, window, scale, use_local, status);
    else
        attn_generic_kernel<__nv_bfloat16><<<grid, 32, 0, stream>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new,
            (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, seq_of_token, pos,
            seq_start, cu_seqlens, slots, tables, table_stride, ring, page_size, num_pages, nh, nkv, hd, window,
            scale, use_local, status);
    return launch_status();
}
