// Rotary position encoding of queries and keys, and the append of keys and
// values to the paged cache.
//
// Rotation (reference: src/model.rs:324-333): per head, half-split pairs
// (i, i + rot/2): a' = a cos - b sin, b' = a sin + b cos with the angle
// float(pos) * inv_freq[i] computed in 32-bit.  Keys are cached after rotation
// (src/model.rs:729-734).
#include "common.cuh"

// qkv: [T, (nh + 2 nkv) * hd] 32-bit, biases already added.  One block per token.
// Writes q [T, nh, hd], k [T, nkv, hd], v [T, nkv, hd] in the activation dtype.
template <typename OT>
__global__ void rope_split_kernel(const float* __restrict__ qkv, const int* __restrict__ pos,
                                  const float* __restrict__ inv_freq, int nh, int nkv, int hd, int rot,
                                  OT* __restrict__ q, OT* __restrict__ k, OT* __restrict__ v) {
    const int t = blockIdx.x;
    const int width = (nh + 2 * nkv) * hd;
    const float* src = qkv + (size_t)t * width;
    const float p = (float)pos[t];
    const int half = rot / 2;
    const int rot_heads = nh + nkv;   // heads that are rotated: queries then keys
    // the token's angles once (all heads share them): cos[half], sin[half]
    extern __shared__ float split_tab[];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &split_tab[half + i], &split_tab[i]);
    __syncthreads();
    // rotated part: one thread per (head, pair)
    for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const float* s = src + (size_t)h * hd;
        const float cs = split_tab[i], sn = split_tab[half + i];
        const float a = s[i], b = s[i + half];
        OT* dst = h < nh ? q + ((size_t)t * nh + h) * hd : k + ((size_t)t * nkv + (h - nh)) * hd;
        st_f(dst + i, rot_lo(a, b, cs, sn));
        st_f(dst + i + half, rot_hi(a, b, cs, sn));
    }
    // pass-through part of rotated heads (rot < hd)
    if (rot < hd) {
        const int rest = hd - rot;
        for (int idx = threadIdx.x; idx < rot_heads * rest; idx += blockDim.x) {
            const int h = idx / rest, i = rot + idx % rest;
            OT* dst = h < nh ? q + ((size_t)t * nh + h) * hd : k + ((size_t)t * nkv + (h - nh)) * hd;
            st_f(dst + i, src[(size_t)h * hd + i]);
        }
    }
    // values
    const float* vs = src + (size_t)(nh + nkv) * hd;
    OT* vd = v + (size_t)t * nkv * hd;
    for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) st_f(vd + i, vs[i]);
}

// Where a token's keys and values go in a paged cache (optional part of rope_split4_kernel).
struct CommitArgs {
    void* k_cache;            // null: no commit
    void* v_cache;
    const int* seq_of_token;
    const int* seq_end;
    const int* slots;
    const int* tables;
    int table_stride, ring, page_size, num_pages;
    int* status;
};

__device__ __forceinline__ void st4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// The same as rope_split_kernel, four elements a thread (16-byte loads, 8- or 16-byte stores), for
// head sizes and rotated widths that are multiples of 8; optionally it also appends the keys and
// values to the cache (the arithmetic of kv_commit_kernel), which spares that launch where nothing
// of this step's attention reads the cache (whole prompts).  One block per token.
template <typename OT>
__global__ void __launch_bounds__(256)
rope_split4_kernel(const float* __restrict__ qkv, const int* __restrict__ pos, const float* __restrict__ inv_freq,
                   int nh, int nkv, int hd, int rot, OT* __restrict__ q, OT* __restrict__ k, OT* __restrict__ v,
                   const CommitArgs c) {
    extern __shared__ __align__(16) float split_tab4[];
    const int t = blockIdx.x;
    const int p_int = pos[t];
    const float p = (float)p_int;
    const int half = rot / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x)
        sincosf(p * inv_freq[i], &split_tab4[half + i], &split_tab4[i]);
    pdl_sync();
    __syncthreads();
    const int width = (nh + 2 * nkv) * hd;
    const float* src = qkv + (size_t)t * width;
    // the cache place of this token, if it is to be written
    OT* kc = nullptr;
    OT* vc = nullptr;
    if (c.k_cache) {
        const int s = c.seq_of_token[t];
        if (s >= 0 && !(c.ring > 0 && p_int < c.seq_end[s] - c.ring)) {
            const CachePos cp = cache_pos(p_int, c.ring, c.tables + (size_t)c.slots[s] * c.table_stride, c.page_size,
                                          c.num_pages, c.status);
            const size_t at = cache_index(cp, 0, nkv, c.page_size, hd);       // head h: + h * page_size * hd
            kc = (OT*)c.k_cache + at, vc = (OT*)c.v_cache + at;
        }
    }
    const size_t head_step = (size_t)c.page_size * hd;
    const int rot_heads = nh + nkv, hq = half / 4;
    for (int idx = threadIdx.x; idx < rot_heads * hq; idx += blockDim.x) {
        const int h = idx / hq, i = (idx % hq) * 4;
        const float* s = src + (size_t)h * hd;
        const float4 a = *reinterpret_cast<const float4*>(s + i), b = *reinterpret_cast<const float4*>(s + i + half);
        const float4 cs = *reinterpret_cast<const float4*>(split_tab4 + i);
        const float4 sn = *reinterpret_cast<const float4*>(split_tab4 + half + i);
        const float l0 = rot_lo(a.x, b.x, cs.x, sn.x), l1 = rot_lo(a.y, b.y, cs.y, sn.y),
                    l2 = rot_lo(a.z, b.z, cs.z, sn.z), l3 = rot_lo(a.w, b.w, cs.w, sn.w);
        const float h0 = rot_hi(a.x, b.x, cs.x, sn.x), h1 = rot_hi(a.y, b.y, cs.y, sn.y),
                    h2 = rot_hi(a.z, b.z, cs.z, sn.z), h3 = rot_hi(a.w, b.w, cs.w, sn.w);
        OT* dst = h < nh ? q + ((size_t)t * nh + h) * hd : k + ((size_t)t * nkv + (h - nh)) * hd;
        st4(dst + i, l0, l1, l2, l3);
        st4(dst + i + half, h0, h1, h2, h3);
        if (h >= nh && kc) {
            OT* cd = kc + (size_t)(h - nh) * head_step;
            st4(cd + i, l0, l1, l2, l3);
            st4(cd + i + half, h0, h1, h2, h3);
        }
    }
    if (rot < hd) {      // pass-through part of rotated heads
        const int rq = (hd - rot) / 4;
        for (int idx = threadIdx.x; idx < rot_heads * rq; idx += blockDim.x) {
            const int h = idx / rq, i = rot + (idx % rq) * 4;
            const float4 a = *reinterpret_cast<const float4*>(src + (size_t)h * hd + i);
            OT* dst = h < nh ? q + ((size_t)t * nh + h) * hd : k + ((size_t)t * nkv + (h - nh)) * hd;
            st4(dst + i, a.x, a.y, a.z, a.w);
            if (h >= nh && kc) st4(kc + (size_t)(h - nh) * head_step + i, a.x, a.y, a.z, a.w);
        }
    }
    const float* vs = src + (size_t)(nh + nkv) * hd;
    OT* vd = v + (size_t)t * nkv * hd;
    for (int i = threadIdx.x * 4; i < nkv * hd; i += blockDim.x * 4) {
        const float4 a = *reinterpret_cast<const float4*>(vs + i);
        st4(vd + i, a.x, a.y, a.z, a.w);
        if (vc) st4(vc + (size_t)(i / hd) * head_step + i % hd, a.x, a.y, a.z, a.w);
    }
}

// With cache arguments (k_cache not null) the keys and values are also appended to the cache, as
// moe_kv_commit would: only for steps whose attention reads nothing from the cache.
MOE_API int moe_rope_split(const float* qkv, const int* pos, const float* inv_freq, int num_tokens, int nh, int nkv,
                           int hd, int rot, void* q, void* k, void* v, int out_dt, void* k_cache, void* v_cache,
                           const int* seq_of_token, const int* seq_end, const int* slots, const int* tables,
                           int table_stride, int ring, int page_size, int num_pages, int* status,
                           cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1)) return (int)cudaErrorInvalidValue;
    if (rot > 0 && !inv_freq) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    if (rot > 8192) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)rot * sizeof(float);
    const bool vec = hd % 8 == 0 && rot % 8 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q % 16 == 0) &&
                     ((uintptr_t)k % 16 == 0) && ((uintptr_t)v % 16 == 0) &&
                     (!k_cache || ((uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0));
    if (k_cache && !vec) return -1;      // the caller commits with moe_kv_commit
    if (vec) {
        CommitArgs c;
        c.k_cache = k_cache, c.v_cache = v_cache, c.seq_of_token = seq_of_token, c.seq_end = seq_end, c.slots = slots;
        c.tables = tables, c.table_stride = table_stride, c.ring = ring, c.page_size = page_size;
        c.num_pages = num_pages, c.status = status;
        if (out_dt == DT_F32)
            return launch_pdl(rope_split4_kernel<float>, num_tokens, threads, smem, stream, qkv, pos, inv_freq, nh, nkv,
                              hd, rot, (float*)q, (float*)k, (float*)v, c);
        return launch_pdl(rope_split4_kernel<__nv_bfloat16>, num_tokens, threads, smem, stream, qkv, pos, inv_freq, nh,
                          nkv, hd, rot, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, c);
    }
    if (out_dt == DT_F32)
        rope_split_kernel<float><<<num_tokens, threads, smem, stream>>>(qkv, pos, inv_freq, nh, nkv, hd, rot, (float*)q,
                                                                         (float*)k, (float*)v);
    else
        rope_split_kernel<__nv_bfloat16><<<num_tokens, threads, smem, stream>>>(
            qkv, pos, inv_freq, nh, nkv, hd, rot, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v);
    return launch_status();
}

// Append this step's keys and values to one layer of a paged cache.
//   k_new, v_new: [T, nkv, hd];  cache: [page][nkv][page_size][hd] each
//   A token is written iff its position is among the last `ring` positions of
//   its sequence after the step (ring == 0: always), so that in a ring no two
//   tokens of one step write the same place.
template <typename T>
__global__ void kv_commit_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, T* __restrict__ k_cache,
                                 T* __restrict__ v_cache, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ pos, const int* __restrict__ seq_end,
                                 const int* __restrict__ slots, const int* __restrict__ tables, int table_stride,
                                 int ring, int page_size, int num_pages, int nkv, int hd, int* status) {
    const int t = blockIdx.x;
    const int s = seq_of_token[t];
    if (s < 0) return;
    const int p = pos[t];
    if (ring > 0 && p < seq_end[s] - ring) return;
    const int* table = tables + (size_t)slots[s] * table_stride;
    const CachePos cp = cache_pos(p, ring, table, page_size, num_pages, status);
    for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) {
        const int h = i / hd, d = i % hd;
        const size_t dst = cache_index(cp, h, nkv, page_size, hd) + d;
        k_cache[dst] = k_new[(size_t)t * nkv * hd + i];
        v_cache[dst] = v_new[(size_t)t * nkv * hd + i];
    }
}

MOE_API int moe_kv_commit(const void* k_new, const void* v_new, void* k_cache, void* v_cache, int dt,
                          const int* seq_of_token, const int* pos, const int* seq_end, const int* slots,
                          const int* tables, int table_stride, int ring, int page_size, int num_pages, int num_tokens,
                          int nkv, int hd, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    const int threads = 128;
    if (dt == DT_F32)
        kv_commit_kernel<float><<<num_tokens, threads, 0, stream>>>(
            (const float*)k_new, (const float*)v_new, (float*)k_cache, (float*)v_cache, seq_of_token, pos, seq_end,
            slots, tables, table_stride, ring, page_size, num_pages, nkv, hd, status);
    else
        kv_commit_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>(
            (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache, seq_of_token, pos, seq_end, slots, tables, table_stride, ring, page_size,
            num_pages, nkv, hd, status);
    return launch_status();
}

// Page-table maintenance: table[slot][index] = page for n (slot, index, page) triples.
__global__ void table_update_kernel(int* __restrict__ table, int stride, const int* __restrict__ upd, int n) {
    pdl_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) table[(size_t)upd[3 * i] * stride + upd[3 * i + 1]] = upd[3 * i + 2];
}
// A decode step (one token per sequence): rotate, write the query, and append key and value
// straight into the cache, in one launch.  Same arithmetic as rope_split_kernel followed by
// kv_commit_kernel.  One block per token.
template <typename OT>
__global__ void rope_commit_kernel(const float* __restrict__ qkv, const int* __restrict__ pos,
                                   const float* __restrict__ inv_freq, int nh, int nkv, int hd, int rot,
                                   OT* __restrict__ q, OT* __restrict__ k_cache, OT* __restrict__ v_cache,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                   const int* __restrict__ tables, int table_stride, int ring, int page_size,
                                   int num_pages, int* status) {
    pdl_sync();
    const int t = blockIdx.x;
    const int width = (nh + 2 * nkv) * hd;
    const float* src = qkv + (size_t)t * width;
    const int s = seq_of_token[t];
    const int p_int = pos[t];
    const float p = (float)p_int;
    const int half = rot / 2;
    CachePos cp;
    cp.page = 0, cp.off = 0;
    if (s >= 0) cp = cache_pos(p_int, ring, tables + (size_t)slots[s] * table_stride, page_size, num_pages, status);
    const int rot_heads = nh + nkv;
    // the token's angles once (all heads share them): cos[half], sin[half]
    extern __shared__ float angle_tab[];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &angle_tab[half + i], &angle_tab[i]);
    __syncthreads();
    for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const float* sp = src + (size_t)h * hd;
        const float cs = angle_tab[i], sn = angle_tab[half + i];
        const float a = sp[i], b = sp[i + half];
        OT* dst;
        if (h < nh) {
            dst = q + ((size_t)t * nh + h) * hd;
        } else {
            if (s < 0) continue;                          // a padding row has no cache
            dst = k_cache + cache_index(cp, h - nh, nkv, page_size, hd);
        }
        st_f(dst + i, rot_lo(a, b, cs, sn));
        st_f(dst + i + half, rot_hi(a, b, cs, sn));
    }
    if (rot < hd) {
        const int rest = hd - rot;
        for (int idx = threadIdx.x; idx < rot_heads * rest; idx += blockDim.x) {
            const int h = idx / rest, i = rot + idx % rest;
            OT* dst;
            if (h < nh) {
                dst = q + ((size_t)t * nh + h) * hd;
            } else {
                if (s < 0) continue;
                dst = k_cache + cache_index(cp, h - nh, nkv, page_size, hd);
            }
            st_f(dst + i, src[(size_t)h * hd + i]);
        }
    }
    if (s >= 0) {
        const float* vs = src + (size_t)(nh + nkv) * hd;
        for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x)
            st_f(v_cache + cache_index(cp, i / hd, nkv, page_size, hd) + i % hd, vs[i]);
    }
}

MOE_API int moe_rope_commit(const float* qkv, const int* pos, const float* inv_freq, int num_tokens, int nh, int nkv,
                            int hd, int rot, void* q, void* k_cache, void* v_cache, int dt, const int* seq_of_token,
                            const int* slots, const int* tables, int table_stride, int ring, int page_size,
                            int num_pages, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (rot < 0 || rot > hd || (rot & 1)) return (int)cudaErrorInvalidValue;
    if (rot > 0 && !inv_freq) return (int)cudaErrorInvalidValue;
    if (rot > 8192) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)rot * sizeof(float);
    if (dt == DT_F32)
        return launch_pdl(rope_commit_kernel<float>, num_tokens, 512, smem, stream, qkv, pos, inv_freq, nh, nkv, hd,
                          rot, (float*)q, (float*)k_cache, (float*)v_cache, seq_of_token, slots, tables, table_stride,
                          ring, page_size, num_pages, status);
    return launch_pdl(rope_commit_kernel<__nv_bfloat16>, num_tokens, 512, smem, stream, qkv, pos, inv_freq, nh, nkv, hd,
                      rot, (__nv_bfloat16*)q, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, seq_of_token, slots,
                      tables, table_stride, ring, page_size, num_pages, status);
}

MOE_API int moe_table_update(int* table, int stride, const int* upd, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return launch_pdl(table_update_kernel, (n + 127) / 128, 128, 0, stream, table, stride, upd, n);
}
