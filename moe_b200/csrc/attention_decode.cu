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
//
// Memory access: a warp takes 32 consecutive positions (half a page), whose keys are
// contiguous in the cache.  Each load instruction moves 512 contiguous bytes (16 per
// lane), all loads of a tile are in flight together, and the scores are formed by a
// transpose-reduction across the lanes that share a key row: no shared memory, no
// per-lane strided walk.  Head sizes whose rows are not 64, 128, 256 or 512 bytes
// take the slower row-per-lane kernel.
#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int MAX_HD = 256;
constexpr int WARPS = 4;

template <typename T>
struct Chunk;   // 16 bytes of a row as floats
template <>
struct Chunk<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& v, float* out) {
        out[0] = __uint_as_float(v.x), out[1] = __uint_as_float(v.y);
        out[2] = __uint_as_float(v.z), out[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ void load(const float* p, float* out) {
        unpack(*reinterpret_cast<const uint4*>(p), out);
    }
};
template <>
struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& v, float* out) {
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        unpack(*reinterpret_cast<const uint4*>(p), out);
    }
};

// partial layout: [token][head][split] records of (hd + 2) floats: acc[hd], m, l

__device__ __forceinline__ float through(float v, const float*) { return v; }
__device__ __forceinline__ float through(float v, const __nv_bfloat16*) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void store_chunk(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_chunk(__nv_bfloat16* p, const float* v) {
    uint4 u;
    unsigned* w = &u.x;
#pragma unroll
    for (int i = 0; i < 4; i++)   // v already holds bfloat16 values: the low halves are zero
        w[i] = (__float_as_uint(v[2 * i]) >> 16) | (__float_as_uint(v[2 * i + 1]) & 0xffff0000u);
    *reinterpret_cast<uint4*>(p) = u;
}

// What the fused form of the kernel needs beside the attention itself: it takes the step's
// 32-bit q/k/v rows (biases added), rotates them, appends key and value to the cache, and the CTA
// that finishes last for a (token, kv head) merges the splits and writes the output.
struct FusedArgs {
    const float* qkv;        // [T, (nh + 2 nkv) * hd]
    const float* inv_freq;   // [rot / 2] (null if rot == 0)
    int rot;
    void* k_append;          // the cache arrays again, as the place of the append
    void* v_append;
    void* out;               // [T, nh * hd]
    int* tickets;            // [T * nkv], zero before and after the launch
};

// EPC consecutive elements d0 .. of one head's 32-bit row, rotated (same arithmetic as
// rope_commit_kernel) and rounded through the storage type.  ang: cos[half], sin[half].
template <typename T, int EPC>
__device__ __forceinline__ void rotated_chunk(const float* __restrict__ src, int d0, int half, int rot,
                                              const float* ang, float* out) {
#pragma unroll
    for (int e = 0; e < EPC; e++) {
        const int d = d0 + e;
        float v;
        if (d < rot) {
            const int i = d < half ? d : d - half;
            const float a = src[i], b = src[i + half], cs = ang[i], sn = ang[half + i];
            v = d < half ? rot_lo(a, b, cs, sn) : rot_hi(a, b, cs, sn);
        } else {
            v = src[d];
        }
        out[e] = through(v, (const T*)nullptr);
    }
}

// LPR: lanes per key row (row bytes / 16); GH: query heads handled together.
template <typename T, int LPR, int GH, bool FUSED>
__global__ void __launch_bounds__(WARPS * 32, (GH == 1 && LPR <= 16) ? 4 : 1)
attn_decode_fast_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        float* __restrict__ partial, const int* __restrict__ seq_of_token,
                        const int* __restrict__ pos, const int* __restrict__ slots, const int* __restrict__ tables,
                        int table_stride, int ring, int page_size, int num_pages, int nh, int nkv, int window,
                        float scale, int* status, const FusedArgs fa, int l2_prefetch_budget) {
    constexpr int EPC = Chunk<T>::N;       // elements per 16-byte chunk
    constexpr int HD = LPR * EPC;
    constexpr int RPI = 32 / LPR;          // rows per load instruction
    constexpr int NI = LPR;                // load instructions per tile of 32 rows
    constexpr int REC = HD + 2;
    __shared__ float red[WARPS][GH][REC];
    __shared__ float ang[FUSED ? HD : 1];
    __shared__ int s_last;

    // Before the wait for the predecessor: everything that depends only on the step's layout
    // (positions, slots and page tables were written at the start of the step, more than one
    // kernel ago) and on the cache of earlier steps.  The CTA asks for its keys and values in L2
    // and forms the rotation angles, so that their latency passes while the predecessor ends.
    // grid.y: the kv heads, each `npass` times: block (kvh, pass) takes the query heads
    // [pass * GH, pass * GH + GH) of the group.  (A group of more than GH heads used to be walked by
    // one block, pass after pass; as blocks of their own the passes run side by side, and a group of
    // seven heads, with many sequences, no longer takes four times the time of its keys.)
    const int group = nh / nkv;
    const int npass = (group + GH - 1) / GH;
    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y / npass, t = blockIdx.z;
    const int h0 = (blockIdx.y % npass) * GH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rgrp = lane / LPR;
    const int s = seq_of_token[t];
    const int p = s < 0 ? 0 : pos[t];
    const int lo = window > 0 ? max(0, p + 1 - window) : 0;
    // fused: position p is this step's own key, which comes from the q/k/v row, not from the cache
    const int hi = FUSED ? p - 1 : p;
    const int half = FUSED ? fa.rot / 2 : 0;
    const int width = (nh + 2 * nkv) * HD;
    const bool owner = FUSED && split == nsplit - 1 && warp == 0;   // takes the new key (and, for h0 == 0, appends it)
    // tiles of 32 positions, aligned to 32: the keys of a tile are contiguous in one page
    const int tile_lo = lo / 32, tile_hi = p / 32 + 1;
    const int tps = (tile_hi - tile_lo + nsplit - 1) / nsplit;
    const int tb = tile_lo + split * tps, te = min(tile_hi, tb + tps);
    const int* table = tables + (size_t)(s < 0 ? 0 : slots[s]) * table_stride;
    if (s >= 0 && h0 == 0) {
        constexpr int LINES = 32 * HD * (int)sizeof(T) / 128;     // 128-byte lines of a tile of keys
        // Only as much as L2 can hold for ALL blocks of the launch (a quarter of it is left to them):
        // with many sequences the blocks' keys and values together are larger than L2, and lines
        // asked for too early would be gone again before they are used, to be read twice.
        constexpr long long TILE_BYTES = 2ll * 32 * HD * (long long)sizeof(T);
        const long long blocks = (long long)gridDim.x * gridDim.y * gridDim.z;
        const long long share = (long long)l2_prefetch_budget / (blocks * TILE_BYTES);
        const int ahead = (int)max(1ll, min((long long)(te - tb), share));
        for (int i = threadIdx.x; i < ahead * 2 * LINES; i += blockDim.x) {
            const int tile = tb + i / (2 * LINES), r = i % (2 * LINES);
            const CachePos cp = cache_pos(tile * 32, ring, table, page_size, num_pages, nullptr);
            const size_t at = cache_index(cp, kvh, nkv, page_size, HD) + (size_t)(r % LINES) * (128 / sizeof(T));
            prefetch_l2((r < LINES ? k_cache : v_cache) + at);
        }
    }
    if (s >= 0 && FUSED)
        for (int i = threadIdx.x; i < half; i += blockDim.x)
            sincosf((float)p * fa.inv_freq[i], &ang[half + i], &ang[i]);
    pdl_sync();
    if (s < 0) {                                         // padding row: zeros (unfused: by the merge kernel)
        if (FUSED && split == 0 && h0 == 0)
            for (int i = threadIdx.x; i < group * HD; i += blockDim.x)
                st_f((T*)fa.out + ((size_t)t * nh + (size_t)kvh * group) * HD + i, 0.f);
        return;
    }
    if (FUSED) __syncthreads();

    {
        const int gh = min(GH, group - h0);
        float qc[GH][EPC];
#pragma unroll
        for (int g = 0; g < GH; g++) {
            if (g < gh && FUSED)
                rotated_chunk<T, EPC>(fa.qkv + (size_t)t * width + (size_t)(kvh * group + h0 + g) * HD, sub * EPC,
                                      half, fa.rot, ang, qc[g]);
            else if (g < gh)
                Chunk<T>::load(q + ((size_t)t * nh + kvh * group + h0 + g) * HD + sub * EPC, qc[g]);
            else
#pragma unroll
                for (int e = 0; e < EPC; e++) qc[g][e] = 0.f;
        }
        float m[GH], l[GH], acc[GH][EPC];
#pragma unroll
        for (int g = 0; g < GH; g++) {
            m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < EPC; e++) acc[g][e] = 0.f;
        }
        for (int tile = tb + warp; tile < te; tile += WARPS) {
            const int j0 = tile * 32;
            const CachePos cp = cache_pos(j0, ring, table, page_size, num_pages, status);
            const size_t base = cache_index(cp, kvh, nkv, page_size, HD);
            const T* kt = k_cache + base + (size_t)rgrp * HD + sub * EPC;
            const T* vt = v_cache + base + (size_t)rgrp * HD + sub * EPC;
            // 16-byte chunks are kept packed until they are used: keys first, values reuse the registers
            uint4 raw[NI];
#pragma unroll
            for (int i = 0; i < NI; i++) raw[i] = *reinterpret_cast<const uint4*>(kt + (size_t)i * RPI * HD);
            const int my_row = sub * RPI + rgrp;          // the row whose score this lane ends up with
            const int my_j = j0 + my_row;
            const bool valid = my_j >= lo && my_j <= hi;
            float sc[GH];
#pragma unroll
            for (int g = 0; g < GH; g++) {
                sc[g] = 0.f;
                if (g >= gh) continue;                    // uniform
                float v[NI];
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    float kc[EPC];
                    Chunk<T>::unpack(raw[i], kc);
                    float d = 0.f;
#pragma unroll
                    for (int e = 0; e < EPC; e++) d = fmaf(kc[e], qc[g][e], d);
                    v[i] = d;
                }
                // transpose-reduce over the LPR lanes of a row: lane `sub` ends with the sum for i == sub
#pragma unroll
                for (int off = NI / 2; off >= 1; off >>= 1) {
                    const bool upper = (sub & off) != 0;
#pragma unroll
                    for (int k = 0; k < off; k++) {
                        const float send = upper ? v[k] : v[k + off];
                        const float keep = upper ? v[k + off] : v[k];
                        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                }
                sc[g] = v[0];
            }
#pragma unroll
            for (int i = 0; i < NI; i++) raw[i] = *reinterpret_cast<const uint4*>(vt + (size_t)i * RPI * HD);
#pragma unroll
            for (int g = 0; g < GH; g++) {
                if (g >= gh) continue;                    // uniform
                const float x = valid ? sc[g] * scale : -INFINITY;
                const float m_new = fmaxf(m[g], warp_max(x));
                float pr = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {                 // uniform: at least one valid key so far
                    alpha = (m[g] == -INFINITY) ? 0.f : expf(m[g] - m_new);
                    pr = valid ? expf(x - m_new) : 0.f;
                }
                l[g] = l[g] * alpha + warp_sum(pr);
                m[g] = m_new;
#pragma unroll
                for (int e = 0; e < EPC; e++) acc[g][e] *= alpha;
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    // rows outside [lo, p] may hold anything: they are skipped, not multiplied by zero
                    const int j = j0 + i * RPI + rgrp;
                    const float pi = __shfl_sync(0xffffffffu, pr, lane - sub + i);   // holder of row (i, rgrp)
                    if (j >= lo && j <= hi) {
                        float vc[EPC];
                        Chunk<T>::unpack(raw[i], vc);
#pragma unroll
                        for (int e = 0; e < EPC; e++) acc[g][e] = fmaf(pi, vc[e], acc[g][e]);
                    }
                }
            }
        }
        if (owner) {
            // this step's own key and value: appended to the cache, and one more position of the
            // running softmax
            float kn[EPC], vn[EPC];
            const float* row = fa.qkv + (size_t)t * width;
            rotated_chunk<T, EPC>(row + (size_t)(nh + kvh) * HD, sub * EPC, half, fa.rot, ang, kn);
            rotated_chunk<T, EPC>(row + (size_t)(nh + nkv + kvh) * HD, sub * EPC, 0, 0, ang, vn);
            if (rgrp == 0 && h0 == 0) {
                const CachePos cp = cache_pos(p, ring, table, page_size, num_pages, status);
                const size_t at = cache_index(cp, kvh, nkv, page_size, HD) + sub * EPC;
                store_chunk((T*)fa.k_append + at, kn);
                store_chunk((T*)fa.v_append + at, vn);
            }
#pragma unroll
            for (int g = 0; g < GH; g++) {
                if (g >= gh) continue;                    // uniform
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < EPC; e++) d = fmaf(kn[e], qc[g][e], d);
#pragma unroll
                for (int off = LPR / 2; off >= 1; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
                const float x = d * scale;
                const float m_new = fmaxf(m[g], x);
                const float alpha = (m[g] == -INFINITY) ? 0.f : expf(m[g] - m_new);
                const float pr = expf(x - m_new);
                l[g] = l[g] * alpha + pr;
                m[g] = m_new;
#pragma unroll
                for (int e = 0; e < EPC; e++) {
                    acc[g][e] *= alpha;
                    if (rgrp == 0) acc[g][e] = fmaf(pr, vn[e], acc[g][e]);
                }
            }
        }
        // add the row groups of the warp, then merge the warps (fixed order) and write the record
#pragma unroll
        for (int g = 0; g < GH; g++) {
#pragma unroll
            for (int e = 0; e < EPC; e++) {
                float a = acc[g][e];
#pragma unroll
                for (int off = LPR; off < 32; off <<= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
                acc[g][e] = a;
            }
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < GH; g++) {
            if (g < gh && rgrp == 0) {
#pragma unroll
                for (int e = 0; e < EPC; e++) red[warp][g][sub * EPC + e] = acc[g][e];
                if (sub == 0) red[warp][g][HD] = m[g], red[warp][g][HD + 1] = l[g];
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < gh * HD; idx += blockDim.x) {
            const int g = idx / HD, d = idx % HD;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; w++) mm = fmaxf(mm, red[w][g][HD]);
            float a = 0.f, ll = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) {
                const float f = (red[w][g][HD] == -INFINITY) ? 0.f : expf(red[w][g][HD] - mm);
                a += f * red[w][g][d];
                ll += f * red[w][g][HD + 1];
            }
            float* out = partial + (((size_t)t * nh + kvh * group + h0 + g) * nsplit + split) * REC;
            out[d] = a;
            if (d == 0) out[HD] = mm, out[HD + 1] = ll;
        }
    }
    if (!FUSED) return;
    // the CTA that arrives last at the ticket of (token, kv head) merges the splits, in split
    // order (same arithmetic as attn_decode_merge_kernel), so the result does not depend on
    // which CTA that is
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* ticket = fa.tickets + (size_t)t * nkv + kvh;
        const int last = atomicAdd(ticket, 1) == nsplit * npass - 1;
        if (last) *ticket = 0;                 // ready for the next launch
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
        const int h = kvh * group + idx / HD, d = idx % HD;
        const float* base = partial + ((size_t)t * nh + h) * nsplit * REC;
        float mm = -INFINITY;
        for (int sp = 0; sp < nsplit; sp++) mm = fmaxf(mm, __ldcg(base + (size_t)sp * REC + HD));
        float ll = 0.f, a = 0.f;
        for (int sp = 0; sp < nsplit; sp++) {
            const float ms = __ldcg(base + (size_t)sp * REC + HD);
            if (ms == -INFINITY) continue;
            const float f = expf(ms - mm);
            ll += f * __ldcg(base + (size_t)sp * REC + HD + 1);
            a += f * __ldcg(base + (size_t)sp * REC + d);
        }
        st_f((T*)fa.out + ((size_t)t * nh + h) * HD + d, a / ll);
    }
}

// The general kernel: one lane per key row, any head size that is a multiple of 16.
constexpr int GHS = 4;
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_rows_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        float* __restrict__ partial, const int* __restrict__ seq_of_token,
                        const int* __restrict__ pos, const int* __restrict__ slots,
                        const int* __restrict__ tables, int table_stride, int ring, int page_size, int num_pages,
                        int nh, int nkv, int hd, int window, float scale, int* status) {
    extern __shared__ float sm[];
    pdl_sync();
    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = nh / nkv;
    const int rec = hd + 2;
    const int s = seq_of_token[t];
    if (s < 0) return;
    const int p = pos[t];
    const int lo = window > 0 ? max(0, p + 1 - window) : 0;
    const int n_keys = p + 1 - lo;
    int per = (n_keys + nsplit - 1) / nsplit;
    per = (per + 31) & ~31;
    const int k_begin = lo + split * per;
    const int k_end = min(p + 1, k_begin + per);
    const int* table = tables + (size_t)slots[s] * table_stride;
    constexpr int EPC = Chunk<T>::N;

    float* qs = sm;                                      // [GHS][hd]
    float* red = sm + GHS * hd;                          // [WARPS][GHS][hd + 2]
    const int dpl = (hd + 31) / 32;

    for (int h0 = 0; h0 < group; h0 += GHS) {
        const int gh = min(GHS, group - h0);
        __syncthreads();
        for (int i = threadIdx.x; i < gh * hd; i += blockDim.x)
            qs[i] = ld_f(q + ((size_t)t * nh + kvh * group + h0 + i / hd) * hd + i % hd);
        __syncthreads();
        float m[GHS], l[GHS], acc[GHS][MAX_HD / 32];
#pragma unroll
        for (int g = 0; g < GHS; g++) {
            m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; i++) acc[g][i] = 0.f;
        }
        for (int j0 = k_begin + warp * 32; j0 < k_end; j0 += WARPS * 32) {
            const int j = j0 + lane;
            const bool valid = j < k_end;
            const T* vp = nullptr;
            float sc[GHS];
#pragma unroll
            for (int g = 0; g < GHS; g++) sc[g] = 0.f;
            if (valid) {
                const CachePos cp = cache_pos(j, ring, table, page_size, num_pages, status);
                const size_t r = cache_index(cp, kvh, nkv, page_size, hd);
                const T* kp = k_cache + r;
                vp = v_cache + r;
#pragma unroll 4
                for (int d = 0; d < hd; d += EPC) {
                    float kv[EPC];
                    Chunk<T>::load(kp + d, kv);
#pragma unroll
                    for (int g = 0; g < GHS; g++) {
                        if (g < gh) {
                            const float* qg = qs + g * hd + d;
#pragma unroll
                            for (int e = 0; e < EPC; e++) sc[g] = fmaf(kv[e], qg[e], sc[g]);
                        }
                    }
                }
            }
            const int n_valid = min(32, k_end - j0);
            float pr[GHS];
#pragma unroll
            for (int g = 0; g < GHS; g++) {
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
                for (int g = 0; g < GHS; g++) {
                    if (g < gh) {
                        const float pj = __shfl_sync(0xffffffffu, pr[g], jj);
#pragma unroll
                        for (int i = 0; i < MAX_HD / 32; i++) acc[g][i] = fmaf(pj, vv[i], acc[g][i]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < GHS; g++) {
            if (g < gh) {
                float* r = red + ((size_t)warp * GHS + g) * rec;
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
            for (int w = 0; w < WARPS; w++) mm = fmaxf(mm, red[((size_t)w * GHS + g) * rec + hd]);
            float a = 0.f, ll = 0.f;
            for (int w = 0; w < WARPS; w++) {
                const float* r = red + ((size_t)w * GHS + g) * rec;
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
    pdl_sync();
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

// Bytes of keys and values that the blocks of one launch may ask for in L2 ahead of their wait:
// a quarter of the device's L2.
int l2_prefetch_bytes() {
    static int bytes = 0;
    if (!bytes) {
        int dev = 0, l2 = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) != cudaSuccess)
            l2 = 0;
        bytes = l2 > 0 ? l2 / 4 : (8 << 20);
        if (const char* e = getenv("MOE_B200_ATTN_L2_MB")) bytes = atoi(e) > 0 ? atoi(e) << 20 : 1;      // for measurements
    }
    return bytes;
}

template <typename T>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, float* partial,
           const int* seq_of_token, const int* pos, const int* slots, const int* tables, int table_stride, int ring,
           int page_size, int num_pages, int num_tokens, int nh, int nkv, int hd, int window, float scale, int nsplit,
           int* status, cudaStream_t stream, const FusedArgs* fused = nullptr) {
    const int group = nh / nkv;
    dim3 grid(nsplit, nkv, num_tokens);
    const int row_bytes = hd * (int)sizeof(T);
    // the fast kernel reads q 16 bytes at a time: a q that is not 16-byte aligned (a view into the
    // middle of a buffer) takes the row-per-lane kernel, which reads it element by element.  Both
    // kernels read cache rows 16 bytes at a time; the entry points refuse a cache that is not aligned so.
    const bool aligned = ((uintptr_t)q % 16) == 0;
    const bool fast = aligned && page_size % 32 == 0 && (ring % 32 == 0) &&
                      (row_bytes == 64 || row_bytes == 128 || row_bytes == 256 || row_bytes == 512);
    if (fused && !fast) return -1;
    const FusedArgs fa = fused ? *fused : FusedArgs{};
    const int budget = l2_prefetch_bytes();
#define FAST(LPR, GH)                                                                                             \
    do {                                                                                                          \
        grid.y = (unsigned)(nkv * ((group + GH - 1) / GH));                                                       \
        if (grid.y > 65535) return (int)cudaErrorInvalidValue;                                                    \
        if (fused)                                                                                                \
            rc = launch_pdl(attn_decode_fast_kernel<T, LPR, GH, true>, grid, WARPS * 32, 0, stream, (const T*)q,  \
                            (const T*)k_cache, (const T*)v_cache, partial, seq_of_token, pos, slots, tables,      \
                            table_stride, ring, page_size, num_pages, nh, nkv, window, scale, status, fa, budget); \
        else                                                                                                      \
            rc = launch_pdl(attn_decode_fast_kernel<T, LPR, GH, false>, grid, WARPS * 32, 0, stream, (const T*)q, \
                            (const T*)k_cache, (const T*)v_cache, partial, seq_of_token, pos, slots, tables,      \
                            table_stride, ring, page_size, num_pages, nh, nkv, window, scale, status, fa, budget); \
    } while (0)
#define FAST_G(LPR)                  \
    do {                             \
        if (group == 1)              \
            FAST(LPR, 1);            \
        else                         \
            FAST(LPR, 2);            \
    } while (0)
    int rc = 0;
    if (fast) {
        switch (row_bytes / 16) {
            case 4: FAST_G(4); break;
            case 8: FAST_G(8); break;
            case 16: FAST_G(16); break;
            default: FAST_G(32); break;
        }
    } else {
        const size_t smem = ((size_t)GHS * hd + (size_t)WARPS * GHS * (hd + 2)) * sizeof(float);
        rc = launch_pdl(attn_decode_rows_kernel<T>, grid, WARPS * 32, smem, stream, (const T*)q, (const T*)k_cache,
                        (const T*)v_cache, partial, seq_of_token, pos, slots, tables, table_stride, ring, page_size,
                        num_pages, nh, nkv, hd, window, scale, status);
    }
#undef FAST
#undef FAST_G
    if (fused || rc) return rc;
    return launch_pdl(attn_decode_merge_kernel<T>, dim3(num_tokens, nh), 128, 0, stream, (const float*)partial, (T*)out,
                      seq_of_token, nh, hd, nsplit);
}

}  // namespace

// A step of ONE token per sequence in one launch: rotation of the step's q/k/v rows, the append
// of key and value to the cache, the attention split along the keys, and the merge of the splits.
//   qkv: [T, (nh + 2 nkv) * hd] 32-bit with biases added; inv_freq: [rot / 2];
//   tickets: T * nkv ints, zero before the call (the kernel leaves them zero);
//   partial: T * nh * nsplit * (hd + 2) floats of scratch; out: [T, nh * hd].
// Returns -1 (nothing launched) for a head size the fast kernel does not take: the caller then
// uses moe_rope_commit and moe_attention_decode.
MOE_API int moe_attention_decode_fused(const float* qkv, const float* inv_freq, int rot, void* k_cache, void* v_cache,
                                       void* out, float* partial, int* tickets, int dt, const int* seq_of_token,
                                       const int* pos, const int* slots, const int* tables, int table_stride,
                                       int ring, int page_size, int num_pages, int num_tokens, int nh, int nkv, int hd,
                                       int window, float scale, int nsplit, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hd % 16 != 0 || hd > MAX_HD || hd <= 0 || nkv <= 0 || nh % nkv != 0 || nsplit < 1 || nsplit > 65535 ||
        nkv > 65535 || num_tokens > 65535 || rot < 0 || rot > hd || (rot & 1) || (rot > 0 && !inv_freq) || !tickets)
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16) return -1;
    FusedArgs fa;
    fa.qkv = qkv, fa.inv_freq = inv_freq, fa.rot = rot, fa.k_append = k_cache, fa.v_append = v_cache, fa.out = out;
    fa.tickets = tickets;
    if (dt == DT_F32)
        return launch<float>(nullptr, k_cache, v_cache, out, partial, seq_of_token, pos, slots, tables, table_stride,
                             ring, page_size, num_pages, num_tokens, nh, nkv, hd, window, scale, nsplit, status,
                             stream, &fa);
    return launch<__nv_bfloat16>(nullptr, k_cache, v_cache, out, partial, seq_of_token, pos, slots, tables,
                                 table_stride, ring, page_size, num_pages, num_tokens, nh, nkv, hd, window, scale,
                                 nsplit, status, stream, &fa);
}

// q: [T, nh, hd]; out: [T, nh * hd]; partial: T * nh * nsplit * (hd + 2) floats of scratch.
MOE_API int moe_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* partial,
                                 int dt, const int* seq_of_token, const int* pos, const int* slots,
                                 const int* tables, int table_stride, int ring, int page_size, int num_pages,
                                 int num_tokens, int nh, int nkv, int hd, int window, float scale, int nsplit,
                                 int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hd % 16 != 0 || hd > MAX_HD || hd <= 0 || nkv <= 0 || nh <= 0 || nh > 65535 || nh % nkv != 0 || nsplit < 1 ||
        nsplit > 65535 || nkv > 65535 || num_tokens > 65535 || !q || !k_cache || !v_cache || !out || !partial)
        return (int)cudaErrorInvalidValue;
    // cache rows are read 16 bytes at a time; q and out at least by whole elements
    if (((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 || ((uintptr_t)q | (uintptr_t)out) % (dt == DT_F32 ? 4 : 2))
        return (int)cudaErrorInvalidValue;
    if (dt == DT_F32)
        return launch<float>(q, k_cache, v_cache, out, partial, seq_of_token, pos, slots, tables, table_stride, ring,
                             page_size, num_pages, num_tokens, nh, nkv, hd, window, scale, nsplit, status, stream);
    return launch<__nv_bfloat16>(q, k_cache, v_cache, out, partial, seq_of_token, pos, slots, tables, table_stride,
                                 ring, page_size, num_pages, num_tokens, nh, nkv, hd, window, scale, nsplit, status,
                                 stream);
}

// ---- the entry point that allocates nothing (see attention_decode_noalloc.h) -----------------
#include "attention_decode_noalloc.h"

#include <mutex>

namespace {

// Scratch for the per-split partial results.  In host code this name is only a handle for
// cudaGetSymbolAddress; the kernels are given the device address obtained below.
static __device__ __align__(256) float g_noalloc_scratch[MOE_NOALLOC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_ptr[MAX_DEVICES] = {};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device; looked up once per device.
float* noalloc_scratch() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_scratch_ptr[dev] = static_cast<float*>(p);
    }
    return g_scratch_ptr[dev];
}

}  // namespace

MOE_API long long moe_attention_decode_noalloc_need(int num_tokens, int num_heads, int head_dim, int nsplit) {
    // each factor is bounded (65535, 65535, 65535, MAX_HD + 2) only by the entry point's own checks, so the
    // product is formed step by step and reported as "too many" (-1) once it leaves what the array could hold
    if (num_tokens <= 0 || num_heads <= 0 || head_dim <= 0 || nsplit <= 0) return -1;
    const long long cap = (long long)MOE_NOALLOC_SCRATCH_FLOATS * 4;
    long long n = num_tokens;
    n *= num_heads;
    if (n > cap) return -1;
    n *= nsplit;
    if (n > cap) return -1;
    n *= (long long)head_dim + 2;
    return n;
}

MOE_API const char* moe_noalloc_strerror(int code) {
    switch (code) {
        case MOE_NOALLOC_OK: return "ok";
        case MOE_NOALLOC_TOO_LARGE:
            return "the call needs more than the 2M floats (8 MiB) of scratch built into the library; "
                   "use fewer key splits or fewer tokens per call, or the entry point that takes scratch";
        case MOE_NOALLOC_BAD_ARGUMENT: return "a size or head layout the decode attention kernels do not take";
        case MOE_NOALLOC_NO_DEVICE: return "the device address of the built-in scratch array could not be obtained";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown code";
    }
}

MOE_API int moe_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, int dt,
                                         const int* seq_of_token, const int* pos, const int* slots,
                                         const int* tables, int table_stride, int ring, int page_size, int num_pages,
                                         int num_tokens, int num_heads, int num_kv_heads, int head_dim, int window,
                                         float scale, int nsplit, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return MOE_NOALLOC_OK;
    if (head_dim % 16 != 0 || head_dim > MAX_HD || head_dim <= 0 || num_kv_heads <= 0 || num_heads <= 0 ||
        num_heads > 65535 || num_heads % num_kv_heads != 0 || nsplit < 1 || nsplit > 65535 || num_kv_heads > 65535 ||
        num_tokens > 65535 || (dt != DT_F32 && dt != DT_BF16))
        return MOE_NOALLOC_BAD_ARGUMENT;
    const long long need = moe_attention_decode_noalloc_need(num_tokens, num_heads, head_dim, nsplit);
    if (need < 0 || need > MOE_NOALLOC_SCRATCH_FLOATS) return MOE_NOALLOC_TOO_LARGE;
    // Missing or misaligned memory is refused here, on the host, so that it never reaches the device: the
    // cache is read 16 bytes at a time by every kernel; q and out must at least be aligned to their
    // elements (a q that is not 16-byte aligned is served by the slower kernel that reads it element by
    // element).
    if (!q || !k_cache || !v_cache || !out || !seq_of_token || !pos || !slots || !tables) return MOE_NOALLOC_BAD_ARGUMENT;
    if (((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 || ((uintptr_t)q | (uintptr_t)out) % (dt == DT_F32 ? 4 : 2))
        return MOE_NOALLOC_BAD_ARGUMENT;
    float* scratch = noalloc_scratch();
    if (!scratch) return MOE_NOALLOC_NO_DEVICE;
    if (dt == DT_F32)
        return launch<float>(q, k_cache, v_cache, out, scratch, seq_of_token, pos, slots, tables, table_stride, ring,
                             page_size, num_pages, num_tokens, num_heads, num_kv_heads, head_dim, window, scale,
                             nsplit, status, stream);
    return launch<__nv_bfloat16>(q, k_cache, v_cache, out, scratch, seq_of_token, pos, slots, tables, table_stride,
                                 ring, page_size, num_pages, num_tokens, num_heads, num_kv_heads, head_dim, window,
                                 scale, nsplit, status, stream);
}
