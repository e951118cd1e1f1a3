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

// LPR: lanes per key row (row bytes / 16); GH: query heads handled together.
template <typename T, int LPR, int GH>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_fast_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        float* __restrict__ partial, const int* __restrict__ seq_of_token,
                        const int* __restrict__ pos, const int* __restrict__ slots, const int* __restrict__ tables,
                        int table_stride, int ring, int page_size, int num_pages, int nh, int nkv, int window,
                        float scale, int* status) {
    constexpr int EPC = Chunk<T>::N;       // elements per 16-byte chunk
    constexpr int HD = LPR * EPC;
    constexpr int RPI = 32 / LPR;          // rows per load instruction
    constexpr int NI = LPR;                // load instructions per tile of 32 rows
    constexpr int REC = HD + 2;
    __shared__ float red[WARPS][GH][REC];
    pdl_sync();

    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rgrp = lane / LPR;
    const int group = nh / nkv;
    const int s = seq_of_token[t];
    if (s < 0) return;                                   // padding row: the merge kernel writes zeros
    const int p = pos[t];
    const int lo = window > 0 ? max(0, p + 1 - window) : 0;
    // tiles of 32 positions, aligned to 32: the keys of a tile are contiguous in one page
    const int tile_lo = lo / 32, tile_hi = p / 32 + 1;
    const int tps = (tile_hi - tile_lo + nsplit - 1) / nsplit;
    const int tb = tile_lo + split * tps, te = min(tile_hi, tb + tps);
    const int* table = tables + (size_t)slots[s] * table_stride;

    for (int h0 = 0; h0 < group; h0 += GH) {
        const int gh = min(GH, group - h0);
        float qc[GH][EPC];
#pragma unroll
        for (int g = 0; g < GH; g++) {
            if (g < gh)
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
            const bool valid = my_j >= lo && my_j <= p;
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
                    if (j >= lo && j <= p) {
                        float vc[EPC];
                        Chunk<T>::unpack(raw[i], vc);
#pragma unroll
                        for (int e = 0; e < EPC; e++) acc[g][e] = fmaf(pi, vc[e], acc[g][e]);
                    }
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

template <typename T>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, float* partial,
           const int* seq_of_token, const int* pos, const int* slots, const int* tables, int table_stride, int ring,
           int page_size, int num_pages, int num_tokens, int nh, int nkv, int hd, int window, float scale, int nsplit,
           int* status, cudaStream_t stream) {
    dim3 grid(nsplit, nkv, num_tokens);
    const int group = nh / nkv;
    const int row_bytes = hd * (int)sizeof(T);
    const bool fast = page_size % 32 == 0 && (ring % 32 == 0) &&
                      (row_bytes == 64 || row_bytes == 128 || row_bytes == 256 || row_bytes == 512);
#define FAST(LPR, GH)                                                                                          \
    launch_pdl(attn_decode_fast_kernel<T, LPR, GH>, grid, WARPS * 32, 0, stream, (const T*)q, (const T*)k_cache, \
               (const T*)v_cache, partial, seq_of_token, pos, slots, tables, table_stride, ring, page_size,      \
               num_pages, nh, nkv, window, scale, status)
#define FAST_G(LPR)                  \
    do {                             \
        if (group == 1)              \
            FAST(LPR, 1);            \
        else                         \
            FAST(LPR, 2);            \
    } while (0)
    if (fast) {
        switch (row_bytes / 16) {
            case 4: FAST_G(4); break;
            case 8: FAST_G(8); break;
            case 16: FAST_G(16); break;
            default: FAST_G(32); break;
        }
    } else {
        const size_t smem = ((size_t)GHS * hd + (size_t)WARPS * GHS * (hd + 2)) * sizeof(float);
        launch_pdl(attn_decode_rows_kernel<T>, grid, WARPS * 32, smem, stream, (const T*)q, (const T*)k_cache,
                   (const T*)v_cache, partial, seq_of_token, pos, slots, tables, table_stride, ring, page_size,
                   num_pages, nh, nkv, hd, window, scale, status);
    }
#undef FAST
#undef FAST_G
    return launch_pdl(attn_decode_merge_kernel<T>, dim3(num_tokens, nh), 128, 0, stream, (const float*)partial, (T*)out,
                      seq_of_token, nh, hd, nsplit);
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
    return (long long)num_tokens * num_heads * nsplit * (head_dim + 2);
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
    if (head_dim % 16 != 0 || head_dim > MAX_HD || head_dim <= 0 || num_kv_heads <= 0 ||
        num_heads % num_kv_heads != 0 || nsplit < 1 || nsplit > 65535 || num_kv_heads > 65535 || num_tokens > 65535 ||
        (dt != DT_F32 && dt != DT_BF16))
        return MOE_NOALLOC_BAD_ARGUMENT;
    if (moe_attention_decode_noalloc_need(num_tokens, num_heads, head_dim, nsplit) > MOE_NOALLOC_SCRATCH_FLOATS)
        return MOE_NOALLOC_TOO_LARGE;
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
