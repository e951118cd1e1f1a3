// Attention of this step's queries over the cache and the step's own keys, tiled through shared
// memory: 64 queries of one (sequence, head) against key tiles of 64, on the CUDA cores in 32-bit.
//
// Same formulas and the same sources of keys as attention_generic.cu (reference:
// src/model.rs:794-827): keys before the step come from the paged cache, those of the step from
// k_new / v_new (use_local), or all from the cache (a layer that reads another layer's cache).
// Scores, the running maximum and sum and the weighted sum are float32 whatever the storage type.
//
// This is the kernel of the true 32-bit path for prompts, and in both dtypes of every step that
// the tensor-core kernels do not take: a prompt that goes on from the cache (chunks of a long
// prompt, steps that mix continued and fresh sequences) and head sizes other than theirs.  Where
// attention_generic.cu fetches every key from global memory once per QUERY, a block here fetches it
// once per 64 queries: a 24,000-token prompt reads 64 times less.
//
// A block of 256 threads: thread (ty, tx), ty = tid / 16, tx = tid % 16, owns the scores of query
// rows 4 ty .. 4 ty + 3 against key columns 4 tx .. 4 tx + 3, and of the output the same rows and
// the head-dimension columns 4 tx + 64 i.  Q and K sit in shared memory transposed ([d][row]), so
// that both operands of the score product are read as float4; P goes through shared memory to
// every thread of its rows (in the keys' place, which keeps a block of heads of 128 at 103 KB: two
// to an SM).  Key tiles start at multiples of 64 = the page size, so a tile of
// cached keys is one contiguous [64][head_dim] block of one page.
#include "common.cuh"

namespace {

constexpr int BQ = 64, BK = 64, PAD = 4, THREADS = 256;

template <typename T>
__device__ __forceinline__ void load_chunk(const T* p, float* out);
template <>
__device__ __forceinline__ void load_chunk<float>(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
}
template <>
__device__ __forceinline__ void load_chunk<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    out[0] = __uint_as_float(v.x << 16), out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16), out[3] = __uint_as_float(v.y & 0xffff0000u);
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_tiled_kernel(const T* __restrict__ q, const T* __restrict__ k_new, const T* __restrict__ v_new,
                  const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start, const int* __restrict__ slots,
                  const int* __restrict__ tables, int table_stride, int ring, int num_pages, int num_seqs, int nh,
                  int nkv, int hd, int window, float scale, int use_local, int* status) {
    extern __shared__ __align__(16) float sm[];
    __shared__ int s_seq, s_tile;
    float* Qt = sm;                               // [hd][BQ + PAD]
    float* Kt = Qt + (size_t)hd * (BQ + PAD);     // [hd][BK + PAD]
    float* V = Kt + (size_t)hd * (BK + PAD);      // [BK][hd + PAD]
    float* P = Kt;                                // [BQ][BK + PAD]: in the keys' place, once the scores are formed
                                                  // (hd >= 64; smaller heads get room of their own behind V)
    if (hd < BQ) P = V + (size_t)BK * (hd + PAD);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int h = blockIdx.y, kvh = h / (nh / nkv);

    // which (sequence, tile of 64 of its new tokens): tiles are numbered sequence by sequence
    if (tid == 0) {
        int tile = blockIdx.x, seq = -1;
        for (int s = 0; s < num_seqs; s++) {
            const int tiles = (cu_seqlens[s + 1] - cu_seqlens[s] + BQ - 1) / BQ;
            if (tile < tiles) {
                seq = s;
                break;
            }
            tile -= tiles;
        }
        s_seq = seq, s_tile = tile;
    }
    __syncthreads();
    const int seq = s_seq;
    if (seq < 0) return;
    const int tok0 = cu_seqlens[seq], cnt = cu_seqlens[seq + 1] - tok0, start = seq_start[seq];
    const int r0 = s_tile * BQ;                                    // first new token of the tile (within the step)
    const int rows = min(BQ, cnt - r0);
    const int p_first = start + r0, p_last = p_first + rows - 1;   // positions of the tile's queries
    const int local_from = use_local ? start : p_last + 1;         // positions from here on come from k_new / v_new
    const int lo_min = window > 0 ? max(0, p_first + 1 - window) : 0;
    const int* table = tables + (size_t)slots[seq] * table_stride;
    const int QS = BQ + PAD, KS = BK + PAD, VS = hd + PAD, PS = BK + PAD;

    // ---- the queries, transposed --------------------------------------------------------------
    for (int idx = tid; idx < BQ * (hd / 4); idx += THREADS) {
        const int r = idx / (hd / 4), d = (idx % (hd / 4)) * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < rows) load_chunk<T>(q + ((size_t)(tok0 + r0 + r) * nh + h) * hd + d, v);
#pragma unroll
        for (int e = 0; e < 4; e++) Qt[(size_t)(d + e) * QS + r] = v[e];
    }

    float m[4], l[4], o[4][16];          // running maximum and sum of this thread's rows; its part of the output
#pragma unroll
    for (int r = 0; r < 4; r++) {
        m[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++) o[r][i] = 0.f;
    }
    const int ncol = hd / 64 + (hd % 64 ? 1 : 0);      // float4 column groups of the output per thread: d = 4 tx + 64 i

    for (int j0 = (lo_min / BK) * BK; j0 <= p_last; j0 += BK) {
        __syncthreads();                 // the previous tile's K, V and P are no longer read
        // ---- a tile of keys (transposed) and values -------------------------------------------
        for (int idx = tid; idx < BK * (hd / 4); idx += THREADS) {
            const int c = idx / (hd / 4), d = (idx % (hd / 4)) * 4;
            const int j = j0 + c;
            float kv[4] = {0.f, 0.f, 0.f, 0.f}, vv[4] = {0.f, 0.f, 0.f, 0.f};
            if (j <= p_last && j >= lo_min) {
                if (j >= local_from) {
                    const size_t at = ((size_t)(tok0 + (j - start)) * nkv + kvh) * hd + d;
                    load_chunk<T>(k_new + at, kv);
                    load_chunk<T>(v_new + at, vv);
                } else {
                    const CachePos cp = cache_pos(j, ring, table, BK, num_pages, status);
                    const size_t at = cache_index(cp, kvh, nkv, BK, hd) + d;
                    load_chunk<T>(k_cache + at, kv);
                    load_chunk<T>(v_cache + at, vv);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; e++) Kt[(size_t)(d + e) * KS + c] = kv[e];
            *reinterpret_cast<float4*>(V + (size_t)c * VS + d) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        }
        __syncthreads();
        // ---- scores of 4 rows x 4 columns -----------------------------------------------------
        float s[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) s[r][c] = 0.f;
#pragma unroll 4
        for (int d = 0; d < hd; d++) {
            const float4 a = *reinterpret_cast<const float4*>(Qt + (size_t)d * QS + ty * 4);
            const float4 b = *reinterpret_cast<const float4*>(Kt + (size_t)d * KS + tx * 4);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) s[r][c] = fmaf(av[r], bv[c], s[r][c]);
        }
        // ---- mask, running maximum and sum, P --------------------------------------------------
        __syncthreads();                 // every thread has read the keys: P may take their place
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int row = ty * 4 + r, p = p_first + row;
            const int lo = window > 0 ? max(0, p + 1 - window) : 0;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int j = j0 + tx * 4 + c;
                const bool seen = row < rows && j <= p && j >= lo;
                s[r][c] = seen ? s[r][c] * scale : -INFINITY;
                mx = fmaxf(mx, s[r][c]);
            }
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m[r], mx);
            float alpha = 1.f, sum = 0.f, pr[4] = {0.f, 0.f, 0.f, 0.f};
            if (m_new != -INFINITY) {                    // (the same for the 16 threads of the row)
                alpha = m[r] == -INFINITY ? 0.f : expf(m[r] - m_new);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    pr[c] = s[r][c] == -INFINITY ? 0.f : expf(s[r][c] - m_new);
                    sum += pr[c];
                }
            }
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            l[r] = l[r] * alpha + sum;
            m[r] = m_new;
#pragma unroll
            for (int i = 0; i < 16; i++) o[r][i] *= alpha;
            *reinterpret_cast<float4*>(P + (size_t)row * PS + tx * 4) = make_float4(pr[0], pr[1], pr[2], pr[3]);
        }
        __syncthreads();
        // ---- output rows += P V -----------------------------------------------------------------
        for (int c0 = 0; c0 < BK; c0 += 4) {
            float pv[4][4];
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const float4 t4 = *reinterpret_cast<const float4*>(P + (size_t)(ty * 4 + r) * PS + c0);
                pv[r][0] = t4.x, pv[r][1] = t4.y, pv[r][2] = t4.z, pv[r][3] = t4.w;
            }
#pragma unroll
            for (int c = 0; c < 4; c++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (i >= ncol) break;
                    const int d = tx * 4 + 64 * i;
                    if (d >= hd) break;
                    const float4 v4 = *reinterpret_cast<const float4*>(V + (size_t)(c0 + c) * VS + d);
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        o[r][4 * i] = fmaf(pv[r][c], v4.x, o[r][4 * i]);
                        o[r][4 * i + 1] = fmaf(pv[r][c], v4.y, o[r][4 * i + 1]);
                        o[r][4 * i + 2] = fmaf(pv[r][c], v4.z, o[r][4 * i + 2]);
                        o[r][4 * i + 3] = fmaf(pv[r][c], v4.w, o[r][4 * i + 3]);
                    }
                }
            }
        }
    }
    // ---- normalise and store --------------------------------------------------------------------
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int row = ty * 4 + r;
        if (row >= rows) continue;
        const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
        T* dst = out + ((size_t)(tok0 + r0 + row) * nh + h) * hd;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = tx * 4 + 64 * i;
            if (i >= ncol || d >= hd) break;
#pragma unroll
            for (int e = 0; e < 4; e++) st_f(dst + d + e, o[r][4 * i + e] * inv);
        }
    }
}

size_t tiled_smem(int hd) {
    // Q, K (P takes K's place when the head is at least as long as a tile is wide), V
    return ((size_t)hd * (BQ + PAD) + (size_t)hd * (BK + PAD) + (size_t)BK * (hd + PAD) +
            (hd < BQ ? (size_t)BQ * (BK + PAD) : 0)) * sizeof(float);
}

}  // namespace

// Same arguments as moe_attention_generic, without the per-token arrays (a block finds its rows from
// cu_seqlens).  The page size must be 64.  Rows of no sequence (a padded step) are not written.
// Returns -1 (nothing launched) for sizes this kernel does not take: the caller uses the plain kernel.
MOE_API int moe_attention_tiled(const void* q, const void* k_new, const void* v_new, const void* k_cache,
                                const void* v_cache, void* out, int dt, const int* cu_seqlens, const int* seq_start,
                                const int* slots, const int* tables, int table_stride, int ring, int page_size,
                                int num_pages, int num_seqs, int num_tokens, int nh, int nkv, int hd, int window,
                                float scale, int use_local, int* status, cudaStream_t stream) {
    if (num_tokens <= 0 || num_seqs <= 0) return 0;
    if (hd % 16 != 0 || hd > 256 || hd <= 0 || nkv <= 0 || nh % nkv != 0 || nh > 65535) return (int)cudaErrorInvalidValue;
    if (page_size != BK || (ring % BK) != 0) return -1;
    const size_t align = dt == DT_F32 ? 16 : 8;          // rows are read four elements at a time
    if (((uintptr_t)q | (uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_cache | (uintptr_t)v_cache) % align) return -1;
    const size_t smem = tiled_smem(hd);
    const long long tiles = (long long)(num_tokens + BQ - 1) / BQ + num_seqs;
    if (tiles > 0x7fffffffLL) return -1;
    dim3 grid((unsigned)tiles, nh);
#define GO(TT)                                                                                                        \
    do {                                                                                                              \
        static size_t configured = 0;                                                                                 \
        if (smem > 48 * 1024 && smem > configured) {                                                                  \
            cudaError_t e = cudaFuncSetAttribute(attn_tiled_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                      \
            configured = smem;                                                                                        \
        }                                                                                                             \
        attn_tiled_kernel<TT><<<grid, THREADS, smem, stream>>>(                                                       \
            (const TT*)q, (const TT*)k_new, (const TT*)v_new, (const TT*)k_cache, (const TT*)v_cache, (TT*)out,       \
            cu_seqlens, seq_start, slots, tables, table_stride, ring, num_pages, num_seqs, nh, nkv, hd, window, scale, \
            use_local, status);                                                                                       \
    } while (0)
    if (dt == DT_F32)
        GO(float);
    else
        GO(__nv_bfloat16);
#undef GO
    return launch_status();
}
