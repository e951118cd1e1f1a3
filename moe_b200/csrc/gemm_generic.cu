// The plain matrix product of the library: C[m, n] = sum_k A[row(m), k] * W[g][n, k] (+ bias[n]).
//
// Every projection of the model is stored [out_features, in_features] row-major
// and applied as y = W x (reference: src/quant.rs:476-506).  This kernel is the
// true 32-bit path (FFMA on CUDA cores, k ascending, no reduced-precision matrix
// mode) and the fallback of the bfloat16 path for shapes and dtypes the
// tensor-core kernels refuse.  It takes any M, N, K.
//
//   * rows of A may be gathered through `a_rows` (expert dispatch);
//   * rows may be partitioned into groups by `group_offsets[G+1]`, group g using
//     the weight slab W + g * w_group_stride (routed experts).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec_ok, int valid, float* out);

template <>
__device__ __forceinline__ void load4<float>(const float* p, bool vec_ok, int valid, float* out) {
    if (vec_ok && valid == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x, out[1] = v.y, out[2] = v.z, out[3] = v.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = i < valid ? p[i] : 0.f;
    }
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool vec_ok, int valid, float* out) {
    if (vec_ok && valid == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        out[0] = __uint_as_float(v.x << 16), out[1] = __uint_as_float(v.x & 0xffff0000u);
        out[2] = __uint_as_float(v.y << 16), out[3] = __uint_as_float(v.y & 0xffff0000u);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = i < valid ? __bfloat162float(p[i]) : 0.f;
    }
}

template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(THREADS)
gemm_generic_kernel(const AT* __restrict__ A, int lda, const int* __restrict__ a_rows, int a_src_rows,
                    const WT* __restrict__ W, long long w_group_stride, OT* __restrict__ C, int ldc,
                    const float* __restrict__ bias, const int* __restrict__ group_offsets, int num_groups, int M,
                    int N, int K, int a_vec_ok, int w_vec_ok, int* status) {
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Ws[BK][BN + 4];
    __shared__ int s_group, s_row0, s_row1;

    // which group and which 64-row tile of it this block owns
    if (threadIdx.x == 0) {
        int g = 0, r0 = 0, r1 = M;
        int tile = blockIdx.y;
        if (group_offsets) {
            g = -1;
            for (int i = 0; i < num_groups; i++) {
                const int b = group_offsets[i], e = group_offsets[i + 1];
                const int tiles = (e - b + BM - 1) / BM;
                if (tile < tiles) {
                    g = i, r0 = b + tile * BM, r1 = e;
                    break;
                }
                tile -= tiles;
            }
        } else {
            r0 = tile * BM;
            if (r0 >= M) g = -1;
        }
        s_group = g, s_row0 = r0, s_row1 = r1;
    }
    __syncthreads();
    const int g = s_group;
    if (g < 0) return;
    const int row0 = s_row0, row_end = s_row1;
    const int n0 = blockIdx.x * BN;
    const WT* Wg = W + (size_t)g * (size_t)w_group_stride;

    const int tid = threadIdx.x;
    const int lr = tid >> 2;         // 0..63: row of the tile this thread loads
    const int lk = (tid & 3) * 4;    // 0,4,8,12: first k it loads
    const int ty = tid >> 4, tx = tid & 15;

    // source row of A for the row this thread loads
    const int arow = row0 + lr;
    long long a_src = -1;
    if (arow < row_end) {
        a_src = a_rows ? a_rows[arow] : arow;
        if (a_src < 0 || a_src >= a_src_rows) {
            atomicOr(status, ST_BAD_ROW);
            a_src = -1;
        }
    }
    const int wrow = n0 + lr;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4], wv[4];
        const int k = k0 + lk;
        int valid = K - k;
        valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
        if (a_src >= 0 && valid > 0)
            load4<AT>(A + (size_t)a_src * lda + k, a_vec_ok, valid, av);
        else
            av[0] = av[1] = av[2] = av[3] = 0.f;
        if (wrow < N && valid > 0)
            load4<WT>(Wg + (size_t)wrow * K + k, w_vec_ok, valid, wv);
        else
            wv[0] = wv[1] = wv[2] = wv[3] = 0.f;
        __syncthreads();   // previous tile fully consumed
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lk + i][lr] = av[i];
            Ws[lk + i][lr] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float ar[4] = {a.x, a.y, a.z, a.w};
            const float br[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = row0 + ty * 4 + i;
        if (r >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = n0 + tx * 4 + j;
            if (c >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[c];
            st_f(C + (size_t)r * ldc + c, v);
        }
    }
}

// The same product for FEW rows (a step of one token per sequence): the time is the weight stream.
// A block takes 64 output features and up to RT rows of A; chunk by chunk of KC k it brings the
// weights [64][KC] (coalesced, 16 bytes a thread) and the rows [RT][KC] into shared memory, and
// thread (feature f, row pair) walks the chunk with ONE accumulator per output, k ascending: the very
// order of the tile kernel above, so that a token's product is the same to the bit whether it comes
// alone (a decode step) or among thousands (a prompt).  Groups and gathered rows as above, in tiles
// of RT rows.
constexpr int RT = 8, RF = 64, KC = 128, WS = KC + 4, RTHREADS = 256;

template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(RTHREADS)
gemm_rows_kernel(const AT* __restrict__ A, int lda, const int* __restrict__ a_rows, int a_src_rows,
                 const WT* __restrict__ W, long long w_group_stride, OT* __restrict__ C, int ldc,
                 const float* __restrict__ bias, const int* __restrict__ group_offsets, int num_groups, int M, int N,
                 int K, int a_vec_ok, int w_vec_ok, int* status) {
    __shared__ __align__(16) float Ws[RF][WS];
    __shared__ __align__(16) float As[RT][KC];
    __shared__ int s_group, s_row0, s_row1;
    __shared__ long long s_src[RT];
    if (threadIdx.x == 0) {
        int g = 0, r0 = 0, r1 = M;
        int tile = blockIdx.y;
        if (group_offsets) {
            g = -1;
            for (int i = 0; i < num_groups; i++) {
                const int b = group_offsets[i], e = group_offsets[i + 1];
                const int tiles = (e - b + RT - 1) / RT;
                if (tile < tiles) {
                    g = i, r0 = b + tile * RT, r1 = e;
                    break;
                }
                tile -= tiles;
            }
        } else {
            r0 = tile * RT;
            if (r0 >= M) g = -1;
        }
        s_group = g, s_row0 = r0, s_row1 = r1;
    }
    __syncthreads();
    const int g = s_group;
    if (g < 0) return;
    const int row0 = s_row0, rows = min(RT, s_row1 - row0);
    if (threadIdx.x < RT) {
        long long src = -1;
        if ((int)threadIdx.x < rows) {
            src = a_rows ? a_rows[row0 + threadIdx.x] : row0 + threadIdx.x;
            if (src < 0 || src >= a_src_rows) {
                atomicOr(status, ST_BAD_ROW);
                src = -1;
            }
        }
        s_src[threadIdx.x] = src;
    }
    const int tid = threadIdx.x, f = tid % RF, rg = tid / RF;      // this thread's feature and pair of rows
    const int n0 = blockIdx.x * RF;
    const WT* Wg = W + (size_t)g * (size_t)w_group_stride;
    float acc0 = 0.f, acc1 = 0.f;

    // A chunk's loads are issued one chunk ahead, into registers, and so are in flight while the
    // chunk before it is multiplied.
    constexpr int WPT = RF * (KC / 4) / RTHREADS;      // 16-byte pieces of the weight chunk per thread
    float wr[WPT][4], ar[4];
    __syncthreads();                                   // s_src is written
    auto fetch = [&](int c0) {
        const int kc = min(KC, K - c0);
#pragma unroll
        for (int i = 0; i < WPT; i++) {
            const int idx = tid + i * RTHREADS, fl = idx / (KC / 4), k = (idx % (KC / 4)) * 4;
            const int valid = min(4, kc - k);
            wr[i][0] = wr[i][1] = wr[i][2] = wr[i][3] = 0.f;
            if (n0 + fl < N && valid > 0) load4<WT>(Wg + (size_t)(n0 + fl) * K + c0 + k, w_vec_ok, valid, wr[i]);
        }
        const int r = tid / (KC / 4), k = (tid % (KC / 4)) * 4;           // RT * KC / 4 == RTHREADS
        const long long src = s_src[r];
        const int valid = min(4, kc - k);
        ar[0] = ar[1] = ar[2] = ar[3] = 0.f;
        if (src >= 0 && valid > 0) load4<AT>(A + (size_t)src * lda + c0 + k, a_vec_ok, valid, ar);
    };
    if (K > 0) fetch(0);
    for (int c0 = 0; c0 < K; c0 += KC) {
        const int kc = min(KC, K - c0);
        __syncthreads();              // the previous chunk is no longer read
#pragma unroll
        for (int i = 0; i < WPT; i++) {
            const int idx = tid + i * RTHREADS, fl = idx / (KC / 4), k = (idx % (KC / 4)) * 4;
            *reinterpret_cast<float4*>(&Ws[fl][k]) = make_float4(wr[i][0], wr[i][1], wr[i][2], wr[i][3]);
        }
        *reinterpret_cast<float4*>(&As[tid / (KC / 4)][(tid % (KC / 4)) * 4]) = make_float4(ar[0], ar[1], ar[2], ar[3]);
        __syncthreads();
        if (c0 + KC < K) fetch(c0 + KC);
#pragma unroll 8
        for (int k = 0; k < KC; k += 4) {
            if (k >= kc) break;       // (a chunk's tail is zero anyway; this only saves the work)
            const float4 w = *reinterpret_cast<const float4*>(&Ws[f][k]);
            const float4 a = *reinterpret_cast<const float4*>(&As[2 * rg][k]);
            const float4 b = *reinterpret_cast<const float4*>(&As[2 * rg + 1][k]);
            acc0 = fmaf(a.x, w.x, acc0), acc0 = fmaf(a.y, w.y, acc0), acc0 = fmaf(a.z, w.z, acc0), acc0 = fmaf(a.w, w.w, acc0);
            acc1 = fmaf(b.x, w.x, acc1), acc1 = fmaf(b.y, w.y, acc1), acc1 = fmaf(b.z, w.z, acc1), acc1 = fmaf(b.w, w.w, acc1);
        }
    }
    const int n = n0 + f;
    if (n < N) {
        const float bv = bias ? bias[n] : 0.f;
        if (2 * rg < rows) st_f(C + (size_t)(row0 + 2 * rg) * ldc + n, bias ? acc0 + bv : acc0);
        if (2 * rg + 1 < rows) st_f(C + (size_t)(row0 + 2 * rg + 1) * ldc + n, bias ? acc1 + bv : acc1);
    }
}
static_assert(RT * (KC / 4) == RTHREADS && RT == 2 * (RTHREADS / RF), "the thread layout of gemm_rows_kernel");

template <typename AT, typename WT, typename OT>
int launch(const void* A, int lda, const int* a_rows, int a_src_rows, const void* W, long long w_group_stride, void* C,
           int ldc, const float* bias, const int* group_offsets, int num_groups, int M, int N, int K, int* status,
           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const int a_vec = (K % 4 == 0) && (lda % 4 == 0) && ((uintptr_t)A % 16 == 0);
    const int w_vec = (K % 4 == 0) && ((uintptr_t)W % 16 == 0) && ((w_group_stride * (long long)sizeof(WT)) % 16 == 0);
    if (M <= (group_offsets ? 8 * RT : 2 * RT)) {
        // few rows: the weight stream is what takes the time
        const int r_tiles = group_offsets ? (M < num_groups ? M : num_groups) + M / RT : (M + RT - 1) / RT;
        dim3 rgrid((N + RF - 1) / RF, r_tiles);
        gemm_rows_kernel<AT, WT, OT><<<rgrid, RTHREADS, 0, stream>>>(
            (const AT*)A, lda, a_rows, a_src_rows, (const WT*)W, w_group_stride, (OT*)C, ldc, bias, group_offsets,
            num_groups, M, N, K, a_vec, w_vec, status);
        return launch_status();
    }
    const int m_tiles = (M + BM - 1) / BM + (group_offsets ? num_groups : 0);
    dim3 grid((N + BN - 1) / BN, m_tiles);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    gemm_generic_kernel<AT, WT, OT><<<grid, THREADS, 0, stream>>>(
        (const AT*)A, lda, a_rows, a_src_rows, (const WT*)W, w_group_stride, (OT*)C, ldc, bias, group_offsets,
        num_groups, M, N, K, a_vec, w_vec, status);
    return launch_status();
}

}  // namespace

// A: [*, lda] of a_dt; W: [G][N, K] of w_dt; C: [M, ldc] of c_dt.  `a_rows` (may be
// null) maps output row -> row of A; `a_src_rows` bounds it.  `group_offsets`
// (may be null) has num_groups + 1 entries on the device.
MOE_API int moe_gemm_generic(const void* A, int a_dt, int lda, const int* a_rows, int a_src_rows, const void* W,
                             int w_dt, long long w_group_stride, void* C, int c_dt, int ldc, const float* bias,
                             const int* group_offsets, int num_groups, int M, int N, int K, int* status,
                             cudaStream_t stream) {
#define GO(AT, WT, OT)                                                                                              \
    return launch<AT, WT, OT>(A, lda, a_rows, a_src_rows, W, w_group_stride, C, ldc, bias, group_offsets, num_groups, \
                              M, N, K, status, stream)
    typedef __nv_bfloat16 bf;
    if (a_dt == DT_F32 && w_dt == DT_F32 && c_dt == DT_F32) GO(float, float, float);
    if (a_dt == DT_F32 && w_dt == DT_F32 && c_dt == DT_BF16) GO(float, float, bf);
    if (a_dt == DT_F32 && w_dt == DT_BF16 && c_dt == DT_F32) GO(float, bf, float);
    if (a_dt == DT_F32 && w_dt == DT_BF16 && c_dt == DT_BF16) GO(float, bf, bf);
    if (a_dt == DT_BF16 && w_dt == DT_F32 && c_dt == DT_F32) GO(bf, float, float);
    if (a_dt == DT_BF16 && w_dt == DT_F32 && c_dt == DT_BF16) GO(bf, float, bf);
    if (a_dt == DT_BF16 && w_dt == DT_BF16 && c_dt == DT_F32) GO(bf, bf, float);
    if (a_dt == DT_BF16 && w_dt == DT_BF16 && c_dt == DT_BF16) GO(bf, bf, bf);
#undef GO
    return (int)cudaErrorInvalidValue;
}
