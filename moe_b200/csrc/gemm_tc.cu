// Tensor-core matrix product of the bfloat16 path: Y[t, n] = sum_k X[t, k] * W[n, k].
//
// Written for sm_100a: operands are brought into shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), multiplied by tcgen05.mma with the
// accumulator in tensor memory, and read back with tcgen05.ld for the epilogue.
//
// The WEIGHT is the M operand of the instruction (tiles of 128 output features)
// and the TOKENS are its N operand (tiles of 16 ... 256), so a decode step of a few
// tokens wastes no tensor-core rows and a prefill uses the widest shape.  One CTA
// computes one (feature tile, token tile[, K split]):
//
//   warp 0      TMA producer: W tile(s) [128 x 64] and X tile [BN x 64] per stage
//   warp 1      allocates tensor memory, issues the MMAs, commits to the barriers
//   warps 2-5   epilogue: tensor memory -> registers -> global memory
//
// Modes
//   PLAIN    out[t, n] = acc (+ bias[n]); out is float32 or bfloat16
//   SWIGLU   W holds gate rows [0, I) and up rows [I, 2I) per group; two accumulators;
//            out[t, j] = silu(gate) * up  (reference: src/model.rs:26-35)
// Groups (routed experts): rows of X are partitioned by group_offsets[G + 1]; group g
// uses the weight slab g.  Split K (few tokens, where the weight stream needs every SM):
// up to 8 splits of a tile form a thread-block cluster; each leaves its float32 partial
// tile in its own shared memory and CTA r of the cluster adds rows r, r + S, ... in split
// order, reading its peers through distributed shared memory.  More than 8 splits write
// their partials to scratch, and the CTA that arrives last at the tile's ticket adds them
// in split order.  Either way the sum does not depend on arrival order.
// Many tokens take the persistent form further down (gemm_tc_persistent_kernel).
//
// Every wait on a barrier is bounded.  A wait that runs out sets ST_WAIT_TIMEOUT in the
// status word and the CTA drains, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int TILE_W = 128;   // output features per CTA (UMMA M)
constexpr int BK = 64;        // K elements per stage = one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int MAX_SMEM_GROUPS = 256;
constexpr int MAX_SPLITS = 16;

// MODE_SWIGLU_IL (persistent form only): gate and up rows of the same 16 features alternate within a
// 128-row weight tile (see gemm_tc_persistent_kernel), so that SwiGLU needs ONE accumulator.
enum { MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_SWIGLU_IL = 2 };

struct Params {
    void* out;
    int out_bf16;
    int ldo;
    const float* bias;
    const int* group_offsets;   // null: one group of M rows
    int num_groups;
    int M;                      // rows of X in total
    int N;                      // output features per group (SWIGLU: the intermediate size I)
    int K;
    int w_rows_per_group;       // N, or 2 N for SWIGLU
    int splits;                 // K splits (>= 1), every split non-empty
    int kb_per_split;
    int cluster;                // 1: the splits of a tile are one cluster and add up through shared memory
    int early_offsets;          // 1: group_offsets were written at least two kernels ago (see the kernel)
    float* partials;            // [splits][M][cols] float32, cols = N or 2 N (not with cluster)
    int* tickets;               // one per (grid.y, grid.x), zero before and after the launch
    int* status;
    uint32_t wait_limit;        // microseconds a wait on a barrier may take (WAIT_LIMIT_US, less in the wait test)
    int test_fault;             // 0; the wait test: 1 = the producer loads nothing, 2 = no MMA is issued
};

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false if the barrier did not complete within limit_us microseconds (the site is then
// recorded in the status word) or another role of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit_us,
                                          int* status, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 1;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 0) {
            if (abort_flag && *abort_flag) return false;
            if (global_ns() - t0 > (unsigned long long)limit_us * 1000ull) break;
        }
    }
    wait_ran_out(status, site);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}
// ---- thread-block clusters (the K splits of one tile) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in the CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// ---- a pair of CTAs on one tile (cta_group::2) ----
// Both CTAs of the pair run these; allocation and release are mirrored in the two tensor memories.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// A tile load whose bytes are counted by a barrier of the pair's first CTA (bar: an address in the
// cluster's shared window, from mapa_cluster).  The data go to this CTA's own shared memory.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// D[256, N] (+)= A[256, 16] B[N, 16]^T over the pair: each CTA holds 128 rows of A and N / 2 rows of B
// at the same shared-memory offsets, and gets its 128 rows of D in its own tensor memory.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// When the pair's MMAs so far are done, arrive on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (SBO), descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 // leading byte offset (ignored with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
    d |= (uint64_t)1 << 46;                 // version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}

__host__ __device__ constexpr uint32_t instr_desc(int n, int m = TILE_W) {
    // c = f32 (1 << 4), a = bf16 (1 << 7), b = bf16 (1 << 10), both K-major, N >> 3 at 17, M >> 4 at 24
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int BN, int MODE>
struct Cfg {
    static constexpr int NW = MODE == MODE_SWIGLU ? 2 : 1;
    static constexpr int W_BYTES = TILE_W * BK * 2;
    static constexpr int X_BYTES = BN * BK * 2;
    static constexpr int XBOX = BN < 64 ? BN : 64;      // rows of one activation box
    static constexpr int STAGE_BYTES = NW * W_BYTES + X_BYTES;
    // few tokens: the weight stream bounds the time, and two CTAs per SM (each with fewer stages)
    // hide one CTA's set-up and epilogue behind the other's loads
    static constexpr int BUDGET = BN <= 64 ? (MODE == MODE_PLAIN ? 100 : 110) * 1024 : 196 * 1024;
    static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW < 2 ? 2 : STAGES_RAW);
    static constexpr int TMEM_COLS_RAW = NW * BN;
    static constexpr int TMEM_COLS = TMEM_COLS_RAW < 32 ? 32 : TMEM_COLS_RAW;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    // the partial tile of a K split fits in the (then free) pipeline stages
    static constexpr bool CLUSTER_OK = NW * BN * TILE_W * 4 <= STAGES * STAGE_BYTES;
};

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

template <int BN, int MODE>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
    using C = Cfg<BN, MODE>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_work[4];          // group, first row, end row, is_last
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_tmem;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TILE_W;
    const int split = blockIdx.z;

    // Programmatic dependent launch: this kernel may have been scheduled while its predecessor
    // still runs.  Weights never depend on the predecessor, so an ungrouped product sets itself up
    // and starts streaming its weight tiles before it waits (in the producer, below); a grouped one
    // needs the group offsets the predecessor wrote, and waits here.
    // A grouped one whose offsets are older than the predecessor (the second product of the routed
    // experts: its offsets were written before the first) may do the same.
    const bool grouped = p.group_offsets != nullptr;
    const bool wait_first = grouped && !p.early_offsets;
    if (wait_first) pdl_sync();

    // ---- which rows of X this CTA owns -------------------------------------------------
    // (the offsets are fetched by all threads at once: a scan straight from global memory would
    // pay one memory latency per group)
    __shared__ int s_offs[MAX_SMEM_GROUPS + 1];
    const bool offs_in_smem = p.group_offsets && p.num_groups <= MAX_SMEM_GROUPS;
    if (offs_in_smem) {
        for (int i = threadIdx.x; i <= p.num_groups; i += blockDim.x) s_offs[i] = p.group_offsets[i];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int g = 0, r0 = 0, r1 = p.M, tile = blockIdx.y;
        if (p.group_offsets) {
            g = -1;
            const int* offs = offs_in_smem ? s_offs : p.group_offsets;
            for (int i = 0; i < p.num_groups; i++) {
                const int b = offs[i], e = offs[i + 1];
                const int tiles = (e - b + BN - 1) / BN;
                if (tile < tiles) {
                    g = i, r0 = b + tile * BN, r1 = e;
                    break;
                }
                tile -= tiles;
            }
        } else {
            r0 = tile * BN;
            if (r0 >= p.M) g = -1;
        }
        s_work[0] = g, s_work[1] = r0, s_work[2] = r1, s_work[3] = 0;
        s_abort = 0;
    }
    __syncthreads();
    const int g = s_work[0];
    if (g < 0) return;                 // uniform: nothing to do for this tile index
    const int row0 = s_work[1], row_end = s_work[2];

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + C::STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    const uint32_t acc_bar = bar_base + 8u * (2 * C::STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int kb_total = (p.K + BK - 1) / BK;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(kb_total, kb0 + p.kb_per_split);
    const int w_row = g * p.w_rows_per_group + n0;
    // A tile with fewer than BN rows multiplies only as many tokens as it has (the MMA's N, in steps
    // of 16) and loads only the 64-row boxes of activations that hold them.
    constexpr int XBOX = C::XBOX;
    const int n_eff = min(BN, (min(BN, row_end - row0) + 15) & ~15);
    const int xchunks = (n_eff + XBOX - 1) / XBOX;
    const uint32_t stage_tx = C::NW * C::W_BYTES + xchunks * XBOX * BK * 2;
    auto load_x = [&](uint32_t st, int kb, uint32_t bar) {
        for (int c = 0; c < xchunks; c++)
            tma_load_2d(st + C::NW * C::W_BYTES + c * XBOX * BK * 2, &tmX, kb * BK, row0 + c * XBOX, bar);
    };

    if (warp == 0) {
        // ---- producer ---------------------------------------------------------------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            int kb_next = kb0;
            if (p.test_fault == 1) {
                if (!wait_first) pdl_sync();
                kb_next = kb1;                   // the wait test: nothing is loaded, the MMA issuer's wait runs out
            } else if (!wait_first) {
                // weight tiles of the first stages, then wait for the predecessor, then their activations
                const int pre = min(C::STAGES, kb1 - kb0);
                for (int i = 0; i < pre; i++) {
                    const uint32_t st = base + i * C::STAGE_BYTES;
                    mbar_expect_tx(full_bar(i), stage_tx);
                    tma_load_2d(st, &tmW, (kb0 + i) * BK, w_row, full_bar(i));
                    if (MODE == MODE_SWIGLU) tma_load_2d(st + C::W_BYTES, &tmW, (kb0 + i) * BK, w_row + p.N, full_bar(i));
                }
                pdl_sync();
                for (int i = 0; i < pre; i++) load_x(base + i * C::STAGE_BYTES, kb0 + i, full_bar(i));
                issued = pre;
                kb_next = kb0 + pre;
            }
            for (int kb = kb_next; kb < kb1 && ok; kb++, issued++) {
                const int s = issued % C::STAGES;
                const uint32_t ph = (issued / C::STAGES) & 1;
                ok = mbar_wait(empty_bar(s), ph ^ 1, &s_abort, p.wait_limit, p.status, 0x11);
                if (!ok) break;
                const uint32_t st = base + s * C::STAGE_BYTES;
                mbar_expect_tx(full_bar(s), stage_tx);
                tma_load_2d(st, &tmW, kb * BK, w_row, full_bar(s));
                if (MODE == MODE_SWIGLU) tma_load_2d(st + C::W_BYTES, &tmW, kb * BK, w_row + p.N, full_bar(s));
                load_x(st, kb, full_bar(s));
            }
            if (!ok) {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
                // copies already issued must land before the CTA may leave
                for (int i = max(0, issued - C::STAGES); i < issued; i++)
                    mbar_wait(full_bar(i % C::STAGES), (i / C::STAGES) & 1, nullptr, p.wait_limit, p.status, 0x12);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc(n_eff);
            const bool issue = p.test_fault != 2;   // the wait test: nothing is issued, producer and epilogue run out
            bool ok = true;
            int it = 0;
            for (int kb = kb0; kb < kb1 && issue; kb++, it++) {
                const int s = it % C::STAGES;
                ok = mbar_wait(full_bar(s), (it / C::STAGES) & 1, &s_abort, p.wait_limit, p.status, 0x14);
                if (!ok) break;
                tc_fence_after();
                const uint32_t st = base + s * C::STAGE_BYTES;
#pragma unroll
                for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                    const uint32_t koff = k4 * UMMA_K * 2;
                    const uint64_t bdesc = smem_desc(st + C::NW * C::W_BYTES + koff);
                    const uint32_t acc = (it > 0 || k4 > 0) ? 1u : 0u;
                    umma_bf16(tmem, smem_desc(st + koff), bdesc, idesc, acc);
                    if (MODE == MODE_SWIGLU) umma_bf16(tmem + BN, smem_desc(st + C::W_BYTES + koff), bdesc, idesc, acc);
                }
                umma_commit(empty_bar(s));      // frees the stage when these MMAs have read it
            }
            if (!issue) {
                // (the others find out by themselves)
            } else if (ok) {
                umma_commit(acc_bar);           // accumulator complete
            } else {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
            }
        }
    } else {
        // ---- epilogue -----------------------------------------------------------------------
        const int q = warp & 3;                        // tensor-memory lane group of this warp
        const int n = n0 + q * 32 + lane;              // output feature of this thread
        const bool n_ok = n < p.N;
        const bool ok = mbar_wait(acc_bar, 0, &s_abort, p.wait_limit, p.status, 0x15);
        if (!ok) {
            if (lane == 0) {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
            }
        } else {
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
            const int cols = MODE == MODE_SWIGLU ? 2 * p.N : p.N;
            const float bias = (MODE == MODE_PLAIN && p.bias && n_ok) ? p.bias[n] : 0.f;
            const int rows_here = min(BN, row_end - row0);
            if (p.cluster) {
                // the K splits of a tile are the CTAs of one cluster: each leaves its partial tile in
                // its own shared memory (the pipeline stages are free by now), as [acc][row][feature]
                float* stage = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
                const int f = q * 32 + lane;
                for (int c0 = 0; c0 < rows_here; c0 += 16) {
                    float a[16], b[16];
                    __syncwarp();
                    tmem_ld16(taddr + c0, a);
                    if (MODE == MODE_SWIGLU) tmem_ld16(taddr + BN + c0, b);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        if (c0 + j < rows_here) {
                            stage[(c0 + j) * TILE_W + f] = a[j];
                            if (MODE == MODE_SWIGLU) stage[(BN + c0 + j) * TILE_W + f] = b[j];
                        }
                    }
                }
            } else if (p.splits == 1) {
                for (int c0 = 0; c0 < rows_here; c0 += 16) {      // trip count uniform per warp
                    float a[16], b[16];
                    __syncwarp();
                    tmem_ld16(taddr + c0, a);
                    if (MODE == MODE_SWIGLU) tmem_ld16(taddr + BN + c0, b);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int t = row0 + c0 + j;
                        if (n_ok && t < row_end) {
                            const float v = MODE == MODE_SWIGLU ? silu_mul(a[j], b[j]) : a[j] + bias;
                            if (p.out_bf16)
                                ((__nv_bfloat16*)p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(v);
                            else
                                ((float*)p.out)[(size_t)t * p.ldo + n] = v;
                        }
                    }
                }
            } else {
                // partial sums of this split
                float* mine = p.partials + (size_t)split * p.M * cols;
                for (int c0 = 0; c0 < rows_here; c0 += 16) {
                    float a[16], b[16];
                    __syncwarp();
                    tmem_ld16(taddr + c0, a);
                    if (MODE == MODE_SWIGLU) tmem_ld16(taddr + BN + c0, b);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int t = row0 + c0 + j;
                        if (n_ok && t < row_end) {
                            mine[(size_t)t * cols + n] = a[j];
                            if (MODE == MODE_SWIGLU) mine[(size_t)t * cols + p.N + n] = b[j];
                        }
                    }
                }
                __threadfence();
                // the four epilogue warps meet, one thread takes the ticket
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    int* ticket = p.tickets + (size_t)blockIdx.y * gridDim.x + blockIdx.x;
                    const int old = atomicAdd(ticket, 1);
                    const int last = old == p.splits - 1;
                    if (last) *ticket = 0;                 // ready for the next launch
                    s_work[3] = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (s_work[3]) {
                    __threadfence();
                    if (n_ok) {
                        const size_t split_stride = (size_t)p.M * cols;
                        // RB rows at a time: the values of all their splits are requested before any
                        // is used, so a block of rows costs one memory latency; each sum keeps the
                        // split order
                        constexpr int RB = MODE == MODE_SWIGLU ? 2 : 4;
                        for (int t0 = row0; t0 < row0 + rows_here; t0 += RB) {
                            float va[RB][MAX_SPLITS], vb[RB][MAX_SPLITS];
#pragma unroll
                            for (int r = 0; r < RB; r++) {
                                const bool live = t0 + r < row0 + rows_here;
                                const float* src = p.partials + (size_t)(t0 + r) * cols + n;
#pragma unroll
                                for (int s = 0; s < MAX_SPLITS; s++) {
                                    const bool on = live && s < p.splits;
                                    va[r][s] = on ? __ldcg(src + s * split_stride) : 0.f;
                                    if (MODE == MODE_SWIGLU) vb[r][s] = on ? __ldcg(src + s * split_stride + p.N) : 0.f;
                                }
                            }
#pragma unroll
                            for (int r = 0; r < RB; r++) {
                                const int t = t0 + r;
                                if (t >= row0 + rows_here) break;
                                float sa = 0.f, sb = 0.f;
#pragma unroll
                                for (int s = 0; s < MAX_SPLITS; s++) {
                                    sa += va[r][s];
                                    if (MODE == MODE_SWIGLU) sb += vb[r][s];
                                }
                                const float v = MODE == MODE_SWIGLU ? silu_mul(sa, sb) : sa + bias;
                                if (p.out_bf16)
                                    ((__nv_bfloat16*)p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(v);
                                else
                                    ((float*)p.out)[(size_t)t * p.ldo + n] = v;
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (p.cluster) {
        // Every thread of every CTA of the cluster comes here (all waits above are bounded), so the
        // two cluster barriers always complete.  Between them CTA r adds, for the rows r, r + S, ...
        // of the tile, the S partial values in split order (reading its peers' shared memory) and
        // writes the result; after the second barrier no peer reads this CTA's memory any more.
        cluster_sync_all();
        if (warp >= 2 && !s_abort) {
            const uint32_t S = (uint32_t)p.splits, rank = cluster_ctarank();
            const int f = (warp & 3) * 32 + lane, n = n0 + f;
            const int rows_here = min(BN, row_end - row0);
            const float bias = (MODE == MODE_PLAIN && p.bias && n < p.N) ? p.bias[n] : 0.f;
            uint32_t peer[8];
#pragma unroll
            for (uint32_t s = 0; s < 8; s++) peer[s] = mapa_cluster(base, s < S ? s : 0);
            for (int t0 = (int)rank; t0 < rows_here; t0 += 2 * (int)S) {
                float va[2][8], vb[2][8];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int t = t0 + r * (int)S;
#pragma unroll
                    for (uint32_t s = 0; s < 8; s++) {
                        const bool on = t < rows_here && s < S;
                        va[r][s] = on ? ld_cluster_f32(peer[s] + (uint32_t)(t * TILE_W + f) * 4u) : 0.f;
                        if (MODE == MODE_SWIGLU)
                            vb[r][s] = on ? ld_cluster_f32(peer[s] + (uint32_t)((BN + t) * TILE_W + f) * 4u) : 0.f;
                    }
                }
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const int t = t0 + r * (int)S;
                    if (t >= rows_here || n >= p.N) continue;
                    float sa = 0.f, sb = 0.f;
#pragma unroll
                    for (int s = 0; s < 8; s++) {
                        sa += va[r][s];
                        if (MODE == MODE_SWIGLU) sb += vb[r][s];
                    }
                    const float v = MODE == MODE_SWIGLU ? silu_mul(sa, sb) : sa + bias;
                    if (p.out_bf16)
                        ((__nv_bfloat16*)p.out)[(size_t)(row0 + t) * p.ldo + n] = __float2bfloat16_rn(v);
                    else
                        ((float*)p.out)[(size_t)(row0 + t) * p.ldo + n] = v;
                }
            }
        }
        cluster_sync_all();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
}

constexpr int EPI_GROUPS = 4;                        // epilogue warps per quarter of the accumulator's lanes
constexpr int P_THREADS = 64 + 128 * EPI_GROUPS;     // producer warp, MMA warp, epilogue warps

// What one epilogue warp of a persistent kernel does with a finished tile: feature n (this lane's row
// of the accumulator at taddr), tokens row0 + [c_lo, c_hi).  The persistent kernels have EPI_GROUPS
// epilogue warps for each quarter of the accumulator's lanes, which share the tile's tokens:
// the epilogue is a chain of tensor-memory loads (each waited for) and scattered stores, and with
// four warps it took twice as long as the tile's MMAs.
template <int BN, int MODE>
__device__ __forceinline__ void epilogue_part(const Params& p, uint32_t taddr, int n, int row0, int row_end, int c_lo,
                                              int c_hi) {
    const bool n_ok = n < p.N;
    const float bias = (MODE == MODE_PLAIN && p.bias && n_ok) ? p.bias[n] : 0.f;
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        float a[32], bb[32];
        __syncwarp();
        tmem_ld32(taddr + c0, a);
        if (MODE == MODE_SWIGLU) tmem_ld32(taddr + BN + c0, bb);
        if (p.out_bf16) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)(row0 + c0) * p.ldo + n;
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (n_ok && row0 + c0 + j < row_end)
                    o[(size_t)j * p.ldo] = __float2bfloat16_rn(MODE == MODE_SWIGLU ? silu_mul(a[j], bb[j]) : a[j] + bias);
        } else {
            float* o = (float*)p.out + (size_t)(row0 + c0) * p.ldo + n;
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (n_ok && row0 + c0 + j < row_end)
                    o[(size_t)j * p.ldo] = MODE == MODE_SWIGLU ? silu_mul(a[j], bb[j]) : a[j] + bias;
        }
    }
}

// The same for MODE_SWIGLU_IL: lanes 0..15 of this warp's quarter hold the gate rows of 16 features,
// lanes 16..31 the up rows of the same features.  Of each pair of tokens the lower lanes take the
// first (they get `up` from lane + 16), the upper lanes the second (they get `gate` from lane - 16).
template <int BN>
__device__ __forceinline__ void epilogue_part_il(const Params& p, uint32_t taddr, int f, bool upper, int row0,
                                                 int row_end, int c_lo, int c_hi) {
    const bool n_ok = f < p.N;
    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        float a[32];
        __syncwarp();
        tmem_ld32(taddr + c0, a);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const float send = upper ? a[j] : a[j + 1];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
            const float v = upper ? silu_mul(recv, a[j + 1]) : silu_mul(a[j], recv);
            const int r = row0 + c0 + j + (upper ? 1 : 0);
            if (n_ok && r < row_end) {
                if (p.out_bf16)
                    ((__nv_bfloat16*)p.out)[(size_t)r * p.ldo + f] = __float2bfloat16_rn(v);
                else
                    ((float*)p.out)[(size_t)r * p.ldo + f] = v;
            }
        }
    }
}

// ---- the persistent form, for many tokens ------------------------------------------------------
// One CTA per SM walks over the tiles (blockIdx.x, blockIdx.x + gridDim.x, ...).  The producer and
// the MMA issuer run ahead across tile borders, and the accumulator in tensor memory is doubled,
// so that the epilogue of one tile (tensor memory -> registers -> global memory) runs while the
// tensor cores work on the next.  No K split here.  Tile order: see tile_of (what is read more
// than once should be read by CTAs that run at the same time, so that it comes from L2).
template <int BN, int MODE>
struct PCfg {
    static constexpr int NW = MODE == MODE_SWIGLU ? 2 : 1;
    static constexpr int W_BYTES = TILE_W * BK * 2;
    static constexpr int XBOX = 64;      // activation rows of one copy: only as many copies as hold a tile's tokens
    static constexpr int STAGE_BYTES = NW * W_BYTES + BN * BK * 2;
    static constexpr int STAGES_RAW = (196 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int ACC_COLS = NW * BN;            // columns of one accumulator buffer
    static constexpr int NBUF = 2;                      // a tile's epilogue runs under the next tile's MMAs
    static constexpr int TMEM_COLS = NBUF * ACC_COLS;   // 256 or 512: a power of two
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(BN >= 64 && TMEM_COLS <= 512 && STAGES >= 2, "tile does not fit");
};

struct Tile {
    int g, row0, row_end, n0;
};

// item -> tile.  prefix[i]: token tiles of the groups before i (grouped), in shared memory.
template <int BN, int TW = TILE_W>
__device__ __forceinline__ Tile tile_of(int item, int m_tiles, const Params& p, const int* prefix, const int* offs) {
    Tile t;
    if (!p.group_offsets) {
        // all token tiles of one feature tile first: CTAs running together share weight tiles in L2
        const int nt = item / m_tiles, m = item % m_tiles;
        t.n0 = nt * TW, t.g = 0, t.row0 = m * BN, t.row_end = p.M;
        return t;
    }
    // grouped: all feature tiles of one token tile first.  A group's weights are read once anyway;
    // its activations are read by every feature tile, and stay in L2 only if those run together
    const int n_tiles = (p.N + TW - 1) / TW;
    const int m = item / n_tiles;
    t.n0 = (item % n_tiles) * TW;
    int lo = 0, hi = p.num_groups;          // the last group whose first tile is <= m
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= m) lo = mid; else hi = mid;
    }
    t.g = lo, t.row0 = offs[lo] + (m - prefix[lo]) * BN, t.row_end = offs[lo + 1];
    return t;
}

template <int BN, int MODE>
__global__ void __launch_bounds__(P_THREADS)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                          const Params p) {
    using C = PCfg<BN, MODE>;
    // features of a tile: 128, or 64 where gate and up rows share the tile's 128 rows
    constexpr int TW = MODE == MODE_SWIGLU_IL ? TILE_W / 2 : TILE_W;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_tmem;
    __shared__ int s_offs[MAX_SMEM_GROUPS + 1], s_prefix[MAX_SMEM_GROUPS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_sync();

    // ---- the list of tiles ---------------------------------------------------------------------
    int m_tiles = (p.M + BN - 1) / BN;
    if (p.group_offsets) {
        for (int i = threadIdx.x; i <= p.num_groups; i += blockDim.x) s_offs[i] = p.group_offsets[i];
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = 0;
            for (int i = 0; i < p.num_groups; i++) {
                s_prefix[i] = run;
                run += (s_offs[i + 1] - s_offs[i] + BN - 1) / BN;
            }
            s_prefix[p.num_groups] = run;
        }
    }
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    if (p.group_offsets) m_tiles = s_prefix[p.num_groups];
    const int items = m_tiles * ((p.N + TW - 1) / TW);

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + C::STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    auto acc_full = [&](int b) { return bar_base + 8u * (2 * C::STAGES + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (2 * C::STAGES + 2 + b); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < C::NBUF; b++) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4 * EPI_GROUPS);      // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const int kbs = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---- producer: one ring of stages across all tiles ---------------------------------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < items && ok && p.test_fault != 1; item += gridDim.x) {
                const Tile t = tile_of<BN, TW>(item, m_tiles, p, s_prefix, s_offs);
                const int n_eff = min(BN, (min(BN, t.row_end - t.row0) + 15) & ~15);
                const int xchunks = (n_eff + C::XBOX - 1) / C::XBOX;
                const uint32_t stage_tx = C::NW * C::W_BYTES + xchunks * C::XBOX * BK * 2;
                const int w_row = t.g * p.w_rows_per_group + t.n0;
                for (int kb = 0; kb < kbs; kb++, issued++) {
                    const int s = issued % C::STAGES;
                    ok = mbar_wait(empty_bar(s), ((issued / C::STAGES) & 1) ^ 1, &s_abort, p.wait_limit, p.status, 0x21);
                    if (!ok) break;
                    const uint32_t st = base + s * C::STAGE_BYTES;
                    mbar_expect_tx(full_bar(s), stage_tx);
                    if (MODE == MODE_SWIGLU_IL) {
                        // tmW is five-dimensional here, (k, row of 16, gate|up, block of 16 features, group):
                        // one box is four times [16 gate rows, the 16 up rows of the same features]
                        tma_load_5d(st, &tmW, kb * BK, 0, 0, t.n0 / 16, t.g, full_bar(s));
                    } else {
                        tma_load_2d(st, &tmW, kb * BK, w_row, full_bar(s));
                    }
                    if (MODE == MODE_SWIGLU) tma_load_2d(st + C::W_BYTES, &tmW, kb * BK, w_row + p.N, full_bar(s));
                    for (int c = 0; c < xchunks; c++)
                        tma_load_2d(st + C::NW * C::W_BYTES + c * C::XBOX * BK * 2, &tmX, kb * BK,
                                    t.row0 + c * C::XBOX, full_bar(s));
                }
            }
            if (!ok) {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
                for (int i = max(0, issued - C::STAGES); i < issued; i++)     // copies in flight must land
                    mbar_wait(full_bar(i % C::STAGES), (i / C::STAGES) & 1, nullptr, p.wait_limit, p.status, 0x22);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: accumulator buffer (tile & 1) -------------------------------------------
        if (lane == 0) {
            int consumed = 0, local = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < items && ok && p.test_fault != 2; item += gridDim.x, local++) {
                const Tile t = tile_of<BN, TW>(item, m_tiles, p, s_prefix, s_offs);
                const int n_eff = min(BN, (min(BN, t.row_end - t.row0) + 15) & ~15);
                const uint32_t idesc = instr_desc(n_eff);
                const int b = local % C::NBUF;
                ok = mbar_wait(acc_empty(b), ((local / C::NBUF) & 1) ^ 1, &s_abort, p.wait_limit, p.status, 0x23);   // the epilogue has drained it
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc_addr = tmem + b * C::ACC_COLS;
                for (int kb = 0; kb < kbs; kb++, consumed++) {
                    const int s = consumed % C::STAGES;
                    ok = mbar_wait(full_bar(s), (consumed / C::STAGES) & 1, &s_abort, p.wait_limit, p.status, 0x24);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = base + s * C::STAGE_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                        const uint32_t koff = k4 * UMMA_K * 2;
                        const uint64_t bdesc = smem_desc(st + C::NW * C::W_BYTES + koff);
                        const uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;
                        umma_bf16(acc_addr, smem_desc(st + koff), bdesc, idesc, acc);
                        if (MODE == MODE_SWIGLU)
                            umma_bf16(acc_addr + BN, smem_desc(st + C::W_BYTES + koff), bdesc, idesc, acc);
                    }
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(acc_full(b));
            }
            if (!ok) {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
            }
        }
    } else {
        // ---- epilogue: warps 2...; warp (q, h) takes lanes 32 q.. and part h of the tile's tokens --------
        const int q = warp & 3, h = (warp - 2) >> 2;
        int local = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x, local++) {
            const Tile t = tile_of<BN, TW>(item, m_tiles, p, s_prefix, s_offs);
            const int b = local % C::NBUF;
            ok = mbar_wait(acc_full(b), (local / C::NBUF) & 1, &s_abort, p.wait_limit, p.status, 0x25);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem + b * C::ACC_COLS + ((uint32_t)(q * 32) << 16);
            const int rows_here = min(BN, t.row_end - t.row0);
            const int part = ((rows_here + 32 * EPI_GROUPS - 1) / (32 * EPI_GROUPS)) * 32;      // a multiple of 32
            if (MODE == MODE_SWIGLU_IL)
                epilogue_part_il<BN>(p, taddr, t.n0 + q * 16 + (lane & 15), (lane & 16) != 0, t.row0, t.row_end,
                                     min(rows_here, h * part), min(rows_here, (h + 1) * part));
            else
                epilogue_part<BN, MODE>(p, taddr, t.n0 + q * 32 + lane, t.row0, t.row_end, min(rows_here, h * part),
                                        min(rows_here, (h + 1) * part));
            // this warp has read its part of the buffer: the MMA issuer may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(b)) : "memory");
        }
        if (!ok && lane == 0) {
            atomicOr(p.status, ST_WAIT_TIMEOUT);
            s_abort = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
}


// ---- the persistent form on pairs of CTAs ------------------------------------------------------
// Two CTAs of a cluster (two SMs) share one tile of 256 features x BN tokens: each loads its own 128
// weight rows and HALF of the tile's tokens, the first CTA issues tcgen05.mma.cta_group::2, which reads
// both shared memories, and each CTA finds its 128 features of the result in its own tensor memory.
// A CTA thus brings 16 + 16 KB a stage into shared memory for the work that 16 + 32 KB bring without
// pairing, which is what bounds the single-CTA form for many tokens (L2 to shared memory).
//   full[s]      in the first CTA: its expect_tx arrival, bytes of both CTAs' loads
//   empty[s]     in each CTA: the MMA issuer's commit, multicast to both
//   acc_full[b]  in each CTA: likewise
//   acc_empty[b] in the first CTA: the epilogue warps of both CTAs
template <int BN, int MODE>
struct PairCfg {
    static constexpr int NW = MODE == MODE_SWIGLU ? 2 : 1;
    static constexpr int W_BYTES = TILE_W * BK * 2;
    static constexpr int XBOX = 64;
    static constexpr int X_ROWS = ((BN / 2 + XBOX - 1) / XBOX) * XBOX;      // this CTA's half of the tokens
    static constexpr int STAGE_BYTES = NW * W_BYTES + X_ROWS * BK * 2;
    static constexpr int STAGES_RAW = (196 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int ACC_COLS = NW * BN;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(BN >= 128 && TMEM_COLS <= 512 && STAGES >= 2, "tile does not fit");
};

template <int BN, int MODE>
__global__ void __launch_bounds__(P_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
    using C = PairCfg<BN, MODE>;
    constexpr int PAIR_W = 2 * TILE_W;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_tmem;
    __shared__ int s_offs[MAX_SMEM_GROUPS + 1], s_prefix[MAX_SMEM_GROUPS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();        // 0: the CTA that issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    pdl_sync();

    int m_tiles = (p.M + BN - 1) / BN;
    if (p.group_offsets) {
        for (int i = threadIdx.x; i <= p.num_groups; i += blockDim.x) s_offs[i] = p.group_offsets[i];
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = 0;
            for (int i = 0; i < p.num_groups; i++) {
                s_prefix[i] = run;
                run += (s_offs[i + 1] - s_offs[i] + BN - 1) / BN;
            }
            s_prefix[p.num_groups] = run;
        }
    }
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    if (p.group_offsets) m_tiles = s_prefix[p.num_groups];
    const int items = m_tiles * ((p.N + PAIR_W - 1) / PAIR_W);

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + C::STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    auto acc_full = [&](int b) { return bar_base + 8u * (2 * C::STAGES + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (2 * C::STAGES + 2 + b); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 8 * EPI_GROUPS);     // one arrival per epilogue warp of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(&s_tmem), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the other CTA's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const int kbs = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ---- producer (in both CTAs): own weight rows, own half of the tokens --------------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int item = pair; item < items && ok; item += pairs) {
                const Tile t = tile_of<BN, PAIR_W>(item, m_tiles, p, s_prefix, s_offs);
                const int n_eff = min(BN, (min(BN, t.row_end - t.row0) + 15) & ~15);
                const int half = n_eff >> 1;
                const int xchunks = (half + C::XBOX - 1) / C::XBOX;
                const uint32_t cta_tx = C::NW * C::W_BYTES + xchunks * C::XBOX * BK * 2;
                const int w_row = t.g * p.w_rows_per_group + t.n0 + (int)rank * TILE_W;
                const int x_row = t.row0 + (int)rank * half;
                for (int kb = 0; kb < kbs; kb++, issued++) {
                    const int s = issued % C::STAGES;
                    ok = mbar_wait(empty_bar(s), ((issued / C::STAGES) & 1) ^ 1, &s_abort, p.wait_limit, p.status, 0x31);
                    if (!ok) break;
                    const uint32_t st = base + s * C::STAGE_BYTES;
                    const uint32_t bar = mapa_cluster(full_bar(s), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * cta_tx);
                    tma_load_2d_pair(st, &tmW, kb * BK, w_row, bar);
                    if (MODE == MODE_SWIGLU) tma_load_2d_pair(st + C::W_BYTES, &tmW, kb * BK, w_row + p.N, bar);
                    for (int c = 0; c < xchunks; c++)
                        tma_load_2d_pair(st + C::NW * C::W_BYTES + c * C::XBOX * BK * 2, &tmX, kb * BK,
                                         x_row + c * C::XBOX, bar);
                }
            }
            if (!ok) {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
                if (rank == 0)
                    for (int i = max(0, issued - C::STAGES); i < issued; i++)     // copies in flight must land
                        mbar_wait(full_bar(i % C::STAGES), (i / C::STAGES) & 1, nullptr, p.wait_limit, p.status, 0x32);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (first CTA only): accumulator buffer (tile & 1) ---------------------------
        if (lane == 0 && rank == 0) {
            int consumed = 0, local = 0;
            bool ok = true;
            for (int item = pair; item < items && ok; item += pairs, local++) {
                const Tile t = tile_of<BN, PAIR_W>(item, m_tiles, p, s_prefix, s_offs);
                const int n_eff = min(BN, (min(BN, t.row_end - t.row0) + 15) & ~15);
                const uint32_t idesc = instr_desc(n_eff, PAIR_W);
                const int b = local & 1;
                ok = mbar_wait(acc_empty(b), ((local >> 1) & 1) ^ 1, &s_abort, p.wait_limit, p.status, 0x33);   // both epilogues have drained it
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc_addr = tmem + b * C::ACC_COLS;
                for (int kb = 0; kb < kbs; kb++, consumed++) {
                    const int s = consumed % C::STAGES;
                    ok = mbar_wait(full_bar(s), (consumed / C::STAGES) & 1, &s_abort, p.wait_limit, p.status, 0x34);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = base + s * C::STAGE_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                        const uint32_t koff = k4 * UMMA_K * 2;
                        const uint64_t bdesc = smem_desc(st + C::NW * C::W_BYTES + koff);
                        const uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;
                        umma_bf16_pair(acc_addr, smem_desc(st + koff), bdesc, idesc, acc);
                        if (MODE == MODE_SWIGLU)
                            umma_bf16_pair(acc_addr + BN, smem_desc(st + C::W_BYTES + koff), bdesc, idesc, acc);
                    }
                    umma_commit_pair(empty_bar(s));
                }
                if (ok) umma_commit_pair(acc_full(b));
            }
            if (!ok) {
                atomicOr(p.status, ST_WAIT_TIMEOUT);
                s_abort = 1;
            }
        }
    } else {
        // ---- epilogue (in both CTAs): this CTA's 128 features of the tile; warps as in the single form --
        const int q = warp & 3, h = (warp - 2) >> 2;
        int local = 0;
        bool ok = true;
        for (int item = pair; item < items && ok; item += pairs, local++) {
            const Tile t = tile_of<BN, PAIR_W>(item, m_tiles, p, s_prefix, s_offs);
            const int b = local & 1;
            ok = mbar_wait(acc_full(b), (local >> 1) & 1, &s_abort, p.wait_limit, p.status, 0x35);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem + b * C::ACC_COLS + ((uint32_t)(q * 32) << 16);
            const int rows_here = min(BN, t.row_end - t.row0);
            const int part = ((rows_here + 32 * EPI_GROUPS - 1) / (32 * EPI_GROUPS)) * 32;
            epilogue_part<BN, MODE>(p, taddr, t.n0 + (int)rank * TILE_W + q * 32 + lane, t.row0, t.row_end,
                                    min(rows_here, h * part), min(rows_here, (h + 1) * part));
            // this warp has read its part of the buffer; the issuer waits for all epilogue warps of the pair
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_cluster(acc_empty(b), 0));
        }
        if (!ok && lane == 0) {
            atomicOr(p.status, ST_WAIT_TIMEOUT);
            s_abort = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither CTA frees tensor memory or leaves while the other may still use it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, C::TMEM_COLS);
    }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    });
    return fn;
}

// 2-D bf16 row-major [rows, cols] with row pitch ld (elements); box [box_rows, 64], 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// W [G][2 I][K] (gate rows, then up rows), I a multiple of 16, seen as (k, row of 16, gate|up, block
// of 16 features, group): a box of 64 x 16 x 2 x 4 x 1 is, four times, 16 gate rows followed by the 16
// up rows of the same features: a 128-row tile of 64 features in one copy.  Blocks past I / 16 read
// as zeros.
bool make_map_gate_up(CUtensorMap* map, const void* ptr, uint64_t groups, uint64_t inter, uint64_t K) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || inter % 16) return false;
    cuuint64_t dims[5] = {K, 16, 2, inter / 16, groups};
    cuuint64_t strides[4] = {K * 2, inter * K * 2, 16 * K * 2, 2 * inter * K * 2};
    cuuint32_t box[5] = {(cuuint32_t)BK, 16, 2, 4, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int MAX_CLUSTER = 8;   // portable cluster size

template <int BN, int MODE>
int launch(const CUtensorMap& tmW, const CUtensorMap& tmX, Params p, dim3 grid, cudaStream_t stream) {
    using C = Cfg<BN, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    p.cluster = (p.splits > 1 && p.splits <= MAX_CLUSTER && C::CLUSTER_OK) ? 1 : 0;
    if (p.splits > 1 && !p.cluster && (!p.partials || !p.tickets)) return -1;
    return launch_pdl_cluster(gemm_tc_kernel<BN, MODE>, grid, dim3(192), (size_t)C::SMEM, stream,
                              p.cluster ? p.splits : 1, tmW, tmX, p);
}

int g_persistent = 1;
uint32_t g_wait_limit = WAIT_LIMIT_US;
int g_test_fault = 0;

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n = 0;
        if (n <= 0) n = 1;
    }
    return n;
}

template <int BN, int MODE>
int launch_persistent(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int max_items,
                      cudaStream_t stream) {
    using C = PCfg<BN, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int ctas = max_items < sm_count() ? max_items : sm_count();
    return launch_pdl(gemm_tc_persistent_kernel<BN, MODE>, dim3(ctas), dim3(P_THREADS), (size_t)C::SMEM, stream, tmW, tmX, p);
}

int g_pair = 0;
int g_swiglu_il = 1;

template <int BN, int MODE>
int launch_pair(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int max_items, cudaStream_t stream) {
    using C = PairCfg<BN, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int most = sm_count() / 2;
    const int pairs = max_items < most ? max_items : most;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs), cfg.blockDim = dim3(P_THREADS), cfg.dynamicSmemBytes = (size_t)C::SMEM, cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = g_pdl_enabled ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN, MODE>, tmW, tmX, p);
}

}  // namespace

// X: [M, K] bf16 with row pitch ldx; W: [G * w_rows, K] bf16 contiguous; out: [M, ldo].
//   mode 0: w_rows = N; mode 1 (SwiGLU): w_rows = 2 N, gate rows first.
//   bn: token tile (16, 32, 64, 128 or 256).  splits >= 1; with splits > 1, partials holds
//   splits * M * (mode ? 2 N : N) floats and tickets grid.y * grid.x zeroed ints.
// Returns 0, a CUDA error code, or -1 if the shape cannot be handled (the caller falls back).
MOE_API int moe_gemm_tc(const void* X, int ldx, const void* W, int num_groups, int N, int K, int mode, void* out,
                        int out_bf16, int ldo, const float* bias, const int* group_offsets, int M, int bn, int splits,
                        float* partials, int* tickets, int* status, int early_offsets, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return -1;
    const int w_rows = mode == MODE_SWIGLU ? 2 * N : N;
    CUtensorMap tmW, tmX;
    if (!make_map(&tmW, W, (uint64_t)num_groups * w_rows, K, K, TILE_W)) return -1;
    if (!make_map(&tmX, X, M, K, ldx, bn < 64 ? bn : 64)) return -1;
    const int kb_total = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits > kb_total) splits = kb_total;
    const int per = (kb_total + splits - 1) / splits;
    splits = (kb_total + per - 1) / per;
    Params p;
    p.cluster = 0, p.early_offsets = (group_offsets && early_offsets) ? 1 : 0;
    p.out = out, p.out_bf16 = out_bf16, p.ldo = ldo, p.bias = bias, p.group_offsets = group_offsets;
    p.num_groups = num_groups, p.M = M, p.N = N, p.K = K, p.w_rows_per_group = w_rows, p.splits = splits;
    p.kb_per_split = per, p.partials = partials, p.tickets = tickets, p.status = status;
    p.wait_limit = g_wait_limit, p.test_fault = g_test_fault;
    // token tiles: sum over groups of ceil(rows / bn) <= (non-empty groups) + floor(M / bn); CTAs past
    // the real count leave at once, but each still reserves its shared memory, so the bound is kept tight
    if (splits == 1 && bn >= 128 && g_persistent && (!group_offsets || num_groups <= MAX_SMEM_GROUPS)) {
        // many tokens: the persistent form (SwiGLU keeps two accumulators, so its widest tile is 128)
        const int pbn = (mode == MODE_SWIGLU || bn == 128) ? 128 : 256;
        const int mt = group_offsets ? (M < num_groups ? M : num_groups) + M / pbn : (M + pbn - 1) / pbn;
        const long long max_items = (long long)mt * ((N + TILE_W - 1) / TILE_W);
        const int cap = max_items > (1 << 30) ? (1 << 30) : (int)max_items;
        if (g_pair && sm_count() >= 2) {
            // pairs of CTAs on tiles of 256 features: half the activation traffic into shared memory
            const long long pair_items = (long long)mt * ((N + 2 * TILE_W - 1) / (2 * TILE_W));
            const int pcap = pair_items > (1 << 30) ? (1 << 30) : (int)pair_items;
            if (mode == MODE_SWIGLU) return launch_pair<128, MODE_SWIGLU>(tmW, tmX, p, pcap, stream);
            if (pbn == 128) return launch_pair<128, MODE_PLAIN>(tmW, tmX, p, pcap, stream);
            return launch_pair<256, MODE_PLAIN>(tmW, tmX, p, pcap, stream);
        }
        if (mode == MODE_SWIGLU && g_swiglu_il) {
            // one accumulator of up to 256 tokens for 64 features (gate and up rows interleaved by the
            // load), instead of two of 128 tokens for 128 features: half the MMA instructions where a
            // group has between 129 and 256 tokens, and room for two accumulator buffers all the same.
            // (Measured equal to the two-accumulator form on a B200: what bounds these products is the
            // weight stream from DRAM, not MMA instructions, copies or bytes into shared memory.)
            CUtensorMap tmG;
            const int ibn = bn >= 256 ? 256 : 128;
            if (make_map_gate_up(&tmG, W, (uint64_t)num_groups, (uint64_t)N, (uint64_t)K)) {
                const int imt = group_offsets ? (M < num_groups ? M : num_groups) + M / ibn : (M + ibn - 1) / ibn;
                const long long il_items = (long long)imt * ((N + TILE_W / 2 - 1) / (TILE_W / 2));
                const int icap = il_items > (1 << 30) ? (1 << 30) : (int)il_items;
                if (ibn == 256) return launch_persistent<256, MODE_SWIGLU_IL>(tmG, tmX, p, icap, stream);
                return launch_persistent<128, MODE_SWIGLU_IL>(tmG, tmX, p, icap, stream);
            }
        }
        if (mode == MODE_SWIGLU) return launch_persistent<128, MODE_SWIGLU>(tmW, tmX, p, cap, stream);
        if (pbn == 128) return launch_persistent<128, MODE_PLAIN>(tmW, tmX, p, cap, stream);
        return launch_persistent<256, MODE_PLAIN>(tmW, tmX, p, cap, stream);
    }
    const int m_tiles = group_offsets ? (M < num_groups ? M : num_groups) + M / bn : (M + bn - 1) / bn;
    dim3 grid((N + TILE_W - 1) / TILE_W, m_tiles, splits);
    if (grid.y > 65535 || grid.z > 65535) return -1;
#define GO(BN_)                                                                              \
    if (bn == BN_)                                                                           \
        return mode == MODE_SWIGLU ? launch<BN_, MODE_SWIGLU>(tmW, tmX, p, grid, stream)     \
                                   : launch<BN_, MODE_PLAIN>(tmW, tmX, p, grid, stream);
    GO(16) GO(32) GO(64) GO(128) GO(256)
#undef GO
    return -1;
}

// Programmatic dependent launch on or off for the kernels of this library (on by default).
MOE_API void moe_tc_set_pdl(int enabled) { g_pdl_enabled = enabled ? 1 : 0; }

// The persistent form for many tokens on or off (on by default; off: one CTA per tile).
MOE_API void moe_tc_set_persistent(int enabled) { g_persistent = enabled ? 1 : 0; }

// The one-accumulator SwiGLU form of the persistent kernel on or off (on by default).
MOE_API void moe_tc_set_swiglu_interleaved(int enabled) { g_swiglu_il = enabled ? 1 : 0; }

// For the test of the bounded waits only: ``fault`` 1 makes the producer of the single-CTA kernels
// load nothing, 2 makes their MMA issuer issue nothing, so that the other roles' waits run out after
// ``wait_limit`` microseconds (0: the normal limit); the CTAs then set ST_WAIT_TIMEOUT in the status word,
// wait for their own copies in flight, free their tensor memory and return.  (0, 0) restores the
// normal behaviour.  Nothing faults and nothing waits without a limit.
MOE_API void moe_tc_set_wait_test(int fault, unsigned wait_limit) {
    g_test_fault = (fault == 1 || fault == 2) ? fault : 0;
    g_wait_limit = wait_limit ? wait_limit : WAIT_LIMIT_US;
}

// Pairs of CTAs (cta_group::2) for the persistent form on or off (off by default: measured equal or
// slower than single CTAs at the sizes tried, so what bounds those is not the activation traffic).
MOE_API void moe_tc_set_pair(int enabled) { g_pair = enabled ? 1 : 0; }

// How many K splits the kernel will really use for (K, splits asked), and its grid.y for tickets.
MOE_API int moe_gemm_tc_plan(int K, int splits, int M, int bn, int num_groups, int grouped, int* grid_y) {
    const int kb_total = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kb_total) splits = kb_total;
    const int per = (kb_total + splits - 1) / splits;
    *grid_y = grouped ? (M < num_groups ? M : num_groups) + M / bn : (M + bn - 1) / bn;
    return (kb_total + per - 1) / per;
}

// dst[i, :] = src[rows[i], :] for bf16 rows of `width` elements (expert dispatch before the grouped product)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ rows,
                                   __nv_bfloat16* __restrict__ dst, int width, int src_rows, int* status) {
    pdl_sync();
    const int i = blockIdx.x;
    int r = rows[i];
    if (r < 0 || r >= src_rows) {
        if (threadIdx.x == 0) atomicOr(status, ST_BAD_ROW);
        r = 0;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)r * width);
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)i * width);
    for (int j = threadIdx.x; j < width / 8; j += blockDim.x) d[j] = s[j];
}
MOE_API int moe_gather_rows_bf16(const void* src, const int* rows, void* dst, int n, int width, int src_rows,
                                 int* status, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width % 8) return (int)cudaErrorInvalidValue;
    return launch_pdl(gather_rows_kernel, n, 128, 0, stream, (const __nv_bfloat16*)src, rows, (__nv_bfloat16*)dst,
                      width, src_rows, status);
}
