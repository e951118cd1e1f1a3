// Attention of a step of several tokens a sequence on the 5th-generation tensor cores (tcgen05),
// head sizes 64 and 128: whole prompts, and sequences that go on from the cache.
//
// Same formulas as attention_prefill.cu (reference: src/model.rs:794-827): causal, optional window
// [p + 1 - w, p], scale 1/sqrt(d), kv head = head / (heads / kv_heads); scores, running maximum
// and sum, and the output accumulator are float32; P enters the second product as two bfloat16
// terms (head and remainder), i.e. with 16 bits.
//
// One CTA takes 128 query rows of one (sequence, head) and walks the key tiles of 128 that the
// causal window allows:
//
// The keys of a query tile come in two runs of tiles: first the positions before the step, from the
// pages of the cache (tiles of 128 absolute positions, each two pages of 64 fetched by a copy of
// its own; none for a sequence that starts at 0), then the step's own keys from its buffers (tiles
// of 128 of its new tokens).  The step's keys are never read from the cache, so they may be put
// there before or after, and a ring of a window's size is enough.
//
//   warp 0      TMA producer: Q once, then K and V tiles through a ring of two stages
//   warp 1      MMA issuer: S = Q K^T (operands in shared memory, S in tensor memory, two
//               buffers), then O_tile = P V with P read from tensor memory and V as the
//               MN-major operand
//   warps 2-9   two threads per query row (half of the columns each): read the scores from tensor
//               memory, mask, keep the running maximum and sum, and write P (two bfloat16 terms)
//               back to tensor memory IN THE PLACE OF THE SCORES they were made from (a thread's
//               64 scores of 32 bits are the room of its 64 + 64 values of 16 bits).  The output
//               row accumulates in tensor memory over all tiles; its threads rescale it there
//               when the running maximum moves
//
// S of tile j + 1 is issued before the softmax of tile j has finished, and since P of tile j + 1
// lies in the other score buffer, its softmax runs while the tensor cores still work on P V of
// tile j.  The MMAs of one thread run in the order they were issued: S of tile j + 2, which
// overwrites P of tile j, is issued after P V of tile j and needs no barrier of its own.
// Every barrier wait is bounded (ST_WAIT_TIMEOUT).
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int QT = 128, KT = 128;
// tensor-memory columns: two score buffers (each later holds P: for every 32 keys 16 columns of the
// first term, then 16 of the second, in the place of their scores), the output rows
constexpr uint32_t COL_S = 0, COL_O = 256, TMEM_COLS = 512;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait: false if the barrier did not complete within WAIT_LIMIT_US (the site is then
// recorded in the status word) or another role of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 1;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 0) {
            if (abort_flag && *abort_flag) return false;
            if (global_ns() - t0 > (unsigned long long)WAIT_LIMIT_US * 1000ull) break;
        }
    }
    wait_ran_out(status, site);
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D (tensor memory) = A (shared memory) x B (shared memory)
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D (tensor memory) = A (tensor memory) x B (shared memory)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 columns of this thread's lane, without the wait: the registers are valid after tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
          "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]),
          "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]),
          "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]),
        "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]), "f"(v[16]), "f"(v[17]),
        "f"(v[18]), "f"(v[19]), "f"(v[20]), "f"(v[21]), "f"(v[22]), "f"(v[23]), "f"(v[24]), "f"(v[25]), "f"(v[26]),
        "f"(v[27]), "f"(v[28]), "f"(v[29]), "f"(v[30]), "f"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory descriptors, 128-byte swizzle, version 1 (sm_100).  A tile is stored as chunks of
// 64 elements (128 bytes) of every row, 128 rows per chunk (16 KB), as TMA writes them.
//   K-major (Q and K: the contraction runs along a row): groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
//   MN-major (V: the contraction runs down the rows, the output dimension along a row): blocks of
//   64 output elements are one chunk (16 KB) apart, groups of 8 contraction rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(16384 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// c = f32, a = b = bf16; bit 16: B is MN-major; N >> 3 at 17; M = 128 (>> 4 at 24)
__host__ __device__ constexpr uint32_t instr_desc(int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ float ex2_approx(float x) {     // 2^x; 0 for -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmKc,
                       const __grid_constant__ CUtensorMap tmVc, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                       const int* __restrict__ slots, const int* __restrict__ tables, int table_stride, int ring,
                       int num_pages, int num_seqs, int nh, int nkv, int window, float scale_log2, int* status) {
    constexpr int CH = HD / 64;                      // 128-byte chunks of a row
    constexpr int TILE_BYTES = CH * 128 * 128;       // a 128-row operand tile
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;      // K, then V
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_seq, s_tile;
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_tmem;
    __shared__ float x_max[2][2][QT], x_sum[2][QT];      // what the two threads of a row tell each other
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which (sequence, query tile, head): tiles are numbered sequence by sequence, and the heads of a
    // tile follow one another, so that the heaviest tiles of ALL heads are handed out first (with the
    // heads outermost, the last heads' heaviest tiles would start late and finish alone)
    if (threadIdx.x == 0) {
        int tile = blockIdx.x / nh, seq = -1;
        for (int s = 0; s < num_seqs; s++) {
            const int tiles = (cu_seqlens[s + 1] - cu_seqlens[s] + QT - 1) / QT;
            if (tile < tiles) {
                seq = s;
                break;
            }
            tile -= tiles;
        }
        s_seq = seq, s_tile = tile, s_abort = 0;
    }
    __syncthreads();
    const int seq = s_seq;
    if (seq < 0) return;
    const int tok0 = cu_seqlens[seq], len = cu_seqlens[seq + 1] - tok0;
    const int q_tile = (len + QT - 1) / QT - 1 - s_tile;        // heavier tiles (later rows) first
    const int q0 = q_tile * QT;
    const int head = blockIdx.x % nh, kvh = head / (nh / nkv);
    const int q_last = min(q0 + QT, len) - 1;
    // positions: the sequence held `start` tokens before the step; the query of row r stands at
    // start + q0 + r.  Key tiles: `nc` tiles of absolute positions [kt_lo * KT, ...) below `start`
    // from the cache, then tiles t_lo ... of the step's own tokens.
    const int start = seq_start ? seq_start[seq] : 0;
    const int lo_pos = window > 0 ? max(0, start + q0 + 1 - window) : 0;      // oldest key any row of the tile sees
    const int kt_lo = lo_pos / KT;
    const int nc = lo_pos < start ? (start - 1) / KT - kt_lo + 1 : 0;
    const int t_lo = window > 0 ? max(0, q0 + 1 - window) / KT : 0;
    const int n_tiles = nc + q_last / KT - t_lo + 1;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base;
    auto sK = [&](int st) { return base + TILE_BYTES + st * STAGE_BYTES; };
    auto sV = [&](int st) { return base + TILE_BYTES + st * STAGE_BYTES + TILE_BYTES; };
    const uint32_t bars = base + TILE_BYTES + 2 * STAGE_BYTES;
    const uint32_t q_full = bars;
    auto k_full = [&](int st) { return bars + 8u * (1 + st); };
    auto k_empty = [&](int st) { return bars + 8u * (3 + st); };
    auto v_full = [&](int st) { return bars + 8u * (15 + st); };
    auto v_empty = [&](int st) { return bars + 8u * (17 + st); };
    auto s_full = [&](int b) { return bars + 8u * (5 + b); };
    const uint32_t p_full = bars + 8u * 9, pv_done = bars + 8u * 10;
    auto x_bar = [&](int q) { return bars + 8u * (11 + q); };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(k_full(i), 1);
            mbar_init(k_empty(i), 1);
            mbar_init(v_full(i), 1);
            mbar_init(v_empty(i), 1);
            mbar_init(s_full(i), 1);
        }
        mbar_init(p_full, 8);
        for (int i = 0; i < 4; i++) mbar_init(x_bar(i), 2);      // the two warps that share 32 rows
        mbar_init(pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    // the set-up above needed nothing of the predecessor's (the sequence lengths are a step's input);
    // its queries, keys and values are read from here on
    pdl_sync();

    if (warp == 0) {
        // ---- producer ------------------------------------------------------------------------------
        if (lane == 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
            for (int c = 0; c < CH; c++) tma_load_3d(sQ + c * 16384, &tmQ, c * 64, head, tok0 + q0, q_full);
            // Keys and values have rings of their own: a key tile is free again as soon as its
            // scores are computed, a value tile only after P V.  The keys run one tile ahead of
            // the values, as the MMA issuer asks for them (scores of tile j + 1 before P V of tile j).
            bool ok = true;
            int nk = 0, nv = 0;                         // tiles whose keys / values have been requested
            const int* table = nc > 0 ? tables + (size_t)slots[seq] * table_stride : nullptr;
            int page_row[2][2];                         // of a cache tile's two pages: first row in the cache seen
                                                        // as rows of one head's keys, [page][kv head][64] of them
            auto find_pages = [&](int it) {
                for (int h = 0; h < 2; h++) {
                    const int a = (kt_lo + it) * KT + h * 64;         // first position of the page
                    int page = table[(ring > 0 ? a % ring : a) >> 6];
                    if (page < 0 || page >= num_pages) {
                        // only a page that holds a key some row needs is an error; the half of a tile
                        // beyond the sequence's cached tokens just has to be finite, and every page is
                        if (a < start && a + 63 >= lo_pos) atomicOr(status, ST_BAD_PAGE);
                        page = 0;
                    }
                    page_row[it & 1][h] = (page * nkv + kvh) * 64;
                }
            };
            auto load_k = [&](int it) {
                const int st = it & 1;
                if (!mbar_wait(k_empty(st), ((it >> 1) & 1) ^ 1, &s_abort, status, 0x41)) return false;
                if (it < nc) find_pages(it);
                mbar_expect_tx(k_full(st), TILE_BYTES);
                for (int c = 0; c < CH; c++) {
                    if (it < nc) {
                        tma_load_2d(sK(st) + c * 16384, &tmKc, c * 64, page_row[st][0], k_full(st));
                        tma_load_2d(sK(st) + c * 16384 + 8192, &tmKc, c * 64, page_row[st][1], k_full(st));
                    } else {
                        tma_load_3d(sK(st) + c * 16384, &tmK, c * 64, kvh, tok0 + (t_lo + it - nc) * KT, k_full(st));
                    }
                }
                nk = it + 1;
                return true;
            };
            auto load_v = [&](int it) {             // (after load_k of the same tile, which found its pages)
                const int st = it & 1;
                if (!mbar_wait(v_empty(st), ((it >> 1) & 1) ^ 1, &s_abort, status, 0x42)) return false;
                mbar_expect_tx(v_full(st), TILE_BYTES);
                for (int c = 0; c < CH; c++) {
                    if (it < nc) {
                        tma_load_2d(sV(st) + c * 16384, &tmVc, c * 64, page_row[st][0], v_full(st));
                        tma_load_2d(sV(st) + c * 16384 + 8192, &tmVc, c * 64, page_row[st][1], v_full(st));
                    } else {
                        tma_load_3d(sV(st) + c * 16384, &tmV, c * 64, kvh, tok0 + (t_lo + it - nc) * KT, v_full(st));
                    }
                }
                nv = it + 1;
                return true;
            };
            ok = load_k(0);
            for (int it = 0; it < n_tiles && ok; it++) {
                if (it + 1 < n_tiles) ok = load_k(it + 1);
                if (ok) ok = load_v(it);
            }
            if (!ok) {
                atomicOr(status, ST_WAIT_TIMEOUT);
                s_abort = 1;
                for (int i = max(0, nk - 2); i < nk; i++)       // copies in flight must land
                    mbar_wait(k_full(i & 1), (i >> 1) & 1, nullptr, status, 0x43);
                for (int i = max(0, nv - 2); i < nv; i++) mbar_wait(v_full(i & 1), (i >> 1) & 1, nullptr, status, 0x43);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(KT, 0), idesc_pv = instr_desc(HD, 1);
            bool ok = mbar_wait(q_full, 0, &s_abort, status, 0x44);
            auto issue_s = [&](int it) {           // scores of tile `it` into buffer it & 1
                const int b = it & 1;
                if (!mbar_wait(k_full(b), (it >> 1) & 1, &s_abort, status, 0x45)) return false;
                // (buffer b held P of tile it - 2: its P V product was issued before this, and the
                // MMAs run in order)
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
                    umma_ss(tmem + COL_S + b * KT, desc_k_major(sQ + off), desc_k_major(sK(b) + off), idesc_s, ks > 0);
                }
                umma_commit(s_full(b));
                umma_commit(k_empty(b));           // the key tile is free when these MMAs have read it
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int it = 0; it < n_tiles && ok; it++) {
                if (it + 1 < n_tiles) ok = issue_s(it + 1);
                if (!ok) break;
                const int st = it & 1;
                ok = mbar_wait(v_full(st), (it >> 1) & 1, &s_abort, status, 0x47) && mbar_wait(p_full, it & 1, &s_abort, status, 0x48);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tp = tmem + COL_S + st * KT;      // P lies where the tile's scores were
#pragma unroll
                for (int term = 0; term < 2; term++) {
#pragma unroll
                    for (int ks = 0; ks < KT / 16; ks++)         // 16 keys per step: 8 columns of packed P
                        umma_ts(tmem + COL_O, tp + (ks / 2) * 32 + term * 16 + (ks % 2) * 8,
                                desc_mn_major(sV(st) + ks * 2048), idesc_pv,
                                (it | term | ks) != 0);          // the output row accumulates over all tiles
                }
                umma_commit(pv_done);
                umma_commit(v_empty(st));
            }
            if (!ok) {
                atomicOr(status, ST_WAIT_TIMEOUT);
                s_abort = 1;
            }
        }
    } else {
        // ---- two threads per query row ---------------------------------------------------------------
        // Warps w and w + 4 share the tensor-memory lanes of 32 rows; each takes one half of the
        // columns (of the scores, of P and of the output row).  They exchange the half-row maxima
        // through shared memory once per tile (a bounded wait on an mbarrier, not a bar.sync: a
        // thread that gives up must not leave its partner waiting).  The output row stays in tensor
        // memory: the P V products of all tiles accumulate there, and its threads touch it only
        // when the running maximum moves (rarely, see below) and at the end.
        const int qd = warp & 3;                               // tensor-memory lane group of this warp
        const int half = (warp - 2) >> 2;                      // which half of the columns
        const int r = qd * 32 + lane;                          // row of the tile
        const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
        const int row = q0 + r;                                // this thread's query among the step's tokens
        const int prow = start + row;                          // and its position
        const uint32_t to = tmem + COL_O + lane_base + half * (HD / 2);
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_tiles; it++) {
            const int b = it & 1;
            ok = mbar_wait(s_full(b), (it >> 1) & 1, &s_abort, status, 0x49);
            if (!ok) break;
            tc_fence_after();
            const uint32_t ts = tmem + COL_S + b * KT + lane_base + half * (KT / 2);
            // the tile's first position, and the end of what its source holds of the sequence
            const int j0 = it < nc ? (kt_lo + it) * KT : start + (t_lo + it - nc) * KT;
            const int jmax = it < nc ? start : start + len;
            const int jh = j0 + half * (KT / 2);
            // a tile strictly below the diagonal, inside the window and inside the sequence needs no mask
            const bool full = j0 + KT - 1 <= start + q0 && j0 + KT <= jmax &&
                              (window <= 0 || j0 >= start + q0 + QT - window);
            auto tile_softmax = [&](auto masked_tag) -> bool {
                constexpr bool MASKED = decltype(masked_tag)::value;
                auto visible = [&](int j) { return j <= prow && j < jmax && (window <= 0 || j >= prow + 1 - window); };
                // pass 1: the maximum of the half row (of the raw scores: the scale is positive)
                float mx0 = -INFINITY, mx1 = -INFINITY;
                {
                    float s[2][32];                              // this thread's 64 scores
                    tmem_ld32_issue(ts, s[0]);
                    tmem_ld32_issue(ts + 32, s[1]);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 2; c++) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            if (!MASKED || visible(jh + c * 32 + i)) mx0 = fmaxf(mx0, s[c][i]);
                            if (!MASKED || visible(jh + c * 32 + i + 1)) mx1 = fmaxf(mx1, s[c][i + 1]);
                        }
                    }
                }
                // ... and of the whole row
                x_max[b][half][r] = fmaxf(mx0, mx1);
                __syncwarp();
                if (lane == 0) mbar_arrive(x_bar(qd));
                if (!mbar_wait(x_bar(qd), it & 1, &s_abort, status, 0x4a)) return false;
                const float mx = fmaxf(x_max[b][0][r], x_max[b][1][r]) * scale_log2;
                // The running maximum only has to keep the exponentials in range: it moves when the
                // tile's maximum exceeds it by more than 8 (a factor 256), which spares most rescalings.
                float m_new = m, alpha = 1.f;
                if (mx > m + 8.f || m == -INFINITY) {
                    m_new = fmaxf(m, mx);
                    alpha = (m == -INFINITY) ? 1.f : ex2_approx(m - m_new);     // nothing accumulated yet: nothing to rescale
                }
                // the products so far belong to the old maximum: wait for the last one, rescale the row
                // (tcgen05.ld / st are warp-wide instructions: if ANY row of the warp has to be rescaled,
                // every lane takes part, the others with a factor of one).  The last product is P V
                // of tile it - 1; none later can have been issued, since that needs this warp's P.
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
                    if (it > 0 && !mbar_wait(pv_done, (it - 1) & 1, &s_abort, status, 0x4b)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < HD / 64; c++) {
                        float t[32];
                        tmem_ld32_issue(to + c * 32, t);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) t[i] *= alpha;
                        tmem_st32(to + c * 32, t);
                    }
                }
                // pass 2: P in two bfloat16 terms, into tensor memory (two keys per 32-bit column), 32
                // scores at a time, read again (they are not kept over the exchange above: registers)
                // and overwritten by their own P: 16 columns of the first term, 16 of the second
                const float neg_m = m_new == -INFINITY ? 0.f : -m_new;     // no key seen yet: every p is 0 anyway
                float rs = 0.f, rs1 = 0.f;
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    float sc[32];
                    uint32_t hi[16], lo[16];
                    tmem_ld32_issue(ts + c * 32, sc);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float x0 = fmaf(sc[i], scale_log2, neg_m), x1 = fmaf(sc[i + 1], scale_log2, neg_m);
                        if (MASKED) {
                            if (!visible(jh + c * 32 + i)) x0 = -INFINITY;
                            if (!visible(jh + c * 32 + i + 1)) x1 = -INFINITY;
                        }
                        const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                        rs += p0, rs1 += p1;
                        const uint32_t h = pack_bf16(p0, p1);
                        hi[i / 2] = h;
                        lo[i / 2] = pack_bf16(p0 - __uint_as_float(h << 16), p1 - __uint_as_float(h & 0xffff0000u));
                    }
                    tmem_st16(ts + c * 32, hi);
                    tmem_st16(ts + c * 32 + 16, lo);
                }
                l = l * alpha + (rs + rs1);
                m = m_new;
                return true;
            };
            ok = full ? tile_softmax(std::false_type{}) : tile_softmax(std::true_type{});
            if (!ok) break;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);       // P is in place, and the output row is rescaled
        }
        // the row's sum: the two halves, in a fixed order
        if (ok) {
            x_sum[half][r] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(x_bar(qd));
            ok = mbar_wait(x_bar(qd), n_tiles & 1, &s_abort, status, 0x4c);
        }
        if (ok) ok = mbar_wait(pv_done, (n_tiles - 1) & 1, &s_abort, status, 0x4d);
        if (!ok) {
            if (lane == 0) {
                atomicOr(status, ST_WAIT_TIMEOUT);
                s_abort = 1;
            }
        } else {
            tc_fence_after();
            const float lsum = x_sum[0][r] + x_sum[1][r];
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)(tok0 + min(row, len - 1)) * nh + head) * HD +
                                                  half * (HD / 2));
#pragma unroll
            for (int c = 0; c < HD / 64; c++) {
                float t[32];
                tmem_ld32_issue(to + c * 32, t);               // (every lane of the warp takes part in the load)
                tmem_ld_wait();
                if (row < len) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 v;
                        v.x = pack_bf16(t[d] * inv, t[d + 1] * inv), v.y = pack_bf16(t[d + 2] * inv, t[d + 3] * inv);
                        v.z = pack_bf16(t[d + 4] * inv, t[d + 5] * inv), v.w = pack_bf16(t[d + 6] * inv, t[d + 7] * inv);
                        dst[(c * 32 + d) / 8] = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---- host side -------------------------------------------------------------------------------------
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

// bf16 [tokens, heads, hd] contiguous; box = 64 elements of one head for 128 tokens, 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, int tokens, int heads, int hd) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)heads * hd * 2};
    cuuint32_t box[3] = {64, 1, 128};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// one layer's keys (or values) in the cache, bf16 [pages][kv heads][64][hd], as rows of hd elements;
// box = 64 elements of the 64 rows of one (page, head), 128-byte swizzle
bool make_cache_map(CUtensorMap* map, const void* ptr, long long rows, int hd) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct CacheArgs {
    CUtensorMap tmK, tmV;
    const int *seq_start, *slots, *tables;
    int table_stride, ring, num_pages;
};

template <int HD>
int launch(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CacheArgs& c, void* out,
           const int* cu_seqlens, int num_seqs, int num_tokens, int nh, int nkv, int window, float scale, int* status,
           cudaStream_t stream) {
    constexpr int TILE_BYTES = (HD / 64) * 128 * 128;
    const int smem = 5 * TILE_BYTES + 1024 + 192;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(((num_tokens + QT - 1) / QT + num_seqs) * nh);
    return launch_pdl(attn_prefill_tc_kernel<HD>, grid, 320, (size_t)smem, stream, tmQ, tmK, tmV, c.tmK, c.tmV,
                      (__nv_bfloat16*)out, cu_seqlens, c.seq_start, c.slots, c.tables, c.table_stride, c.ring,
                      c.num_pages, num_seqs, nh, nkv, window, scale * 1.4426950408889634f, status);
}

int run(const void* q, const void* k, const void* v, CacheArgs& c, void* out, const int* cu_seqlens, int num_seqs,
        int num_tokens, int nh, int nkv, int hd, int window, float scale, int* status, cudaStream_t stream) {
    CUtensorMap tmQ, tmK, tmV;
    if (!make_map(&tmQ, q, num_tokens, nh, hd) || !make_map(&tmK, k, num_tokens, nkv, hd) ||
        !make_map(&tmV, v, num_tokens, nkv, hd))
        return -1;
    if (!c.seq_start) c.tmK = tmK, c.tmV = tmV;         // never used: no tile comes from the cache
    if (hd == 64)
        return launch<64>(tmQ, tmK, tmV, c, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, window, scale, status, stream);
    return launch<128>(tmQ, tmK, tmV, c, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, window, scale, status, stream);
}

}  // namespace

// q: [T, nh, hd], k, v: [T, nkv, hd], out: [T, nh * hd], all bfloat16, 16-byte aligned; sequences
// start at position 0.  Returns -1 (nothing launched) for a head size or an alignment this kernel
// does not take: the caller then uses moe_attention_prefill_bf16.
MOE_API int moe_attention_prefill_tc(const void* q, const void* k, const void* v, void* out, const int* cu_seqlens,
                                     int num_seqs, int num_tokens, int nh, int nkv, int hd, int window, float scale,
                                     int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || nh > 65535) return (int)cudaErrorInvalidValue;
    if (hd != 64 && hd != 128) return -1;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) != 0) return -1;
    CacheArgs c{};
    return run(q, k, v, c, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, hd, window, scale, status, stream);
}

// The same for sequences that go on from the cache: sequence i held seq_start[i] tokens before the
// step (0: a fresh one), whose keys and values lie in the pages of one layer's cache, k_cache and
// v_cache [num_pages][nkv][64][hd] bfloat16, listed in row slots[i] of `tables` (table_stride ints a
// row; position p in page table[(ring ? p % ring : p) / 64]).  The step's own keys and values are
// read from k and v, never from the cache.  Returns -1 for what this kernel does not take (then with
// nothing launched): the caller uses the kernel on the CUDA cores.
MOE_API int moe_attention_cached_tc(const void* q, const void* k, const void* v, const void* k_cache,
                                    const void* v_cache, void* out, const int* cu_seqlens, const int* seq_start,
                                    const int* slots, const int* tables, int table_stride, int ring, int page_size,
                                    int num_pages, int num_seqs, int num_tokens, int nh, int nkv, int hd, int window,
                                    float scale, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || nh > 65535 || num_pages <= 0) return (int)cudaErrorInvalidValue;
    if (!seq_start || !slots || !tables || !k_cache || !v_cache) return (int)cudaErrorInvalidValue;
    if (hd != 64 && hd != 128) return -1;
    if (page_size != 64 || ring % 64 != 0 || (long long)num_pages * nkv * 64 > 0x7fffffffLL) return -1;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
        return -1;
    CacheArgs c{};
    c.seq_start = seq_start, c.slots = slots, c.tables = tables;
    c.table_stride = table_stride, c.ring = ring, c.num_pages = num_pages;
    if (!make_cache_map(&c.tmK, k_cache, (long long)num_pages * nkv * 64, hd) ||
        !make_cache_map(&c.tmV, v_cache, (long long)num_pages * nkv * 64, hd))
        return -1;
    return run(q, k, v, c, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, hd, window, scale, status, stream);
}
