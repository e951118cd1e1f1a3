// Attention of whole prompts (every sequence of the step starts at position 0): the
// tensor-core kernel of the bfloat16 path.
//
// Formulas as in attention_generic.cu (reference: src/model.rs:794-827): causal, optional
// window [p + 1 - w, p], scale 1/sqrt(d), kv head = head / (heads / kv_heads).  Queries,
// keys and values of the step are read from the step's own buffers (nothing is read from
// the cache, so it may be appended before or after).  Q K^T and P V run on the tensor
// cores (mma.sync m16n8k16, bfloat16 inputs, float32 accumulation); scores, the running
// maximum and sum, and the output accumulator are float32; P enters the second product as
// two bfloat16 terms (head and remainder), i.e. with 16 bits.
//
// One CTA of 4 warps takes 64 query rows of one (sequence, head); it walks the key tiles of
// 64 that the causal window allows, double-buffered with cp.async.  Rows are padded by 16
// bytes in shared memory so that ldmatrix is conflict-free for every head size.
// Head sizes 16, 32, 64 and 128; others use the plain kernel.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, THREADS = 128;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                    const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ cu_seqlens, int num_seqs, int nh, int nkv, int window, float scale_log2) {
    constexpr int ROW = HD * 2 + 16;                     // padded row bytes
    constexpr int CPR = HD / 8;                          // 16-byte chunks per row
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ int s_seq, s_tile;
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sK = sQ + BM * ROW;                   // two buffers
    const uint32_t sV = sK + 2 * BN * ROW;               // two buffers

    // which (sequence, query tile): tiles are numbered sequence by sequence
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, seq = -1;
        for (int s = 0; s < num_seqs; s++) {
            const int tiles = (cu_seqlens[s + 1] - cu_seqlens[s] + BM - 1) / BM;
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
    const int tok0 = cu_seqlens[seq], len = cu_seqlens[seq + 1] - tok0;
    // heavier tiles (later rows see more keys) first
    const int q_tile = (len + BM - 1) / BM - 1 - s_tile;
    const int q0 = q_tile * BM;
    const int head = blockIdx.y, kvh = head / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- load Q tile (rows past the sequence are clamped; their results are not written) ----
    for (int c = threadIdx.x; c < BM * CPR; c += THREADS) {
        const int r = c / CPR, ch = c % CPR;
        const int row = min(q0 + r, len - 1);
        cp_async16(sQ + r * ROW + ch * 16, q + ((size_t)(tok0 + row) * nh + head) * HD + ch * 8);
    }
    cp_async_commit();

    const int q_last = min(q0 + BM, len) - 1;
    const int kv_lo = window > 0 ? max(0, q0 + 1 - window) / BN : 0;
    const int kv_hi = q_last / BN;                       // inclusive
    auto load_kv = [&](int tile, int buf) {
        const int j0 = tile * BN;
        for (int c = threadIdx.x; c < BN * CPR; c += THREADS) {
            const int r = c / CPR, ch = c % CPR;
            const int row = min(j0 + r, len - 1);
            const size_t g = ((size_t)(tok0 + row) * nkv + kvh) * HD + ch * 8;
            cp_async16(sK + (buf * BN + r) * ROW + ch * 16, k + g);
            cp_async16(sV + (buf * BN + r) * ROW + ch * 16, v + g);
        }
        cp_async_commit();
    };
    load_kv(kv_lo, 0);

    // Q fragments of this warp's 16 rows: HD / 16 k-steps x 4 registers
    uint32_t qf[HD / 16][4];
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
        const int r = warp * 16 + (lane & 15), cb = ks * 32 + (lane >> 4) * 16;
        ldsm_x4(sQ + r * ROW + cb, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int row_a = q0 + warp * 16 + (lane >> 2), row_b = row_a + 8;     // the two query rows of this thread

    for (int tile = kv_lo; tile <= kv_hi; tile++) {
        const int buf = (tile - kv_lo) & 1;
        if (tile + 1 <= kv_hi) {
            load_kv(tile + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t kb = sK + buf * BN * ROW, vb = sV + buf * BN * ROW;

        // ---- S = Q K^T: 8 key tiles of 8 ---------------------------------------------------
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
#pragma unroll
            for (int np = 0; np < BN / 16; np++) {          // two key tiles per ldmatrix.x4
                uint32_t b0, b1, b2, b3;
                const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3), cb = ks * 32 + ((lane >> 3) & 1) * 16;
                ldsm_x4(kb + r * ROW + cb, b0, b1, b2, b3);
                mma_bf16(s[2 * np], qf[ks], b0, b1);
                mma_bf16(s[2 * np + 1], qf[ks], b2, b3);
            }
        }
        // ---- mask, online softmax (base 2) ----------------------------------------------------
        const int j0 = tile * BN;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < BN / 8; i++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int j = j0 + i * 8 + (lane & 3) * 2 + (e & 1);
                const int row = (e & 2) ? row_b : row_a;
                const bool ok = j <= row && j < len && (window <= 0 || j >= row + 1 - window);
                const float x = ok ? s[i][e] * scale_log2 : -INFINITY;
                s[i][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m[h], mx[h]);
            alpha[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new);
            m[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        // P as A fragments (4 k-steps of 16 keys), split into a bfloat16 head and a bfloat16 remainder:
        // together they carry 16 bits of P, so that a prompt and a token-by-token replay of the same
        // sequence differ by float32 rounding only
        uint32_t pf[BN / 16][4], pr[BN / 16][4];
#pragma unroll
        for (int i = 0; i < BN / 8; i++) {
            float pvals[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float mm = m[e >> 1];
                const float pe = (mm == -INFINITY) ? 0.f : exp2f(s[i][e] - mm);
                pvals[e] = pe;
                rs[e >> 1] += pe;
            }
            // accumulator layout of tile i -> A fragment halves of k-step i / 2
            float rem[4];
#pragma unroll
            for (int e = 0; e < 4; e++) rem[e] = pvals[e] - __bfloat162float(__float2bfloat16_rn(pvals[e]));
            pf[i / 2][(i & 1) * 2] = pack_bf16(pvals[0], pvals[1]);
            pf[i / 2][(i & 1) * 2 + 1] = pack_bf16(pvals[2], pvals[3]);
            pr[i / 2][(i & 1) * 2] = pack_bf16(rem[0], rem[1]);
            pr[i / 2][(i & 1) * 2 + 1] = pack_bf16(rem[2], rem[3]);
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            l[h] = l[h] * alpha[h] + rs[h];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            o[i][0] *= alpha[0], o[i][1] *= alpha[0];
            o[i][2] *= alpha[1], o[i][3] *= alpha[1];
        }
        // ---- O += P V ----------------------------------------------------------------------------
#pragma unroll
        for (int ks = 0; ks < BN / 16; ks++) {               // 16 keys per step
#pragma unroll
            for (int dp = 0; dp < HD / 16; dp++) {           // two dim tiles of 8 per ldmatrix.x4.trans
                uint32_t b0, b1, b2, b3;
                const int r = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, cb = dp * 32 + (lane >> 4) * 16;
                ldsm_x4_t(vb + r * ROW + cb, b0, b1, b2, b3);
                mma_bf16(o[2 * dp], pf[ks], b0, b1);
                mma_bf16(o[2 * dp + 1], pf[ks], b2, b3);
                mma_bf16(o[2 * dp], pr[ks], b0, b1);
                mma_bf16(o[2 * dp + 1], pr[ks], b2, b3);
            }
        }
        __syncthreads();                                     // this buffer is refilled two tiles on
    }

    // ---- normalise and store ---------------------------------------------------------------------
    const float inv_a = l[0] > 0.f ? 1.f / l[0] : 0.f, inv_b = l[1] > 0.f ? 1.f / l[1] : 0.f;
#pragma unroll
    for (int i = 0; i < HD / 8; i++) {
        const int d = i * 8 + (lane & 3) * 2;
        if (row_a < len) {
            __nv_bfloat162 w = __floats2bfloat162_rn(o[i][0] * inv_a, o[i][1] * inv_a);
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + row_a) * nh + head) * HD + d) = w;
        }
        if (row_b < len) {
            __nv_bfloat162 w = __floats2bfloat162_rn(o[i][2] * inv_b, o[i][3] * inv_b);
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + row_b) * nh + head) * HD + d) = w;
        }
    }
}

template <int HD>
int launch(const void* q, const void* k, const void* v, void* out, const int* cu_seqlens, int num_seqs,
           int num_tokens, int nh, int nkv, int window, float scale, cudaStream_t stream) {
    constexpr int ROW = HD * 2 + 16;
    const int smem = (BM + 4 * BN) * ROW;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((num_tokens + BM - 1) / BM + num_seqs, nh);
    attn_prefill_kernel<HD><<<grid, THREADS, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, cu_seqlens,
        num_seqs, nh, nkv, window, scale * 1.4426950408889634f);
    return launch_status();
}

}  // namespace

// q: [T, nh, hd], k, v: [T, nkv, hd], out: [T, nh * hd], all bfloat16; sequences start at position 0.
// Returns -1 for a head size this kernel does not take.
MOE_API int moe_attention_prefill_bf16(const void* q, const void* k, const void* v, void* out, const int* cu_seqlens,
                                       int num_seqs, int num_tokens, int nh, int nkv, int hd, int window, float scale,
                                       cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || nh > 65535) return (int)cudaErrorInvalidValue;
    switch (hd) {
        case 16: return launch<16>(q, k, v, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, window, scale, stream);
        case 32: return launch<32>(q, k, v, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, window, scale, stream);
        case 64: return launch<64>(q, k, v, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, window, scale, stream);
        case 128: return launch<128>(q, k, v, out, cu_seqlens, num_seqs, num_tokens, nh, nkv, window, scale, stream);
        default: return -1;
    }
}
