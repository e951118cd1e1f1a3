// Shared helpers for every kernel file: storage-type conversion, warp and block
// reductions, the device status word, and launch error reporting.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MOE_API extern "C" __attribute__((visibility("default")))

// Storage type tags passed across the C boundary.
enum : int { DT_F32 = 0, DT_BF16 = 1 };

// Bits of the device status word.  Kernels OR them in and carry on with a safe
// value; the host reads the word after a step and raises.
enum : int {
    ST_BAD_TOKEN = 1,     // token id outside the vocabulary
    ST_BAD_PAGE = 2,      // page table entry outside the pool
    ST_BAD_EXPERT = 4,    // routing produced an expert id outside [0, E)
    ST_WAIT_TIMEOUT = 8,  // a bounded wait on a barrier ran out
    ST_BAD_ROW = 16,      // gather index outside its tensor
};

// status[1]: where the FIRST bounded wait ran out (a site number, see WAIT_SITES in ops/core.py); 0 if none.
__device__ __forceinline__ void wait_ran_out(int* status, int site) {
    if (status) {
        atomicOr(status, ST_WAIT_TIMEOUT);
        atomicCAS(status + 1, 0, site);
    }
}
// Nanoseconds of the device's global timer: bounds a wait by time, not by a number of tries (one
// try of an mbarrier wait may itself suspend the thread for a while).
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// A wait on a barrier inside a kernel may take this long (microseconds) before it gives up.  No
// wait of a healthy kernel comes near it; it only turns a hang into an error.
constexpr uint32_t WAIT_LIMIT_US = 2000000u;

__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_f(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `red` is shared memory of at least 32 floats.  All threads get
// the result.  Order of additions is fixed, so the result is reproducible.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch ------------------------------------------------------
// A decode step is a chain of short kernels.  Launched with the programmatic-serialization
// attribute, a kernel may be scheduled while its predecessor in the stream is still running;
// it must then call pdl_wait() before it reads anything the predecessor wrote or writes
// anything the predecessor may still read (the wait returns once the predecessor grid has
// completed and its memory operations are visible).  pdl_launch_dependents() lets the NEXT
// kernel be scheduled early in the same way.  Both are no-ops for a kernel launched normally.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// The usual opening of a kernel in the chain: wait for the predecessor, then let the successor
// be scheduled.  In this order only ONE successor is ever resident ahead of the running kernel;
// releasing the successor before the wait lets the whole chain pile up on the SMs as waiting
// CTAs, which takes room from a running kernel that needs several waves.
__device__ __forceinline__ void pdl_sync() {
    pdl_wait();
    pdl_launch_dependents();
}

// Ask for the 128-byte line of `p` in L2.  Weights (and cache contents of earlier steps) do not
// depend on the predecessor, so a kernel may ask for them BEFORE pdl_wait(): the memory latency
// then passes while the predecessor finishes.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// One switch per shared library (set through moe_set_pdl / moe_tc_set_pdl).
inline int g_pdl_enabled = 1;

// Launch `kernel` with the attribute (if enabled).  ONLY for kernels that call pdl_wait().
template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_enabled ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with thread-block clusters of `cluster_z` CTAs along grid.z (1: no clusters).
template <typename... KArgs, typename... Args>
static inline int launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     int cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1, attr[n].val.clusterDim.y = 1, attr[n].val.clusterDim.z = (unsigned)cluster_z;
        n++;
    }
    if (g_pdl_enabled) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- thread-block clusters -------------------------------------------------------------------
__device__ __forceinline__ unsigned cl_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// all threads of all CTAs of the cluster; orders shared-memory writes before it against reads after
__device__ __forceinline__ void cl_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the 32-bit word at the same shared-memory address in CTA `rank` of the cluster
__device__ __forceinline__ unsigned cl_peer_u32(const void* local, unsigned rank) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(local);
    unsigned pa, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(pa) : "r"(a), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(pa) : "memory");
    return v;
}

// The rotation of one pair (a at i, b at i + half) by the angle whose cosine and sine are cs, sn:
// products and sums rounded one by one, as the reference's plain 32-bit code does (no fused
// multiply-add), and the same in every kernel that rotates, so that they agree to the bit.
__device__ __forceinline__ float rot_lo(float a, float b, float cs, float sn) {
    return __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
}
__device__ __forceinline__ float rot_hi(float a, float b, float cs, float sn) {
    return __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
}

// Logical position -> (page, offset) of a paged, optionally ring-shaped, cache.
//   ring:  positions wrap at `ring` (a multiple of the page size); 0 = no wrap
//   table: the sequence's page list; page p holds `page_size` consecutive positions
// One layer's keys (or values) are laid out [page][kv_head][offset][head_dim].
struct CachePos {
    int page, off;
};
__device__ __forceinline__ CachePos cache_pos(int pos, int ring, const int* table, int page_size, int num_pages,
                                              int* status) {
    int r = ring > 0 ? pos % ring : pos;
    int page = table[r / page_size];
    if (page < 0 || page >= num_pages) {
        if (status) atomicOr(status, ST_BAD_PAGE);
        page = 0;
    }
    CachePos c;
    c.page = page;
    c.off = r % page_size;
    return c;
}
__device__ __forceinline__ size_t cache_index(CachePos c, int kv_head, int num_kv_heads, int page_size, int head_dim) {
    return (((size_t)c.page * num_kv_heads + kv_head) * page_size + c.off) * head_dim;
}
