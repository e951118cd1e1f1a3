// Decode attention for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference engine (JGalego/Moe runs on the CPU and
// has no device memory to manage); it exists for hosts that drive this library from a context
// in which cudaMalloc is off limits: a serving process that has handed every free byte of the
// GPU to its own pool and must not let a dependency grow behind its back, a latency-critical
// loop that cannot afford the device-wide synchronisation an allocation implies, or a plugin
// interface whose contract forbids allocation inside the call.
//
// It computes exactly what moe_attention_decode computes (attention of one new token per
// sequence over the paged cache, split along the keys and merged), but the float32 scratch for
// the per-split partial results lives in a fixed array inside the library instead of being
// passed in.  Inputs and outputs are still the caller's.
//
// Limits and rules
//   * The scratch array holds MOE_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  Every GPU on which
//     the library is loaded keeps that much memory until the process exits.
//   * A call needs num_tokens * num_heads * nsplit * (head_dim + 2) floats.  A call that needs
//     more is refused with MOE_NOALLOC_TOO_LARGE and launches nothing; moe_noalloc_strerror
//     gives the message.
//   * The first call on a device looks up the device address of the array (one
//     cudaGetSymbolAddress with that device current).  The CUDA runtime may load this
//     library's device code lazily: that first lookup, and the first launch of each kernel
//     variant (one per element type, head size and "more than one query head per kv head"),
//     can make the driver place code and this array in device memory and synchronise.  So
//     warm up: make one call per variant you will use, on each device, before the region in
//     which nothing may be allocated and before any stream capture begins on the device.
//   * k_cache and v_cache must be 16-byte aligned; q and out aligned to their element type.
//     Anything else, zero or negative head counts included, is refused with
//     MOE_NOALLOC_BAD_ARGUMENT before anything is launched.
//   * No cudaMalloc, cudaFree or other allocating routine is called, by this library or through it.
//   * All calls on a device share the one array, and it keeps whatever the previous call left.
//     The kernels write every record they later read, so nothing has to be cleared between
//     calls; but two calls that overlap on the GPU (different streams, or one stream per thread)
//     race on it.  Serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

enum {
    MOE_NOALLOC_OK = 0,
    MOE_NOALLOC_TOO_LARGE = -2,     // the call needs more scratch than the library holds
    MOE_NOALLOC_BAD_ARGUMENT = -3,  // a size or a head layout the kernels do not take
    MOE_NOALLOC_NO_DEVICE = -4,     // the device address of the scratch array could not be obtained
};

// Same arguments as moe_attention_decode without `partial`.  dt: 0 = float32, 1 = bfloat16.
// Returns MOE_NOALLOC_OK, one of the codes above, or a positive cudaError_t from the launch.
int moe_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, int dt,
                                 const int* seq_of_token, const int* pos, const int* slots, const int* tables,
                                 int table_stride, int ring, int page_size, int num_pages, int num_tokens,
                                 int num_heads, int num_kv_heads, int head_dim, int window, float scale, int nsplit,
                                 int* status, cudaStream_t stream);

// Floats of scratch a call with these sizes needs.
long long moe_attention_decode_noalloc_need(int num_tokens, int num_heads, int head_dim, int nsplit);

// A sentence for a code returned by moe_attention_decode_noalloc.
const char* moe_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
