// Allocation-free attention backward.
//
// This entry point has no counterpart in the reference engine: the reference allocates every
// scratch buffer once through its buffer manager, while arb_attn_bwd expects its caller to
// bring the per-row softmax statistic buffer ("delta", B*H*T floats).  Some callers cannot
// provide device memory at the point of the call: a C, C++ or Rust host that links this
// library without a caching allocator, a serving thread that must never block (cudaMalloc
// synchronises the whole device and may fail when memory is fragmented), or code that runs
// inside somebody else's callback where creating allocations is forbidden.  For them the
// scratch lives in a fixed array inside the library image.
//
//   * Capacity: B*H*T <= ARB_ATTN_NOALLOC_MAX_ROWS (1 Mi rows = 4 MiB of device memory that
//     every GPU loading this library holds until the process exits).  Larger problems are
//     rejected with ARB_ERR_NOALLOC_TOO_LARGE before anything is launched.
//   * The first call on each device looks up the device address of the array (with that device
//     current) and caches it; make that first call outside any stream capture.  The cache is
//     atomic: host threads may make their first calls concurrently.
//   * `stream` must belong to the device that is current in the calling thread: the array of
//     THAT device is used, and a stream of another device fails at launch with a CUDA error
//     code as the return value.
//   * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.  Inputs and
//     outputs are still the caller's.
//   * All calls on one device share the one array and it keeps whatever the previous call left
//     there; the kernels overwrite every element they later read, so nothing has to be cleared.
//     Two calls whose kernels overlap on the GPU (different streams) race on it: serialise them.
#pragma once
#include <cuda_runtime.h>

#define ARB_ATTN_NOALLOC_MAX_ROWS (1 << 20)
#define ARB_ERR_NOALLOC_TOO_LARGE (-20)
#define ARB_ERR_NOALLOC_SYMBOL (-21)

extern "C" int arb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                    const float* lse, void* dq, void* dk, void* dv, int B, int T, int H,
                                    long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
                                    long long lddq, long long lddk, long long lddv, int window, float scale,
                                    int* err_flag, cudaStream_t stream);
