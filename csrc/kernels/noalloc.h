// Allocation-free entry point for exact top-k selection with error feedback.
//
// This entry point has no counterpart in the reference project.  It exists for
// callers that must not allocate device memory at all: a host process whose own
// memory pool has already claimed the whole GPU (a second cudaMalloc would fail
// or fragment its pool), code that runs where taking an allocator lock is not
// allowed (for example from inside another framework's hook or callback that
// already holds that lock), and plain C callers that link this library without
// torch and have no caching allocator to draw scratch from.
//
// What it does: the same selection as the regular top-k path
// (adjusted = grad + residual; pick the k entries of largest magnitude, ties to
// the lower index; write them as (u32 index, f32 value) pairs sorted by index;
// residual = adjusted with the picked entries zeroed), but the kernels' scratch
// (radix histograms, selection state, per-block counters: about 53 KB of a 64 KB array) lives in
// one fixed device array that is part of the library image instead of being
// allocated per call.
//
// Rules for callers:
//  * grad, residual and pairs_out are device pointers the caller owns:
//    n floats, n floats (read and written) and k * 8 bytes.
//  * The device that holds these buffers must be the current device of the calling thread
//    (cudaSetDevice): each device has its own copy of the scratch array and the call uses the
//    current device's.  Buffers on another device are rejected with code 1.
//  * Limits: 1 <= k <= n <= MCCL_NOALLOC_TOPK_MAX_N.  Anything else is rejected
//    with a non-zero return code and a message (mccl_noalloc_last_error()).
//  * The first call on each device looks up the address of the scratch array
//    (a host-side step, once per device).  Make that first call before you start
//    capturing a stream on that device.
//  * All calls on one device share the one scratch array, and it keeps whatever
//    the previous call left in it; every call re-initialises the parts it needs.
//    Two calls whose kernels can overlap on the GPU (different streams without
//    ordering between them) would corrupt each other's counters: keep calls on
//    one stream or order them yourself.
//  * Every GPU that loads the library carries the array until the process exits.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once

#include <cuda_runtime_api.h>

#define MCCL_NOALLOC_TOPK_MAX_N 2147483647LL

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success.  1: bad argument / size beyond the limit, 2: CUDA error
// (set-up or launch).  The kernels are enqueued on `stream`; nothing synchronises.
int mccl_topk_select_noalloc(const float* grad, float* residual, long long n, long long k, void* pairs_out,
                             cudaStream_t stream);

// Message of the last failure on the calling thread ("" if none).
const char* mccl_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
