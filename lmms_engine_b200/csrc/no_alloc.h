// Allocation-free entry point of the native library.
//
// This entry point has no counterpart in the reference (which has no native code at all).
// It exists for hosts that embed these kernels in a place where device memory must not be
// allocated: an execution callback of another runtime (an inference-engine plugin's
// enqueue function, a custom call inside another framework's executor, a communication
// plugin), or a service with a fixed device-memory budget.  There cudaMalloc is either
// forbidden outright or unacceptable because it synchronises the whole device, and
// torch's caching allocator is not available to draw the scratch buffer from.
//
// b200_rmsnorm_bwd_noalloc computes exactly what b200_norm_bwd computes for RMSNorm
// (dx, and dw reduced over rows) but takes its fp32 partial-sum scratch from a fixed
// array that lives inside the library image instead of from the caller.
//
//  * Limits: H <= B200_NOALLOC_MAX_H (4096) and H % 8 == 0.  Larger rows are rejected with
//    B200_NOALLOC_ERR_TOO_LARGE and nothing is launched.  The array is
//    B200_NOALLOC_MAX_PARTS x B200_NOALLOC_MAX_H floats = 8 MiB; every GPU that loads the
//    library carries it until the process exits.
//  * The first call on each device looks the array's device address up (once per device,
//    with that device current).  Make that first call outside of any stream capture.
//  * All calls share the one array.  Each call overwrites the part it uses before reading
//    it, so stale contents of an earlier call are harmless, but two calls that overlap on
//    the GPU (different streams, no ordering between them) race on it: order them.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define B200_NOALLOC_MAX_H 4096
#define B200_NOALLOC_MAX_PARTS 512
#define B200_NOALLOC_ERR_TOO_LARGE (-20)
#define B200_NOALLOC_ERR_SETUP (-21)

#ifdef __cplusplus
extern "C" {
#endif

// dy, x, dx: bf16 [rows, H]; w: bf16 [H]; rstd: fp32 [rows]; dw: fp32 [H] (overwritten).
// Returns 0 on a successful launch, a negative code otherwise.
int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const void* rstd, void* dx, void* dw,
                             int rows, int H, float w_offset, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
