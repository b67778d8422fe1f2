// Entry points of libtft_kernels.so that never allocate device memory.
//
// This header has no counterpart in the reference (pytorch-labs/torchft contains no GPU
// code at all).  It exists for callers of this library that are not in a position to
// allocate: code running where cudaMalloc / cudaFree are off limits (inside another
// allocator's callback, in a plug-in that only ever receives raw device pointers and a
// stream, or wherever an allocation could synchronise the device at a bad moment).
//
// The one entry point declared here is a variant of the RMSNorm backward kernel.  The
// regular entry point (tft_rmsnorm_bwd) takes a caller-provided fp32 scratch buffer for
// the per-block partial sums of the weight gradient; this variant uses a fixed array inside
// the library's device image instead.
//
//   * Size limit: dim <= tft_rmsnorm_bwd_noalloc_max_dim() (8192).  Larger sizes are rejected
//     with return code -10 and a message on stderr.  The array occupies 4.6 MiB on every GPU
//     that loads the library, for the life of the process.
//   * Sharing: every call on a device uses the same array, which keeps whatever the last
//     call left in it (the kernel rewrites all of what it reads, so nothing needs clearing).
//     Calls that overlap on the GPU race; keep them on one stream or order them.
//   * First call: the first call on each device resolves the array's device address; make
//     it before any stream capture begins.
//   * Device: the array is per GPU and is looked up for the CURRENT device, so the current
//     device must be the one `stream` belongs to (cudaSetDevice first, as for any launch).  A
//     stream of another device is rejected with return code -11.
//   * Threads: any host thread may call; the per-device address cache is atomic, and two
//     threads that race on the first call both store the same value.
//   * No cudaMalloc, cudaFree or allocating library call is made.
#pragma once

#include <cuda_runtime.h>

#if defined(__GNUC__)
#define TFT_NOALLOC_API __attribute__((visibility("default")))
#else
#define TFT_NOALLOC_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

// Largest supported row width.
TFT_NOALLOC_API int tft_rmsnorm_bwd_noalloc_max_dim(void);

// dy, x, dres (optional), dx: [rows, dim] bf16;  w, dw: [dim] bf16;  rstd: [rows] fp32.
//   dx = d loss / d x of y = x * rstd * w  (+ dres if given)
//   dw = sum over rows of dy * x * rstd    (added to dw when accumulate != 0)
// Returns 0 on success, -10 if dim is too large, -11 if `stream` is not a stream of the current
// device, another non-zero code on failure.
TFT_NOALLOC_API int tft_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, void* dw, int rows, int dim, int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
