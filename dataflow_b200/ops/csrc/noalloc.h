// Allocation-free entry point (C ABI).
//
// This entry point has no counterpart in the reference framework.  It exists for callers that
// cannot allocate device memory at the moment they need the kernel: code running while a CUDA
// stream is being captured into a graph, a host thread that sits inside a library's callback and
// must not re-enter the CUDA allocator, or an embedding application that hands this library a fixed
// memory budget and forbids cudaMalloc after start-up.  The regular RMSNorm backward needs a
// scratch buffer for its per-CTA weight-gradient partial sums, which its caller has to allocate;
// this variant keeps that scratch in a device array that is part of the library image, so the
// caller passes only inputs and outputs.
#pragma once
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest row width the built-in scratch covers.  Wider rows are refused (return code -1).
#define DFB_NOALLOC_RMSNORM_MAX_COLS 8192
// Bytes of device memory the scratch array occupies on every GPU that loads this library
// (296 partial rows x 2 planes x DFB_NOALLOC_RMSNORM_MAX_COLS floats); it is held until the process exits.
#define DFB_NOALLOC_RMSNORM_SCRATCH_BYTES (296ull * 2ull * DFB_NOALLOC_RMSNORM_MAX_COLS * 4ull)

// RMSNorm backward without any allocation:
//   dx = rstd * (w*dy - xhat * mean(w*dy*xhat))      (bf16, rows x cols)
//   dw = sum over rows of dy * xhat                   (bf16, cols)       xhat = x * rstd
// dy, x, dx: bf16 (rows x cols, contiguous); w, dw: bf16 (cols); rstd: fp32 (rows), as produced by the forward.
// All pointers are device pointers on the current device; work is enqueued on `stream`.
// dy, x, w, dx and dw must be 16-byte aligned (the kernels move 16-byte vectors; since cols is a
// multiple of 8 every row then is too) and rstd 4-byte aligned: a view that starts in the middle
// of a caller's arena has to respect this.
//
// Return value: 0 on success; -1 if cols is not a multiple of 8 or exceeds DFB_NOALLOC_RMSNORM_MAX_COLS
// or rows < 0; -2 if a pointer is null; -3 if the CUDA runtime reported an error (one already pending
// on this thread when the call came in, in which case nothing is launched, or one from set-up or launch);
// -4 if a pointer is misaligned.
// dfb_noalloc_strerror() turns the code into text.
//
// The first call on each device looks up the device address of the scratch array
// (cudaGetSymbolAddress).  Make that first call outside of any stream capture.  The address is
// cached for the life of the process: after cudaDeviceReset the cache is stale and this entry point
// must not be used again in that process.
// The call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
// Every call on a device shares the one scratch array.  The kernel overwrites the part it uses
// before reading it, so stale contents from an earlier call are harmless and nothing needs to be
// cleared; but two calls whose kernels overlap in time on the same GPU (different streams) would
// race on it — serialise them.
int dfb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                            int rows, int cols, cudaStream_t stream);

const char* dfb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
