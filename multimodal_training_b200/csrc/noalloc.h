// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference (the reference is pure Python over
// library kernels and never exposes a C ABI).
//
// Who needs it: callers that hold raw device pointers and are not allowed to allocate device
// memory when they call us -- for example a plugin running inside another runtime's memory pool,
// a real-time or embedded host that fixes its device memory map at start-up, or code running
// inside a region where cudaMalloc would synchronise the device or fail (a tightly budgeted
// process that has already handed all free memory to its own allocator).  The regular RMSNorm
// backward (mmt_rmsnorm_bwd) needs an fp32 scratch buffer for its per-CTA partial sums of the
// weight gradient and leaves it to the caller to allocate one; this variant carries its scratch
// inside the library instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the library reserves: 2^21 floats (8 MiB), held by every GPU that loads the
// library, from load until the process exits.
#define MMT_NOALLOC_SCRATCH_FLOATS (1 << 21)
// Largest row width (columns) accepted; the same limit as mmt_rmsnorm_bwd.
#define MMT_NOALLOC_MAX_COLS 8192

// RMSNorm backward without any allocation:
//   dx[r, :] = rstd[r] * (dy*w - x * rstd[r]^2 * mean(dy*w*x))        (bf16, [rows, cols])
//   dw[:]    = sum_r dy[r, :] * x[r, :] * rstd[r]                      (bf16, [cols]; added to the
//                                                                       old dw if accumulate_dw != 0)
// dy, x, dx: bf16 [rows, cols] contiguous; w, dw: bf16 [cols]; rstd: fp32 [rows] (from the forward).
// All pointers are device pointers supplied by the caller; `stream` is a cudaStream_t (0 = default).
//
// Returns 0 on success.  Errors (nothing is launched): -2 cols not a multiple of 8; -5 cols <= 0 or larger
// than MMT_NOALLOC_MAX_COLS, or rows outside [0, 2^31); -6 the scratch address could not be resolved
// on the current device.  A message naming the limit is written to stderr for -5 and -6.
//
// Set-up: the first call on each device resolves the device address of the built-in scratch array
// (cudaGetSymbolAddress with that device current) and caches it; make that first call before any
// stream capture begins.  The function never calls cudaMalloc, cudaFree or any allocating library
// routine.
//
// Sharing: every call on a device uses the same scratch array, which keeps the previous call's
// contents.  Nothing in it has to start at zero (each launch overwrites every partial sum it later
// reads), but two calls that overlap on the GPU (different streams, no ordering between them) race
// on it and give wrong dw; order such calls with events or use one stream.
int mmt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                            long rows, int cols, int accumulate_dw, void* stream);

#ifdef __cplusplus
}
#endif
