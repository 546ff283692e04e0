// Column sum for callers that must not allocate.  This entry point has no counterpart in the
// reference framework.
//
// Who needs it: code that runs where device allocation is forbidden or unsafe — inside a region
// whose memory budget was fixed up front, from a host callback or a thread that must not touch an
// allocator, or in an embedding application that hands this library raw device pointers and keeps
// its own memory manager.  itb_colsum() needs a caller-provided fp32 scratch buffer for its first
// stage; this variant keeps that scratch in a fixed array inside the library instead.
//
//   out[n] (+)= sum over rows of x[row, n]        x: [rows, N] bf16 or fp32, row stride ld
//
// Limits and rules
//   * ceil(rows / 128) * N must not exceed kItbColsumStaticMaxPartials (1 Mi floats = 4 MiB, enough
//     for 32768 rows x 4096 columns); larger requests return kItbErrScratchTooSmall and launch
//     nothing.  N and ld must be multiples of 8 (as for itb_colsum).
//   * The scratch array is part of the loaded library image: every GPU that loads the library holds
//     its 4 MiB until the process exits.
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress)
//     with that device current.  Make that first call outside any CUDA stream capture, and from one
//     thread per device: the cached address is written without a lock (concurrent first calls on one
//     device would each look up and store the same value, which is harmless but not synchronised).
//   * x must be 16-byte aligned, ld >= N, and rows at most 65535 * 128; otherwise -3 is returned.
//   * No cudaMalloc / cudaFree / allocating library routine is called, here or in the kernels.
//   * All calls on a device share the one array.  The first stage overwrites every partial sum it
//     later reads, so nothing needs clearing between calls, but two calls that can run at the same
//     time on the GPU (different streams) race on it: serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { kItbColsumStaticMaxPartials = 1 << 20, kItbErrScratchTooSmall = -100 };

// dtype: kItbF32 (0) or kItbBF16 (1).  accumulate != 0 adds to out instead of overwriting it.
// Returns 0, a negative argument error, or a CUDA error code.
int itb_colsum_static(const void* x, int dtype, long long ld, float* out, int rows, int N,
                      int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
