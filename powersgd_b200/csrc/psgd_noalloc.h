// Allocation-free entry point of the native library.
//
// This entry point has no counterpart in the reference implementation (which is pure Python
// and leaves all memory management to PyTorch). It exists for callers that must not, or
// cannot, allocate device memory at the moment they need a factor product:
//   * code running while the framework's caching allocator is frozen or being recorded (a
//     cudaMalloc there would either fail or synchronise the whole device and stall every stream
//     that overlaps communication with the backward pass);
//   * communication hooks and real-time loops with a fixed memory budget, where any hidden
//     allocation counts as a defect;
//   * embedders that link this library without PyTorch and have no allocator to hand us.
//
// The grouped product kernels of this library need two pieces of scratch memory: partial sums
// of row blocks and arrival counters. Here that scratch is a fixed array that is part of the
// library image itself, so every GPU that loads the library holds PSGD_NOALLOC_SCRATCH_BYTES
// (4 MiB + 16 KiB) from load until exit, and the caller passes only inputs and outputs.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSGD_NOALLOC_MAX_RANK 8                     /* factor columns */
#define PSGD_NOALLOC_PARTIAL_FLOATS (1 << 20)       /* 4 MiB of partial sums */
#define PSGD_NOALLOC_MAX_COL_BLOCKS 4096            /* m <= 128 * 4096 columns */
#define PSGD_NOALLOC_SCRATCH_BYTES (PSGD_NOALLOC_PARTIAL_FLOATS * 4 + PSGD_NOALLOC_MAX_COL_BLOCKS * 4)

// Q[m, r] = M^T P for ONE row-major matrix M[n, m] (contiguous rows) and P[n, r], r <= 8,
// all float32 device pointers valid on the current device; Q is overwritten.
//
// Calls no cudaMalloc / cudaFree and no allocating library routine. Limits: r <= 8,
// ceil(m / 128) <= 4096, and ceil(m / 128) * ceil(n / 256) * 128 * rt <= 2^20 where rt is r
// rounded up to a power of two; anything larger is rejected with a non-zero return code and a
// message retrievable through psgd_last_error(), and nothing is launched.
//
// The first call on each device looks up the device address of the built-in scratch array
// (cudaGetSymbolAddress) and caches it; make that first call outside of any stream capture.
//
// All calls share the one scratch array. It keeps the previous call's contents; the counters
// are cleared on the stream at the start of every call. Two calls whose kernels may overlap on
// the GPU (different streams, or different host threads without ordering) race on it: order
// them on one stream or with events.
//
// Returns 0 on success, a CUDA error code or -1 otherwise.
int psgd_matmul_tn_noalloc(const float* M, int n, int m, const float* P, int r, float* Q, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
