// Shared device / host helpers for the PowerSGD sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "psgd_types.h"

#define PSGD_API extern "C" __attribute__((visibility("default")))

// ---- host-side error plumbing -------------------------------------------------------------
void psgd_set_error(const char* fmt, ...);
#define PSGD_CUDA_OK(expr)                                                          \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess) {                                                        \
      psgd_set_error("%s:%d %s -> %s", __FILE__, __LINE__, #expr, cudaGetErrorString(_e)); \
      return (int)_e;                                                               \
    }                                                                               \
  } while (0)

// Status word written by kernels whose waits ran out. 0 = fine.
enum PsgdStatus : int {
  PSGD_OK = 0,
  PSGD_TIMEOUT_PEER_BARRIER = 2,
  PSGD_TIMEOUT_MBARRIER = 3,
  PSGD_BAD_ARGUMENT = 4,
};

// ---- device helpers -----------------------------------------------------------------------
__device__ __forceinline__ uint64_t psgd_globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float psgd_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double psgd_warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int psgd_atom_add_acqrel_gpu(int* p, int v) {
  int old;
  asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

static inline int psgd_ceil_div(int a, int b) { return (a + b - 1) / b; }
