// Consumer side of the in-kernel factor all-reduce, and a stand-alone one-launch all-reduce
// built from the same primitives (collective micro-benchmark, tests).
#include "psgd_comm.cuh"

constexpr int RED_THREADS = 256;

// out[i] = sum over ranks (in rank order) of this epoch's slot[r][i], i < total; each word is
// polled until its tag shows the epoch. Optionally writes a second copy. Replaces the blocking
// NCCL all_reduce of the reference (powersgd/powersgd.py:205-209).
__global__ void __launch_bounds__(RED_THREADS) psgd_factor_reduce_kernel(const PsgdCommDev* comm, long long total,
                                                                           float* __restrict__ out1,
                                                                           float* __restrict__ out2) {
  const PsgdCommDev c = *comm;
  const int e1 = *c.epoch + 1;
  bool ok = true;
  const long long stride = (long long)gridDim.x * RED_THREADS;
  for (long long i = (long long)blockIdx.x * RED_THREADS + threadIdx.x; i < total; i += stride) {
    const float s = psgd_comm_reduce(c, e1, i, ok);
    out1[i] = s;
    if (out2) out2[i] = s;
  }
  psgd_comm_close_epoch(c, e1);
}

PSGD_API int psgd_factor_reduce_launch(const void* comm, long long total, float* out1, float* out2,
                                       cudaStream_t stream) {
  if (total <= 0) return 0;
  long long blocks = (total + RED_THREADS * 2 - 1) / (RED_THREADS * 2);
  if (blocks > 296) blocks = 296;
  psgd_factor_reduce_kernel<<<(int)blocks, RED_THREADS, 0, stream>>>((const PsgdCommDev*)comm, total, out1, out2);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// All-reduce (SUM, times `scale`) of a contiguous buffer in a single launch: every thread pushes
// its elements to all peers, then polls the same elements of the own arena and adds them in rank
// order. CTAs do not depend on each other, so the grid may be of any size.
__global__ void __launch_bounds__(RED_THREADS) psgd_allreduce_oneshot_kernel(const PsgdCommDev* comm,
                                                                               const float* __restrict__ in,
                                                                               float* __restrict__ out, long long total,
                                                                               float scale) {
  const PsgdCommDev c = *comm;
  const int e1 = *c.epoch + 1;
  const long long stride = (long long)gridDim.x * RED_THREADS;
  const long long start = (long long)blockIdx.x * RED_THREADS + threadIdx.x;
  for (long long i = start; i < total; i += stride) {
    const float v = in[i];
    for (int p = 0; p < c.world; ++p) psgd_comm_store(psgd_comm_slot(c, p, e1, c.rank) + i, v, e1);
  }
  bool ok = true;
  for (long long i = start; i < total; i += stride) out[i] = psgd_comm_reduce(c, e1, i, ok) * scale;
  psgd_comm_close_epoch(c, e1);
}

PSGD_API int psgd_allreduce_oneshot_launch(const void* comm, const float* in, float* out, long long total, float scale,
                                           int max_blocks, cudaStream_t stream) {
  if (total <= 0) return 0;
  long long blocks = (total + RED_THREADS * 2 - 1) / (RED_THREADS * 2);
  if (max_blocks <= 0) max_blocks = 296;
  if (blocks > max_blocks) blocks = max_blocks;
  psgd_allreduce_oneshot_kernel<<<(int)blocks, RED_THREADS, 0, stream>>>((const PsgdCommDev*)comm, in, out, total, scale);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
