// Consumer side of the in-kernel factor all-reduce, and stand-alone collectives built from
// the same primitives (used by the collective micro-benchmark and by tests).
#include "psgd_comm.cuh"

constexpr int RED_THREADS = 256;

// Wait until every peer published the next epoch, then out[i] = sum over ranks (in rank
// order) of slot[r][i] for i < total. Optionally writes a second copy. The last CTA closes
// the epoch. Replaces the blocking NCCL all_reduce of the reference (powersgd/powersgd.py:205-209).
__global__ void __launch_bounds__(RED_THREADS) psgd_factor_reduce_kernel(const PsgdCommDev* comm, long long total,
                                                                           float* __restrict__ out1,
                                                                           float* __restrict__ out2) {
  const PsgdCommDev c = *comm;
  const int e1 = *c.epoch + 1;
  psgd_comm_wait_all(c, e1);
  const long long stride = (long long)gridDim.x * RED_THREADS;
  for (long long i = (long long)blockIdx.x * RED_THREADS + threadIdx.x; i < total; i += stride) {
    float s = 0.f;
    for (int r = 0; r < c.world; ++r) s += __ldcg(psgd_comm_slot(c, c.rank, e1, r) + i);
    out1[i] = s;
    if (out2) out2[i] = s;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (psgd_atom_add_acqrel_gpu(c.arrive + 1, 1) == (int)gridDim.x - 1) {
      c.arrive[1] = 0;
      *c.epoch = e1;
    }
  }
}

PSGD_API int psgd_factor_reduce_launch(const void* comm, long long total, float* out1, float* out2,
                                       cudaStream_t stream) {
  if (total <= 0) return 0;
  long long blocks = (total + RED_THREADS * 4 - 1) / (RED_THREADS * 4);
  if (blocks > 128) blocks = 128;  // co-resident on any part; every CTA waits at its start
  psgd_factor_reduce_kernel<<<(int)blocks, RED_THREADS, 0, stream>>>((const PsgdCommDev*)comm, total, out1, out2);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// One-shot all-reduce (SUM) of a contiguous buffer in a single launch: push, publish, wait,
// add in rank order. The grid is capped so that all CTAs are resident at once (they wait on
// each other's ranks after pushing). `scale` multiplies the result (1/W gives the mean).
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
    for (int p = 0; p < c.world; ++p) psgd_comm_slot(c, p, e1, c.rank)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (psgd_atom_add_acqrel_gpu(c.arrive + 0, 1) == (int)gridDim.x - 1) {
      c.arrive[0] = 0;
      psgd_comm_publish(c, e1);
    }
  }
  psgd_comm_wait_all(c, e1);
  for (long long i = start; i < total; i += stride) {
    float s = 0.f;
    for (int r = 0; r < c.world; ++r) s += __ldcg(psgd_comm_slot(c, c.rank, e1, r) + i);
    out[i] = s * scale;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (psgd_atom_add_acqrel_gpu(c.arrive + 1, 1) == (int)gridDim.x - 1) {
      c.arrive[1] = 0;
      *c.epoch = e1;
    }
  }
}

PSGD_API int psgd_allreduce_oneshot_launch(const void* comm, const float* in, float* out, long long total, float scale,
                                           int max_blocks, cudaStream_t stream) {
  if (total <= 0) return 0;
  long long blocks = (total + RED_THREADS * 4 - 1) / (RED_THREADS * 4);
  if (max_blocks <= 0) max_blocks = 128;
  if (blocks > max_blocks) blocks = max_blocks;
  psgd_allreduce_oneshot_kernel<<<(int)blocks, RED_THREADS, 0, stream>>>((const PsgdCommDev*)comm, in, out, total, scale);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
