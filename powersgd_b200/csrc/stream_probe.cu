// Read-only streaming pass: the floor for any kernel that has to read a buffer once.
//
// The roofline denominators used for this library are a copy (read + write) bandwidth. A kernel
// that only READS a few hundred megabytes of cold data also pays launch, ramp-up and tail, so its
// floor is measured, not derived: this kernel sums a buffer with 16-byte streaming loads (eight
// independent loads in flight per thread) and discards the result. The compression micro-benchmark
// prints its time beside the product kernels' (`bench_compress.py --read-floor`).
#include "psgd_common.cuh"

__global__ void __launch_bounds__(256) psgd_read_pass_kernel(const float4* __restrict__ p, long long n4, float* sink) {
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * 256;
  long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  for (; i + 7 * stride < n4; i += 8 * stride) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcs(p + i + u * stride);
#pragma unroll
    for (int u = 0; u < 8; ++u) acc += v[u].x + v[u].y + v[u].z + v[u].w;
  }
  for (; i < n4; i += stride) {
    const float4 v = __ldcs(p + i);
    acc += v.x + v.y + v.z + v.w;
  }
  if (acc == 1.2345678e33f) *sink = acc;   // never true for finite data: keeps the loads alive
}

// Sums `numel` floats (16-byte aligned, numel a multiple of 4) with `ctas` CTAs of 256 threads.
PSGD_API int psgd_read_pass_launch(const float* p, long long numel, float* sink, int ctas, cudaStream_t stream) {
  if (numel <= 0 || (numel & 3) != 0 || (((uintptr_t)p) & 15u) != 0 || ctas <= 0) {
    psgd_set_error("psgd_read_pass_launch: needs a 16-byte aligned buffer of a multiple of 4 floats");
    return -1;
  }
  psgd_read_pass_kernel<<<ctas, 256, 0, stream>>>((const float4*)p, numel / 4, sink);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
