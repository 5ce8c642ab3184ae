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

// All-gather of `n` 32-bit words per rank in a single launch: every thread pushes its words (tagged)
// into slot[rank] of every peer, then polls the W slots of the own arena and writes them out rank
// after rank. Replaces the library all_gather of the sign, top-k and SVD reducers
// (paper-code/gradient_reducers.py:69-70, 133, 180, 259-260, 330-331, 631-633). Words are moved as
// bit patterns, so any 4-byte element type (packed sign words, int32 positions, float values) works.
__global__ void __launch_bounds__(RED_THREADS) psgd_allgather_oneshot_kernel(const PsgdCommDev* comm,
                                                                               const uint32_t* __restrict__ in,
                                                                               uint32_t* __restrict__ out, long long n) {
  const PsgdCommDev c = *comm;
  const int e1 = *c.epoch + 1;
  const long long stride = (long long)gridDim.x * RED_THREADS;
  const long long start = (long long)blockIdx.x * RED_THREADS + threadIdx.x;
  for (long long i = start; i < n; i += stride) {
    const float v = __uint_as_float(in[i]);
    for (int p = 0; p < c.world; ++p) psgd_comm_store(psgd_comm_slot(c, p, e1, c.rank) + i, v, e1);
  }
  bool ok = true;
  for (long long i = start; i < n; i += stride)
    for (int r = 0; r < c.world; ++r)
      out[(long long)r * n + i] = __float_as_uint(psgd_comm_load(c, psgd_comm_slot(c, c.rank, e1, r) + i, e1, ok));
  psgd_comm_close_epoch(c, e1);
}

PSGD_API int psgd_allgather_oneshot_launch(const void* comm, const void* in, void* out, long long n, int max_blocks,
                                           cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + RED_THREADS * 2 - 1) / (RED_THREADS * 2);
  if (max_blocks <= 0) max_blocks = 296;
  if (blocks > max_blocks) blocks = max_blocks;
  psgd_allgather_oneshot_kernel<<<(int)blocks, RED_THREADS, 0, stream>>>((const PsgdCommDev*)comm, (const uint32_t*)in,
                                                                        (uint32_t*)out, n);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---- bulk two-shot all-reduce of the flat data region of the arena --------------------------
// Step 1 (this kernel): push every chunk of the slices that other ranks own into the owner's
// landing area, then publish the chunk's flag there. Nothing is loaded across the link.
constexpr int BULK_THREADS = 256;
constexpr int BULK_VEC = PSGD_BULK_CHUNK / 4 / BULK_THREADS;  // float4 per thread per chunk
static_assert(BULK_VEC * 4 * BULK_THREADS == PSGD_BULK_CHUNK, "chunk must be whole float4 per thread");

__global__ void __launch_bounds__(BULK_THREADS) psgd_bulk_scatter_kernel(PsgdBulk b) {
  const PsgdCommDev c = *b.comm;
  const int e1 = *c.epoch + 1;
  const int q = blockIdx.x % b.cps;
  const int owner = (c.rank + 1 + blockIdx.x / b.cps) % c.world;  // every rank starts at another peer
  const long long slice = (long long)b.cps * PSGD_BULK_CHUNK;
  const float4* src = (const float4*)(psgd_bulk_data(c, c.rank) + owner * slice + (long long)q * PSGD_BULK_CHUNK);
  float4* dst = (float4*)(psgd_bulk_stage(c, b, owner) + c.rank * slice + (long long)q * PSGD_BULK_CHUNK);
  float4 v[BULK_VEC];
#pragma unroll
  for (int k = 0; k < BULK_VEC; ++k) v[k] = src[threadIdx.x + k * BULK_THREADS];
#pragma unroll
  for (int k = 0; k < BULK_VEC; ++k) dst[threadIdx.x + k * BULK_THREADS] = v[k];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    psgd_flag_publish(psgd_bulk_flag(c, b, owner, 0, c.rank, q), e1);
  }
}

// Step 2: the owner of a slice waits for the W-1 pushes of a chunk, adds the W contributions in
// rank order (its own straight from the data region), writes the sum into everybody's data region
// and publishes the chunk there. Step 3 is the consumer (the unpack kernels), which waits for the
// chunks it reads and closes the epoch.
__global__ void __launch_bounds__(BULK_THREADS) psgd_bulk_reduce_kernel(PsgdBulk b) {
  const PsgdCommDev c = *b.comm;
  const int e1 = *c.epoch + 1;
  const long long slice = (long long)b.cps * PSGD_BULK_CHUNK;
  for (int q = blockIdx.x; q < b.cps; q += gridDim.x) {
    if (threadIdx.x < c.world && threadIdx.x != c.rank) psgd_flag_wait(c, psgd_bulk_flag(c, b, c.rank, 0, threadIdx.x, q), e1);
    __syncthreads();
    const long long off = c.rank * slice + (long long)q * PSGD_BULK_CHUNK;
    float4 acc[BULK_VEC];
#pragma unroll
    for (int k = 0; k < BULK_VEC; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < c.world; ++r) {
      const float4* src = r == c.rank ? (const float4*)(psgd_bulk_data(c, c.rank) + off)
                                      : (const float4*)(psgd_bulk_stage(c, b, c.rank) + r * slice + (long long)q * PSGD_BULK_CHUNK);
#pragma unroll
      for (int k = 0; k < BULK_VEC; ++k) {
        const float4 v = __ldcg(src + threadIdx.x + k * BULK_THREADS);
        acc[k].x += v.x; acc[k].y += v.y; acc[k].z += v.z; acc[k].w += v.w;
      }
    }
    for (int p = 0; p < c.world; ++p) {
      float4* dst = (float4*)(psgd_bulk_data(c, (c.rank + p) % c.world) + off);
#pragma unroll
      for (int k = 0; k < BULK_VEC; ++k) dst[threadIdx.x + k * BULK_THREADS] = acc[k];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int p = 1; p < c.world; ++p) psgd_flag_publish(psgd_bulk_flag(c, b, (c.rank + p) % c.world, 1, c.rank, q), e1);
    }
  }
}

PSGD_API long long psgd_bulk_chunk_floats() { return PSGD_BULK_CHUNK; }

// Arena bytes that a bulk all-reduce of n_pad floats needs on every rank.
PSGD_API long long psgd_bulk_arena_bytes(long long n_pad, int world) {
  const long long cps = n_pad / world / PSGD_BULK_CHUNK;
  return 8 * n_pad + 2LL * world * cps * (long long)sizeof(int32_t);
}

static int bulk_args(PsgdBulk* b, const void* comm, long long n_pad, int world) {
  if (world < 2 || world > PSGD_MAX_WORLD || n_pad <= 0 || n_pad % ((long long)world * PSGD_BULK_CHUNK) != 0) {
    psgd_set_error("bulk all-reduce: n_pad=%lld must be a positive multiple of world (%d) x %d", n_pad, world, PSGD_BULK_CHUNK);
    return -1;
  }
  b->comm = (const PsgdCommDev*)comm;
  b->n_pad = n_pad;
  b->cps = (int)(n_pad / world / PSGD_BULK_CHUNK);
  return 0;
}

// Steps 1 and 2 on `stream`; the caller then launches a consumer (psgd_flat_launch modes 12/13, or
// psgd_bulk_finish_launch) that waits for the gathered chunks and closes the epoch.
PSGD_API int psgd_bulk_allreduce_launch(const void* comm, long long n_pad, int world, cudaStream_t stream) {
  PsgdBulk b;
  if (bulk_args(&b, comm, n_pad, world) != 0) return -1;
  psgd_bulk_scatter_kernel<<<(world - 1) * b.cps, BULK_THREADS, 0, stream>>>(b);
  PSGD_CUDA_OK(cudaGetLastError());
  int blocks = b.cps < 148 * 8 ? b.cps : 148 * 8;
  psgd_bulk_reduce_kernel<<<blocks, BULK_THREADS, 0, stream>>>(b);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// Stand-alone consumer: waits for every gathered chunk and closes the epoch (the data is then
// complete in the arena's data region). Used when no unpack kernel follows.
__global__ void __launch_bounds__(BULK_THREADS) psgd_bulk_finish_kernel(PsgdBulk b) {
  const PsgdCommDev c = *b.comm;
  const int e1 = *c.epoch + 1;
  const int total = c.world * b.cps;
  for (int i = blockIdx.x * BULK_THREADS + threadIdx.x; i < total; i += gridDim.x * BULK_THREADS) {
    const int src = i / b.cps;
    if (src != c.rank) psgd_flag_wait(c, psgd_bulk_flag(c, b, c.rank, 1, src, i % b.cps), e1);
  }
  psgd_comm_close_epoch(c, e1);
}

PSGD_API int psgd_bulk_finish_launch(const void* comm, long long n_pad, int world, cudaStream_t stream) {
  PsgdBulk b;
  if (bulk_args(&b, comm, n_pad, world) != 0) return -1;
  int blocks = (world * b.cps + BULK_THREADS - 1) / BULK_THREADS;
  if (blocks > 148) blocks = 148;
  psgd_bulk_finish_kernel<<<blocks, BULK_THREADS, 0, stream>>>(b);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

