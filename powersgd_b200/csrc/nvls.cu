// In-switch all-reduce of a flat float32 buffer (NVLink SHARP through `multimem`).
//
// The buffer lives in memory that every rank has bound to ONE NVLink multicast object, so a
// single address (`mc`) names the W replicas at once: `multimem.ld_reduce` has the switch read
// the same offset on every GPU and return the sum, `multimem.st` has it write a value to all of
// them. Each rank reduces the slice it owns and broadcasts the result, so a byte leaves every
// GPU 1 + 1/W times instead of the 2 (W-1)/W of the two-shot peer-store kernels in
// comm_kernels.cu - the path NCCL takes on NVSwitch machines (powersgd/powersgd.py:22-31 and
// paper-code/gradient_reducers.py:959-978 issue that NCCL all-reduce for whole models).
//
// Two cross-rank barriers bracket the reduction - one so that every rank's buffer is complete
// before anyone reads it through the switch, one so that every slice has been written back
// before anyone unpacks. The fused kernel carries both itself, as tagged tokens on an in-kernel
// channel (psgd_comm.cuh: peer stores, bounded polls of the own arena): CTA 0 announces this
// rank, every CTA waits for the W announcements, and the CTA that finishes last announces
// completion and waits for the peers' completions. The plain kernel has no wait and is bracketed
// by two token all-reduces launched by the caller. The summed value of an element is computed
// once, by its owner, and the same bits are stored on every GPU, so replicas stay identical.
#include "psgd_comm.cuh"

namespace {

constexpr int NVLS_THREADS = 512;
constexpr int NVLS_UNROLL = 4;

__device__ __forceinline__ float4 nvls_ld_reduce(const float4* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void nvls_st(float4* p, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// mc: multicast address of the buffer; this rank owns float4 elements [first, first + count).
__global__ void __launch_bounds__(NVLS_THREADS) psgd_nvls_allreduce_kernel(float4* __restrict__ mc, long long first, long long count) {
  float4* p = mc + first;
  const long long stride = (long long)gridDim.x * NVLS_THREADS;
  long long i = (long long)blockIdx.x * NVLS_THREADS + threadIdx.x;
  for (; i + (NVLS_UNROLL - 1) * stride < count; i += NVLS_UNROLL * stride) {
    float4 v[NVLS_UNROLL];
#pragma unroll
    for (int u = 0; u < NVLS_UNROLL; ++u) v[u] = nvls_ld_reduce(p + i + u * stride);
#pragma unroll
    for (int u = 0; u < NVLS_UNROLL; ++u) nvls_st(p + i + u * stride, v[u]);
  }
  for (; i < count; i += stride) nvls_st(p + i, nvls_ld_reduce(p + i));
  __threadfence_system();
}

// One launch: entry barrier, reduction of the own slice, exit barrier. Uses two epochs of `comm`
// (a channel of its own with at least one word per slot).
__global__ void __launch_bounds__(NVLS_THREADS) psgd_nvls_allreduce_fused_kernel(const PsgdCommDev* comm, float4* __restrict__ mc,
                                                                                 long long count) {
  const PsgdCommDev c = *comm;
  const int e1 = *c.epoch + 1, e2 = e1 + 1;
  __shared__ int entry_ok;
  if (threadIdx.x == 0) entry_ok = 1;
  __syncthreads();
  // entry: "my replica is complete" to every rank (the launch follows the pack in stream order)
  if (blockIdx.x == 0 && threadIdx.x < c.world) psgd_comm_store(psgd_comm_slot(c, threadIdx.x, e1, c.rank), 0.f, e1);
  if (threadIdx.x < c.world) {
    bool ok = true;
    psgd_comm_load(c, psgd_comm_slot(c, c.rank, e1, threadIdx.x), e1, ok);
    if (!ok) entry_ok = 0;
  }
  __syncthreads();
  if (entry_ok) {  // a peer that never arrived: nothing is read or written through the switch
    float4* p = mc + (long long)c.rank * count;
    const long long stride = (long long)gridDim.x * NVLS_THREADS;
    long long i = (long long)blockIdx.x * NVLS_THREADS + threadIdx.x;
    for (; i + (NVLS_UNROLL - 1) * stride < count; i += NVLS_UNROLL * stride) {
      float4 v[NVLS_UNROLL];
#pragma unroll
      for (int u = 0; u < NVLS_UNROLL; ++u) v[u] = nvls_ld_reduce(p + i + u * stride);
#pragma unroll
      for (int u = 0; u < NVLS_UNROLL; ++u) nvls_st(p + i + u * stride, v[u]);
    }
    for (; i < count; i += stride) nvls_st(p + i, nvls_ld_reduce(p + i));
  }
  __threadfence_system();  // this thread's stores have reached every replica
  __syncthreads();
  // exit: the CTA that arrives last speaks for the rank
  __shared__ int last;
  if (threadIdx.x == 0) last = psgd_atom_add_acqrel_gpu(c.arrive + 2, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  if (threadIdx.x < c.world) {
    __threadfence_system();
    psgd_comm_store(psgd_comm_slot(c, threadIdx.x, e2, c.rank), 0.f, e2);
    bool ok = true;
    psgd_comm_load(c, psgd_comm_slot(c, c.rank, e2, threadIdx.x), e2, ok);
    __threadfence_system();  // the peers' slices are in this replica before the launch ends
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    c.arrive[2] = 0;
    *c.epoch = e2;
  }
}

}  // namespace

static int nvls_blocks(long long count, int max_blocks) {
  long long blocks = (count + (long long)NVLS_THREADS * NVLS_UNROLL - 1) / ((long long)NVLS_THREADS * NVLS_UNROLL);
  if (max_blocks <= 0) max_blocks = 74;  // measured at 4 GPUs: 74-148 CTAs saturate the links, more only contend
  if (max_blocks > 148) max_blocks = 148;  // one CTA per SM at most: every CTA of the launch is resident
  if (blocks > max_blocks) blocks = max_blocks;
  return (int)blocks;
}

// Fused form: `comm` is an in-kernel channel used by nothing else; rank and world come from it.
PSGD_API int psgd_nvls_allreduce_fused_launch(const void* comm, void* mc, long long n_floats, int world, int max_blocks,
                                              cudaStream_t stream) {
  if (n_floats <= 0) return 0;
  if (comm == nullptr || mc == nullptr || ((uintptr_t)mc & 15) != 0 || world < 2 || world > PSGD_MAX_WORLD || n_floats % (4ll * world) != 0) {
    psgd_set_error("psgd_nvls_allreduce_fused_launch: need a channel, a 16-byte aligned multicast address and n_floats (%lld) a multiple of 4 x world (%d)",
                   n_floats, world);
    return -1;
  }
  const long long count = n_floats / 4 / world;
  psgd_nvls_allreduce_fused_kernel<<<nvls_blocks(count, max_blocks), NVLS_THREADS, 0, stream>>>((const PsgdCommDev*)comm, (float4*)mc, count);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// In-place SUM over ranks of n_floats floats at the multicast address `mc` (n_floats a multiple
// of 4 * world; `mc` 16-byte aligned). Rank r reduces and rewrites elements
// [r * n_floats / world, (r + 1) * n_floats / world). Every rank calls this between two
// cross-rank barriers on the same stream.
PSGD_API int psgd_nvls_allreduce_launch(void* mc, long long n_floats, int rank, int world, int max_blocks, cudaStream_t stream) {
  if (n_floats <= 0) return 0;
  if (mc == nullptr || ((uintptr_t)mc & 15) != 0 || world < 2 || rank < 0 || rank >= world || n_floats % (4ll * world) != 0) {
    psgd_set_error("psgd_nvls_allreduce_launch: need a 16-byte aligned multicast address, 0 <= rank < world and n_floats (%lld) a multiple of 4 x world (%d)",
                   n_floats, world);
    return -1;
  }
  const long long count = n_floats / 4 / world;
  psgd_nvls_allreduce_kernel<<<nvls_blocks(count, max_blocks), NVLS_THREADS, 0, stream>>>((float4*)mc, (long long)rank * count, count);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
