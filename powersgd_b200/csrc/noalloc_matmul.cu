// Allocation-free variant of the transposed factor product (see psgd_noalloc.h).
//
// Same arithmetic and the same fixed-order reduction as psgd_gemm_nt_kernel in
// lowrank_ffma.cu, but the tile geometry is derived from blockIdx (there is no descriptor
// table to allocate) and the partial sums and arrival counters live in a file-scope device
// array instead of caller-provided scratch.
#include <mutex>

#include "psgd_common.cuh"
#include "psgd_noalloc.h"

namespace {

constexpr int NA_THREADS = 256;
constexpr int NA_WARPS = NA_THREADS / 32;
constexpr int NA_COLS = 128;
constexpr int NA_ROWS = 256;

struct __align__(256) NoAllocScratch {
  float partial[PSGD_NOALLOC_PARTIAL_FLOATS];
  int tickets[PSGD_NOALLOC_MAX_COL_BLOCKS];
};

// Lives in the library image: every device that loads the library holds it until exit.
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;

template <int RT, int VEC>
__global__ void __launch_bounds__(NA_THREADS) psgd_matmul_tn_noalloc_kernel(const float* __restrict__ M, int n, int m,
                                                                             const float* __restrict__ P, int r,
                                                                             float* __restrict__ Q,
                                                                             NoAllocScratch* __restrict__ scratch) {
  const int cb = blockIdx.x, rb = blockIdx.y, nrb = gridDim.y;
  const int col0 = cb * NA_COLS, cols = min(NA_COLS, m - col0);
  const int row0 = rb * NA_ROWS, rows = min(NA_ROWS, n - row0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  __shared__ float sP[NA_ROWS * RT];
  __shared__ float sSum[NA_COLS * RT];
  __shared__ int sLast;

  for (int e = tid; e < rows * RT; e += NA_THREADS) {
    const int row = e / RT, k = e % RT;
    sP[e] = (k < r) ? P[(long long)(row0 + row) * r + k] : 0.f;
  }
  __syncthreads();

  float acc[4][RT];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < RT; ++k) acc[c][k] = 0.f;

  int colv[4];
  bool colok[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    colv[c] = col0 + (VEC == 4 ? 4 * lane + c : lane + 32 * c);
    colok[c] = colv[c] < col0 + cols;
  }
  for (int i0 = warp; i0 < rows; i0 += NA_WARPS * 4) {
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * NA_WARPS;
      const bool rok = i < rows;
      const float* rowp = M + (long long)(row0 + (rok ? i : 0)) * m;
      if (VEC == 4) {
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rok && colok[0]) q = __ldg(reinterpret_cast<const float4*>(rowp + colv[0]));
        v[u][0] = q.x; v[u][1] = q.y; v[u][2] = q.z; v[u][3] = q.w;
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) v[u][c] = (rok && colok[c]) ? __ldg(rowp + colv[c]) : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * NA_WARPS;
      if (i < rows) {
        const float* pr = sP + i * RT;
#pragma unroll
        for (int k = 0; k < RT; ++k) {
          const float pk = pr[k];
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[c][k] = fmaf(v[u][c], pk, acc[c][k]);
        }
      }
    }
  }

  for (int w = 0; w < NA_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int lc = (VEC == 4 ? 4 * lane + c : lane + 32 * c);
#pragma unroll
        for (int k = 0; k < RT; ++k) {
          if (w == 0) sSum[lc * RT + k] = acc[c][k];
          else sSum[lc * RT + k] += acc[c][k];
        }
      }
    }
    __syncthreads();
  }

  constexpr int tile_elems = NA_COLS * RT;
  if (nrb > 1) {
    float* base = scratch->partial + (long long)cb * nrb * tile_elems;
    for (int e = tid; e < tile_elems; e += NA_THREADS) __stcg(base + (long long)rb * tile_elems + e, sSum[e]);
    __threadfence();
    __syncthreads();
    if (tid == 0) sLast = (psgd_atom_add_acqrel_gpu(scratch->tickets + cb, 1) == nrb - 1);
    __syncthreads();
    if (!sLast) return;
    __threadfence();
    for (int e = tid; e < tile_elems; e += NA_THREADS) {
      float s = 0.f;
      for (int p = 0; p < nrb; ++p) s += __ldcg(base + (long long)p * tile_elems + e);
      sSum[e] = s;
    }
    __syncthreads();
  }
  for (int e = tid; e < cols * r; e += NA_THREADS) {
    const int lc = e / r, k = e % r;
    Q[(long long)(col0 + lc) * r + k] = sSum[lc * RT + k];
  }
}

constexpr int NA_MAX_DEVICES = 64;
std::mutex g_setup_mutex;
NoAllocScratch* g_scratch_addr[NA_MAX_DEVICES] = {nullptr};

// Device address of the scratch array for the CURRENT device, looked up once per device.
// (In host code the symbol itself is only a stand-in; kernels need the looked-up address.)
int scratch_for_current_device(NoAllocScratch** out) {
  int dev = 0;
  PSGD_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NA_MAX_DEVICES) {
    psgd_set_error("psgd_matmul_tn_noalloc: device ordinal %d not supported", dev);
    return -1;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* addr = nullptr;
    PSGD_CUDA_OK(cudaGetSymbolAddress(&addr, g_noalloc_scratch));
    g_scratch_addr[dev] = static_cast<NoAllocScratch*>(addr);
  }
  *out = g_scratch_addr[dev];
  return 0;
}

template <int RT>
int launch(const float* M, int n, int m, const float* P, int r, float* Q, NoAllocScratch* scratch, dim3 grid,
           cudaStream_t stream) {
  const bool vec4 = (m % 4 == 0) && ((reinterpret_cast<uintptr_t>(M) & 15u) == 0);
  if (vec4) psgd_matmul_tn_noalloc_kernel<RT, 4><<<grid, NA_THREADS, 0, stream>>>(M, n, m, P, r, Q, scratch);
  else psgd_matmul_tn_noalloc_kernel<RT, 1><<<grid, NA_THREADS, 0, stream>>>(M, n, m, P, r, Q, scratch);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int psgd_matmul_tn_noalloc(const float* M, int n, int m,
                                                                              const float* P, int r, float* Q,
                                                                              cudaStream_t stream) {
  if (M == nullptr || P == nullptr || Q == nullptr || n <= 0 || m <= 0 || r <= 0) {
    psgd_set_error("psgd_matmul_tn_noalloc: null pointer or non-positive size (n=%d m=%d r=%d)", n, m, r);
    return -1;
  }
  if (r > PSGD_NOALLOC_MAX_RANK) {
    psgd_set_error("psgd_matmul_tn_noalloc: rank %d exceeds the built-in maximum %d", r, PSGD_NOALLOC_MAX_RANK);
    return -1;
  }
  const int rt = r <= 1 ? 1 : r <= 2 ? 2 : r <= 4 ? 4 : 8;
  const long long col_blocks = ((long long)m + NA_COLS - 1) / NA_COLS;
  const long long row_blocks = ((long long)n + NA_ROWS - 1) / NA_ROWS;
  if (col_blocks > PSGD_NOALLOC_MAX_COL_BLOCKS || row_blocks > 65535 ||
      (row_blocks > 1 && col_blocks * row_blocks * NA_COLS * rt > PSGD_NOALLOC_PARTIAL_FLOATS)) {
    psgd_set_error(
        "psgd_matmul_tn_noalloc: a %d x %d matrix at rank %d needs %lld floats of scratch in %lld column blocks; the "
        "built-in scratch holds %d floats and %d column blocks",
        n, m, r, col_blocks * row_blocks * NA_COLS * rt, col_blocks, PSGD_NOALLOC_PARTIAL_FLOATS,
        PSGD_NOALLOC_MAX_COL_BLOCKS);
    return -1;
  }
  NoAllocScratch* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // the counters must start at zero; the partial sums are fully overwritten before they are read
  PSGD_CUDA_OK(cudaMemsetAsync(scratch->tickets, 0, sizeof(int) * (size_t)col_blocks, stream));
  const dim3 grid((unsigned)col_blocks, (unsigned)row_blocks);
  switch (rt) {
    case 1: return launch<1>(M, n, m, P, r, Q, scratch, grid, stream);
    case 2: return launch<2>(M, n, m, P, r, Q, scratch, grid, stream);
    case 4: return launch<4>(M, n, m, P, r, Q, scratch, grid, stream);
    default: return launch<8>(M, n, m, P, r, Q, scratch, grid, stream);
  }
}
