// Exact magnitude top-k selection (unsorted), fused with the error-feedback write.
//
// The sparsifying reducers of the research harness call torch.topk on |x|, gather the values,
// then copy the tensor and zero the selected entries (paper-code/gradient_reducers.py:226-253,
// 296-324). Here one radix select does all of it in four launches over x:
//   3 x histogram pass over the 31-bit magnitude key (bits 30..20, 19..9, 8..0), each pass
//       restricted to the keys that matched the digits chosen so far (every CTA re-derives the
//       chosen digit from the previous histogram, so no separate "scan" launches are needed);
//   1 x compaction: keys above the threshold key are all taken, keys equal to it fill the rest;
//       writes values[k], positions[k] (int32) and, optionally, memory = x with the taken
//       entries zeroed.
// The magnitude key of a finite float orders like |x|. The output order is unspecified (as with
// torch.topk(sorted=False)); among exact ties at the threshold any subset may be taken.
#include "psgd_common.cuh"

namespace {

constexpr int TK_THREADS = 512;
constexpr int TK_BINS0 = 2048, TK_BINS1 = 2048, TK_BINS2 = 512;

// workspace layout (ints): hist0[2048] hist1[2048] hist2[512] | cnt_gt, cnt_eq
constexpr int TK_WS_INTS = TK_BINS0 + TK_BINS1 + TK_BINS2 + 8;

struct Pick {
  unsigned prefix;   // digits chosen so far, already shifted into place
  long long remain;  // how many entries still to take inside the chosen bin
};

__device__ __forceinline__ unsigned tk_key(float v) { return __float_as_uint(v) & 0x7FFFFFFFu; }

// Scan a histogram from its top bin down until `remain` entries are covered; returns the bin and
// updates `remain` to the number to take inside it. Executed redundantly by thread 0 of each CTA.
__device__ int tk_choose(const int* hist, int bins, long long& remain) {
  for (int b = bins - 1; b >= 0; --b) {
    const int c = hist[b];
    if (remain <= c) return b;
    remain -= c;
  }
  return 0;
}

__device__ void tk_derive(const int* ws, int upto, long long k, Pick& p) {
  p.prefix = 0u;
  p.remain = k;
  if (upto >= 1) p.prefix |= (unsigned)tk_choose(ws, TK_BINS0, p.remain) << 20;
  if (upto >= 2) p.prefix |= (unsigned)tk_choose(ws + TK_BINS0, TK_BINS1, p.remain) << 9;
  if (upto >= 3) p.prefix |= (unsigned)tk_choose(ws + TK_BINS0 + TK_BINS1, TK_BINS2, p.remain);
}

// pass = 0, 1, 2
__global__ void __launch_bounds__(TK_THREADS) psgd_topk_hist_kernel(const float* __restrict__ x, long long n, long long k,
                                                                     int* __restrict__ ws, int pass) {
  __shared__ int sh[TK_BINS0];
  __shared__ Pick pick;
  const int bins = pass == 2 ? TK_BINS2 : TK_BINS0;
  for (int b = threadIdx.x; b < bins; b += TK_THREADS) sh[b] = 0;
  if (threadIdx.x == 0) tk_derive(ws, pass, k, pick);
  __syncthreads();
  const unsigned prefix = pick.prefix;
  const unsigned mask = pass == 0 ? 0u : (pass == 1 ? 0x7FF00000u : 0x7FFFFE00u);
  const int shift = pass == 0 ? 20 : (pass == 1 ? 9 : 0);
  const unsigned digit_mask = pass == 2 ? 0x1FFu : 0x7FFu;
  const long long stride = (long long)gridDim.x * TK_THREADS;
  for (long long i = (long long)blockIdx.x * TK_THREADS + threadIdx.x; i < n; i += stride) {
    const unsigned key = tk_key(__ldg(x + i));
    if ((key & mask) == prefix) atomicAdd(&sh[(key >> shift) & digit_mask], 1);
  }
  __syncthreads();
  int* hist = ws + (pass == 0 ? 0 : (pass == 1 ? TK_BINS0 : TK_BINS0 + TK_BINS1));
  for (int b = threadIdx.x; b < bins; b += TK_THREADS)
    if (sh[b]) atomicAdd(hist + b, sh[b]);
}

__global__ void __launch_bounds__(TK_THREADS) psgd_topk_compact_kernel(const float* __restrict__ x, long long n, long long k,
                                                                        int* __restrict__ ws, float* __restrict__ values,
                                                                        int* __restrict__ positions,
                                                                        float* __restrict__ memory) {
  __shared__ Pick pick;
  if (threadIdx.x == 0) tk_derive(ws, 3, k, pick);
  __syncthreads();
  const unsigned threshold = pick.prefix;
  const long long take_equal = pick.remain;       // entries with key == threshold to take
  const long long base_equal = k - take_equal;    // entries with key > threshold come first
  int* cnt_gt = ws + TK_BINS0 + TK_BINS1 + TK_BINS2;
  int* cnt_eq = cnt_gt + 1;
  const long long stride = (long long)gridDim.x * TK_THREADS;
  for (long long i = (long long)blockIdx.x * TK_THREADS + threadIdx.x; i < n; i += stride) {
    const float v = __ldg(x + i);
    const unsigned key = tk_key(v);
    long long slot = -1;
    if (key > threshold) slot = atomicAdd(cnt_gt, 1);
    else if (key == threshold) {
      const long long e = atomicAdd(cnt_eq, 1);
      if (e < take_equal) slot = base_equal + e;
    }
    if (slot >= 0) {
      values[slot] = v;
      positions[slot] = (int)i;
    }
    if (memory) memory[i] = slot >= 0 ? 0.f : v;
  }
}

}  // namespace

PSGD_API int psgd_topk_workspace_ints() { return TK_WS_INTS; }

// Top-k of |x| over n float32 entries (k <= n, n < 2^31): values[k], positions[k] (int32), and
// if `memory` is non-null, memory[i] = 0 where taken else x[i] (memory may alias x only if it IS x).
PSGD_API int psgd_topk_abs(const float* x, long long n, long long k, int* workspace, float* values, int* positions,
                           float* memory, cudaStream_t stream) {
  if (n <= 0 || k <= 0) return 0;
  if (k > n || n >= (1ll << 31)) {
    psgd_set_error("psgd_topk_abs: need 0 < k <= n < 2^31 (k = %lld, n = %lld)", k, n);
    return -1;
  }
  PSGD_CUDA_OK(cudaMemsetAsync(workspace, 0, sizeof(int) * TK_WS_INTS, stream));
  long long blocks = (n + TK_THREADS * 8 - 1) / (TK_THREADS * 8);
  if (blocks > 592) blocks = 592;
  for (int pass = 0; pass < 3; ++pass)
    psgd_topk_hist_kernel<<<(int)blocks, TK_THREADS, 0, stream>>>(x, n, k, workspace, pass);
  psgd_topk_compact_kernel<<<(int)blocks, TK_THREADS, 0, stream>>>(x, n, k, workspace, values, positions, memory);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
