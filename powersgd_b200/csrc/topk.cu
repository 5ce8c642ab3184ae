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

// ---------------------------------------------------------------------------------------------
// The same selection for MANY tensors at once. The per-tensor reducer of the harness calls the
// selection once per parameter (62 times for ResNet-18, paper-code/gradient_reducers.py:226-253),
// which is launch-bound; here the three histogram passes and the compaction are four launches for
// the whole list. Every block serves one (tensor, chunk) pair from a block table; every tensor has
// its own histograms and counters in the workspace, and the digit is chosen by the whole block
// with a parallel suffix scan instead of one thread walking the bins.
namespace {

struct TopkItem {
  const float* x;      // tensor, n entries
  float* memory;       // optional: x with the taken entries zeroed
  long long n;
  long long k;         // entries to take (1 <= k <= n)
  long long out_off;   // start of this tensor's k pairs in values / positions
};

// Block-wide: walks `bins` (<= 2048, TK_THREADS threads x 4 bins) from the top until `remain` entries are
// covered; returns the bin in *bin_out and the number to take inside it in *remain_io. `scan` is
// TK_THREADS ints of shared memory.
__device__ void tk_choose_block(const int* __restrict__ hist, int bins, long long* remain_io, int* bin_out, int* scan) {
  const int t = threadIdx.x;
  // thread t owns bins [4t, 4t + 4), counted from the TOP: bin index bins - 1 - j
  int c[4], local = 0;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int j = 4 * t + u;
    c[u] = j < bins ? hist[bins - 1 - j] : 0;
    local += c[u];
  }
  scan[t] = local;
  __syncthreads();
  // inclusive prefix sum over the TK_THREADS partials (Hillis-Steele; 9 rounds)
  for (int off = 1; off < TK_THREADS; off <<= 1) {
    const int v = t >= off ? scan[t - off] : 0;
    __syncthreads();
    scan[t] += v;
    __syncthreads();
  }
  const long long remain = *remain_io;
  const long long before = t == 0 ? 0 : scan[t - 1];   // entries in the bins above this thread's
  __syncthreads();
  if (before < remain && remain <= before + local) {    // exactly one thread
    long long left = remain - before;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (left <= c[u]) {
        *bin_out = bins - 1 - (4 * t + u);
        *remain_io = left;
        break;
      }
      left -= c[u];
    }
  }
  __syncthreads();
}

// Digits chosen so far for one tensor (block-wide; result in shared `pick`).
__device__ void tk_derive_block(const int* ws, int upto, long long k, Pick* pick, long long* remain_sh, int* bin_sh, int* scan) {
  if (threadIdx.x == 0) {
    pick->prefix = 0u;
    *remain_sh = k;
    *bin_sh = 0;
  }
  __syncthreads();
  if (upto >= 1) {
    tk_choose_block(ws, TK_BINS0, remain_sh, bin_sh, scan);
    if (threadIdx.x == 0) pick->prefix |= (unsigned)(*bin_sh) << 20;
    __syncthreads();
  }
  if (upto >= 2) {
    tk_choose_block(ws + TK_BINS0, TK_BINS1, remain_sh, bin_sh, scan);
    if (threadIdx.x == 0) pick->prefix |= (unsigned)(*bin_sh) << 9;
    __syncthreads();
  }
  if (upto >= 3) {
    tk_choose_block(ws + TK_BINS0 + TK_BINS1, TK_BINS2, remain_sh, bin_sh, scan);
    if (threadIdx.x == 0) pick->prefix |= (unsigned)(*bin_sh);
    __syncthreads();
  }
  if (threadIdx.x == 0) pick->remain = *remain_sh;
  __syncthreads();
}

__global__ void __launch_bounds__(TK_THREADS) psgd_topk_many_hist_kernel(const TopkItem* __restrict__ items, const int* __restrict__ block_item,
                                                                          const int* __restrict__ block_part, const int* __restrict__ item_parts,
                                                                          int* __restrict__ ws_all, int pass) {
  __shared__ int sh[TK_BINS0];
  __shared__ int scan[TK_THREADS];
  __shared__ Pick pick;
  __shared__ long long remain_sh;
  __shared__ int bin_sh;
  const int it = block_item[blockIdx.x];
  const TopkItem item = items[it];
  int* ws = ws_all + (long long)it * TK_WS_INTS;
  const int bins = pass == 2 ? TK_BINS2 : TK_BINS0;
  for (int b = threadIdx.x; b < bins; b += TK_THREADS) sh[b] = 0;
  tk_derive_block(ws, pass, item.k, &pick, &remain_sh, &bin_sh, scan);
  const unsigned prefix = pick.prefix;
  const unsigned mask = pass == 0 ? 0u : (pass == 1 ? 0x7FF00000u : 0x7FFFFE00u);
  const int shift = pass == 0 ? 20 : (pass == 1 ? 9 : 0);
  const unsigned digit_mask = pass == 2 ? 0x1FFu : 0x7FFu;
  const long long stride = (long long)item_parts[it] * TK_THREADS;
#pragma unroll 4
  for (long long i = (long long)block_part[blockIdx.x] * TK_THREADS + threadIdx.x; i < item.n; i += stride) {
    const unsigned key = tk_key(__ldg(item.x + i));
    if ((key & mask) == prefix) atomicAdd(&sh[(key >> shift) & digit_mask], 1);
  }
  __syncthreads();
  int* hist = ws + (pass == 0 ? 0 : (pass == 1 ? TK_BINS0 : TK_BINS0 + TK_BINS1));
  for (int b = threadIdx.x; b < bins; b += TK_THREADS)
    if (sh[b]) atomicAdd(hist + b, sh[b]);
}

__global__ void __launch_bounds__(TK_THREADS) psgd_topk_many_compact_kernel(const TopkItem* __restrict__ items, const int* __restrict__ block_item,
                                                                             const int* __restrict__ block_part, const int* __restrict__ item_parts,
                                                                             int* __restrict__ ws_all, float* __restrict__ values,
                                                                             int* __restrict__ positions) {
  __shared__ int scan[TK_THREADS];
  __shared__ Pick pick;
  __shared__ long long remain_sh;
  __shared__ int bin_sh;
  const int it = block_item[blockIdx.x];
  const TopkItem item = items[it];
  int* ws = ws_all + (long long)it * TK_WS_INTS;
  tk_derive_block(ws, 3, item.k, &pick, &remain_sh, &bin_sh, scan);
  const unsigned threshold = pick.prefix;
  const long long take_equal = pick.remain;
  const long long base_equal = item.k - take_equal;
  int* cnt_gt = ws + TK_BINS0 + TK_BINS1 + TK_BINS2;
  int* cnt_eq = cnt_gt + 1;
  float* val = values + item.out_off;
  int* pos = positions + item.out_off;
  const long long stride = (long long)item_parts[it] * TK_THREADS;
  for (long long i = (long long)block_part[blockIdx.x] * TK_THREADS + threadIdx.x; i < item.n; i += stride) {
    const float v = __ldg(item.x + i);
    const unsigned key = tk_key(v);
    long long slot = -1;
    if (key > threshold) slot = atomicAdd(cnt_gt, 1);
    else if (key == threshold) {
      const long long e = atomicAdd(cnt_eq, 1);
      if (e < take_equal) slot = base_equal + e;
    }
    if (slot >= 0) {
      val[slot] = v;
      pos[slot] = (int)i;
    }
    if (item.memory) item.memory[i] = slot >= 0 ? 0.f : v;
  }
}

}  // namespace

PSGD_API int psgd_topk_item_bytes() { return (int)sizeof(TopkItem); }

// Top-k of |x| for `nitems` tensors in four launches. items: device array of TopkItem; block_item /
// block_part: device tables of `nblocks` entries (which tensor a block serves and which of that
// tensor's `item_parts[item]` interleaved parts); workspace: nitems * psgd_topk_workspace_ints() ints.
// values / positions receive every tensor's k pairs at its `out_off`.
PSGD_API int psgd_topk_abs_many(const void* items, int nitems, const int* block_item, const int* block_part, const int* item_parts,
                                int nblocks, int* workspace, float* values, int* positions, cudaStream_t stream) {
  if (nitems <= 0 || nblocks <= 0) return 0;
  PSGD_CUDA_OK(cudaMemsetAsync(workspace, 0, sizeof(int) * (size_t)TK_WS_INTS * nitems, stream));
  const TopkItem* it = (const TopkItem*)items;
  for (int pass = 0; pass < 3; ++pass)
    psgd_topk_many_hist_kernel<<<nblocks, TK_THREADS, 0, stream>>>(it, block_item, block_part, item_parts, workspace, pass);
  psgd_topk_many_compact_kernel<<<nblocks, TK_THREADS, 0, stream>>>(it, block_item, block_part, item_parts, workspace, values, positions);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Combine step of the top-k reducers: after the all-gather every worker holds W lists of
// (value, position) pairs and adds value / W into dense, zeroed outputs
// (paper-code/gradient_reducers.py:262-271 and 333-339 do it with one index_add_ per worker).
// One cooperative launch does the zero fill and the W scatter passes. Positions are unique
// within a worker's list, so a pass is race-free with plain read-modify-writes; a grid barrier
// separates the passes, which keeps the summation order (worker 0, 1, ...) fixed and the result
// bit-identical on every replica and in every run, unlike floating-point atomics.
namespace {

constexpr int SC_THREADS = 256;
constexpr int SC_MAX_SEGMENTS = 1024;

struct SparseSeg {
  float* out;        // dense output of this segment
  long long numel;   // its length
  long long end;     // end of this segment's pairs inside a worker's list (exclusive)
};

// Barrier over all CTAs of a cooperative launch on a counter that only grows (barrier b is passed
// once it reaches b * gridDim.x). Bounded: a CTA that waits longer than ~2 s gives up (all CTAs of a
// cooperative launch are resident, so this only guards against a broken launch).
__device__ bool sc_grid_barrier(unsigned* counter, unsigned& target) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) {
    target += gridDim.x;
    __threadfence();
    atomicAdd(counter, 1u);
    const unsigned long long t0 = psgd_globaltimer_ns();
    while (*(volatile unsigned*)counter < target) {
      if (psgd_globaltimer_ns() - t0 > 2000000000ull) { ok = false; break; }
    }
    __threadfence();
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(SC_THREADS) psgd_sparse_combine_kernel(const float* __restrict__ values,
                                                                          const int* __restrict__ positions, int workers,
                                                                          long long per_worker, const SparseSeg* __restrict__ segs,
                                                                          int nsegs, float divisor, unsigned* barrier, int* status) {
  __shared__ long long ends[SC_MAX_SEGMENTS];
  for (int s = threadIdx.x; s < nsegs; s += SC_THREADS) ends[s] = segs[s].end;
  __syncthreads();
  const long long tid = (long long)blockIdx.x * SC_THREADS + threadIdx.x;
  const long long stride = (long long)gridDim.x * SC_THREADS;
  for (int s = 0; s < nsegs; ++s) {
    float* out = segs[s].out;
    const long long n = segs[s].numel;
    for (long long i = tid; i < n; i += stride) out[i] = 0.f;
  }
  // value * (1 / W) rounded, then added: what torch's division by a scalar followed by index_add_
  // computes on the GPU (no fused multiply-add), so the result matches that sequence bit for bit
  const float inv = 1.0f / divisor;
  unsigned target = 0;
  for (int w = 0; w < workers; ++w) {
    if (!sc_grid_barrier(barrier, target)) {
      if (threadIdx.x == 0) atomicExch(status, 1);
      return;
    }
    const float* val = values + (long long)w * per_worker;
    const int* pos = positions + (long long)w * per_worker;
    for (long long j = tid; j < per_worker; j += stride) {
      int lo = 0, hi = nsegs - 1;   // first segment whose end is above j
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (ends[mid] > j) hi = mid; else lo = mid + 1;
      }
      const long long p = pos[j];
      if (p >= 0 && p < segs[lo].numel) segs[lo].out[p] = __fadd_rn(segs[lo].out[p], __fmul_rn(val[j], inv));
    }
  }
}

}  // namespace

PSGD_API int psgd_sparse_combine_max_segments() { return SC_MAX_SEGMENTS; }

// values / positions: [workers][per_worker] as gathered; segs: device array of `nsegs` SparseSeg
// (segment s covers pairs [segs[s-1].end, segs[s].end) of every worker's list; positions are local
// to the segment's output); barrier: one zeroed unsigned per launch; status: set to 1 if the grid
// barrier gave up. Writes out_s = sum over workers (in rank order) of the scattered value / divisor.
PSGD_API int psgd_sparse_combine_launch(const float* values, const int* positions, int workers, long long per_worker,
                                        const void* segs, int nsegs, float divisor, unsigned* barrier, int* status,
                                        cudaStream_t stream) {
  if (nsegs <= 0 || workers <= 0) return 0;
  if (nsegs > SC_MAX_SEGMENTS) {
    psgd_set_error("psgd_sparse_combine_launch: %d segments exceed the maximum %d", nsegs, SC_MAX_SEGMENTS);
    return -1;
  }
  static int blocks_cached = 0;
  if (!blocks_cached) {
    int dev = 0, sms = 0, per_sm = 0;
    PSGD_CUDA_OK(cudaGetDevice(&dev));
    PSGD_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    PSGD_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, psgd_sparse_combine_kernel, SC_THREADS, 0));
    blocks_cached = sms * (per_sm > 4 ? 4 : (per_sm < 1 ? 1 : per_sm));
  }
  PSGD_CUDA_OK(cudaMemsetAsync(barrier, 0, sizeof(unsigned), stream));
  const SparseSeg* segs_t = (const SparseSeg*)segs;
  void* params[] = {(void*)&values, (void*)&positions, (void*)&workers, (void*)&per_worker, (void*)&segs_t,
                    (void*)&nsegs, (void*)&divisor, (void*)&barrier, (void*)&status};
  PSGD_CUDA_OK(cudaLaunchCooperativeKernel((const void*)psgd_sparse_combine_kernel, dim3(blocks_cached), dim3(SC_THREADS), params, 0, stream));
  return 0;
}
