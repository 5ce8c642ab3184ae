// Decompression fused with error feedback and the optimizer step.
//
// After the half-iterations of one step every compressed matrix has T factor pairs:
//     local pairs  (Lloc_t [n,r], Rloc_t [m,r])   what THIS worker removed from its gradient
//     summed pairs (Lsum_t [n,r], Rsum_t [m,r])   the same with the fresh factor summed over workers
// One pass over M then produces everything the reference spreads over `baddbmm_` (deflation),
// `baddbmm_` (approximation), two `copy_`s and `optimizer.step()`
// (powersgd/powersgd.py:195-230; powersgd/__init__.py:17-25):
//     residual  M   <- M - sum_t Lloc_t Rloc_t^T            (error feedback memory, in place)
//     update    A    = (1/W) sum_t Lsum_t Rsum_t^T          (mean low-rank gradient)
//     either    out <- A
//     or        SGD with momentum / dampening / nesterov / weight decay applied to `param`
// HBM traffic: read + write M, plus param / momentum when fused. The rank-(T*r) updates run on
// FP32 FMAs from shared-memory panels (4x4 register micro-tiles).
#include "psgd_comm.cuh"

constexpr int FIN_THREADS = 256;
constexpr int FIN_ROWS = 32;    // 8 warps x 4 rows
constexpr int FIN_COLS = 128;   // 32 lanes x 4 columns
constexpr int FIN_KC = 16;      // factor columns staged per pass

struct FinalizeArgs {
  const PsgdMat* mats;
  const PsgdTile* tiles;
  const PsgdHyper* hyper;
  int nhist;
  const float* lloc[PSGD_MAX_HIST];
  const float* rloc[PSGD_MAX_HIST];
  const float* lsum[PSGD_MAX_HIST];
  const float* rsum[PSGD_MAX_HIST];
  float inv_world;
  int fused_sgd;
};

__device__ __forceinline__ float psgd_sgd_update(float g, float& p, float* mom_ptr, const PsgdHyper& h) {
  // torch.optim.SGD semantics: weight decay folded into the gradient, then momentum.
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) g = fmaf(h.weight_decay, p, g);
  if (h.has_momentum) {
    float b = fmaf(h.momentum, *mom_ptr, h.one_minus_dampening * g);
    *mom_ptr = b;
    g = h.nesterov ? fmaf(h.momentum, b, g) : b;
  }
  p = fmaf(-h.lr, g, p);
  return p;
}

// SAME: one worker, so the summed factors ARE the local ones and the update equals what is
// removed from the gradient: one accumulator, half the shared-memory traffic and FMAs.
template <int VEC, bool SAME>
__global__ void __launch_bounds__(FIN_THREADS) psgd_finalize_kernel(FinalizeArgs a) {
  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  const int r = mt.r, m = mt.m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.nhist * r;

  __shared__ __align__(16) float sLl[FIN_KC][FIN_ROWS];
  __shared__ __align__(16) float sLs[FIN_KC][FIN_ROWS];
  __shared__ __align__(16) float sRl[FIN_KC][FIN_COLS];
  __shared__ __align__(16) float sRs[FIN_KC][FIN_COLS];

  float accE[4][4], accA[4][4];
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int c = 0; c < 4; ++c) accE[u][c] = accA[u][c] = 0.f;

  // Single-worker variant: there is register room to issue the loads of the gradient tile before
  // the rank-K update is computed, so their latency overlaps the panel staging and the FMA loop.
  float4 gpre[4];
  if (VEC == 4 && SAME) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int lr = warp * 4 + u;
      gpre[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (lr < t.rows && lane * 4 < t.cols)
        gpre[u] = *reinterpret_cast<const float4*>(mt.grad + (long long)(t.row0 + lr) * m + t.col0 + lane * 4);
    }
  }

  for (int k0 = 0; k0 < K; k0 += FIN_KC) {
    const int kc = min(FIN_KC, K - k0);
    __syncthreads();
    // stage panels: element (k, row) of L panels, (k, col) of R panels
    for (int e = tid; e < FIN_KC * FIN_ROWS; e += FIN_THREADS) {
      const int lr = e / FIN_KC, kk = e % FIN_KC;  // consecutive threads walk k: contiguous in memory
      float vl = 0.f, vs = 0.f;
      if (kk < kc && lr < t.rows) {
        const int k = k0 + kk, h = k / r, j = k % r;
        const long long off = mt.p_off + (long long)(t.row0 + lr) * r + j;
        vl = a.lloc[h][off];
        if (!SAME) vs = a.lsum[h][off];
      }
      sLl[kk][lr] = vl;
      if (!SAME) sLs[kk][lr] = vs;
    }
    for (int e = tid; e < FIN_KC * FIN_COLS; e += FIN_THREADS) {
      const int lc = e / FIN_KC, kk = e % FIN_KC;
      float vl = 0.f, vs = 0.f;
      if (kk < kc && lc < t.cols) {
        const int k = k0 + kk, h = k / r, j = k % r;
        const long long off = mt.q_off + (long long)(t.col0 + lc) * r + j;
        vl = a.rloc[h][off];
        if (!SAME) vs = a.rsum[h][off];
      }
      // lane-major placement so that each lane's 4 columns are adjacent for VEC == 4
      const int pos = (VEC == 4) ? lc : ((lc & 31) * 4 + (lc >> 5));
      sRl[kk][pos] = vl;
      if (!SAME) sRs[kk][pos] = vs;
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < kc; ++kk) {
      const float4 ll = *reinterpret_cast<const float4*>(&sLl[kk][warp * 4]);
      const float4 rl = *reinterpret_cast<const float4*>(&sRl[kk][lane * 4]);
      const float4 ls = SAME ? ll : *reinterpret_cast<const float4*>(&sLs[kk][warp * 4]);
      const float4 rs = SAME ? rl : *reinterpret_cast<const float4*>(&sRs[kk][lane * 4]);
      const float lv[4] = {ll.x, ll.y, ll.z, ll.w}, sv[4] = {ls.x, ls.y, ls.z, ls.w};
      const float rlv[4] = {rl.x, rl.y, rl.z, rl.w}, rsv[4] = {rs.x, rs.y, rs.z, rs.w};
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          accE[u][c] = fmaf(lv[u], rlv[c], accE[u][c]);
          if (!SAME) accA[u][c] = fmaf(sv[u], rsv[c], accA[u][c]);
        }
    }
  }

  if (SAME) {
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int c = 0; c < 4; ++c) accA[u][c] = accE[u][c];
  }
  const PsgdHyper h = a.hyper[mt.hyper];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int lr = warp * 4 + u;
    if (lr >= t.rows) continue;
    const long long rowoff = (long long)(t.row0 + lr) * m;
    if (VEC == 4) {
      const int col = t.col0 + lane * 4;
      if (lane * 4 >= t.cols) continue;
      const float4 g = SAME ? gpre[u] : *reinterpret_cast<const float4*>(mt.grad + rowoff + col);
      float gv[4] = {g.x, g.y, g.z, g.w};
      float av[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        gv[c] -= accE[u][c];
        av[c] = accA[u][c] * a.inv_world;
      }
      *reinterpret_cast<float4*>(mt.grad + rowoff + col) = make_float4(gv[0], gv[1], gv[2], gv[3]);
      if (a.fused_sgd) {
        float4 p = *reinterpret_cast<const float4*>(mt.param + rowoff + col);
        float pv[4] = {p.x, p.y, p.z, p.w};
        float mv[4] = {0.f, 0.f, 0.f, 0.f};
        if (h.has_momentum) {
          float4 mo = *reinterpret_cast<const float4*>(mt.mom + rowoff + col);
          mv[0] = mo.x; mv[1] = mo.y; mv[2] = mo.z; mv[3] = mo.w;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) psgd_sgd_update(av[c], pv[c], &mv[c], h);
        *reinterpret_cast<float4*>(mt.param + rowoff + col) = make_float4(pv[0], pv[1], pv[2], pv[3]);
        if (h.has_momentum)
          *reinterpret_cast<float4*>(mt.mom + rowoff + col) = make_float4(mv[0], mv[1], mv[2], mv[3]);
      } else {
        *reinterpret_cast<float4*>(mt.out + rowoff + col) = make_float4(av[0], av[1], av[2], av[3]);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int lc = lane + 32 * c;
        if (lc >= t.cols) continue;
        const long long off = rowoff + t.col0 + lc;
        const float res = mt.grad[off] - accE[u][c];
        const float av = accA[u][c] * a.inv_world;
        mt.grad[off] = res;
        if (a.fused_sgd) {
          float p = mt.param[off];
          float mo = h.has_momentum ? mt.mom[off] : 0.f;
          psgd_sgd_update(av, p, &mo, h);
          mt.param[off] = p;
          if (h.has_momentum) mt.mom[off] = mo;
        } else {
          mt.out[off] = av;
        }
      }
    }
  }
}

PSGD_API int psgd_finalize_launch(int vec4, const void* mats, const void* tiles, int ntiles, const void* hyper,
                                  int nhist, const float* const* lloc, const float* const* rloc,
                                  const float* const* lsum, const float* const* rsum, float inv_world,
                                  int fused_sgd, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  if (nhist > PSGD_MAX_HIST) {
    psgd_set_error("psgd_finalize_launch: %d half-iterations beyond the compiled maximum", nhist);
    return -1;
  }
  FinalizeArgs a;
  a.mats = (const PsgdMat*)mats;
  a.tiles = (const PsgdTile*)tiles;
  a.hyper = (const PsgdHyper*)hyper;
  a.nhist = nhist;
  for (int i = 0; i < PSGD_MAX_HIST; ++i) {
    a.lloc[i] = i < nhist ? lloc[i] : nullptr;
    a.rloc[i] = i < nhist ? rloc[i] : nullptr;
    a.lsum[i] = i < nhist ? lsum[i] : nullptr;
    a.rsum[i] = i < nhist ? rsum[i] : nullptr;
  }
  a.inv_world = inv_world;
  a.fused_sgd = fused_sgd;
  bool same = true;
  for (int i = 0; i < nhist; ++i) same = same && lloc[i] == lsum[i] && rloc[i] == rsum[i];
  if (vec4) {
    if (same) psgd_finalize_kernel<4, true><<<ntiles, FIN_THREADS, 0, stream>>>(a);
    else psgd_finalize_kernel<4, false><<<ntiles, FIN_THREADS, 0, stream>>>(a);
  } else {
    if (same) psgd_finalize_kernel<1, true><<<ntiles, FIN_THREADS, 0, stream>>>(a);
    else psgd_finalize_kernel<1, false><<<ntiles, FIN_THREADS, 0, stream>>>(a);
  }
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------
// Flat (uncompressed) tensors: multi-tensor pack / unpack fused with scaling, zeroing of the
// inputs and the optimizer step. Replaces torch.cat + div_ + zero_ + optimizer.step for the
// tensors that stay uncompressed (powersgd/powersgd.py:22-31; powersgd/utils.py:6-22, 43-49).
// ------------------------------------------------------------------------------------------
struct FlatArgs {
  const PsgdFlat* items;
  const int* block_item;     // block -> item
  const int* block_first;    // block -> first element of the item handled by the block
  const PsgdHyper* hyper;
  float* flat;
  float divisor;
  int mode;  // 0: pack (flat = grad / divisor, grad = 0)
             // 1: unpack (out = flat) ; 2: unpack + SGD on param
             // 3: local (no communication): out = grad / divisor, grad = 0 ; 4: local + SGD
             // 5: pack + push {value, epoch} words to every peer's slot (in-kernel all-reduce, part 1)
             // 6: poll the own slots, sum them in rank order -> out ; 7: same + SGD (part 2)
  const PsgdCommDev* comm;
};

constexpr int FLAT_THREADS = 256;
constexpr int FLAT_PER_BLOCK = FLAT_THREADS * 8;

__global__ void __launch_bounds__(FLAT_THREADS) psgd_flat_kernel(FlatArgs a) {
  const PsgdFlat it = a.items[a.block_item[blockIdx.x]];
  const long long first = a.block_first[blockIdx.x];
  const PsgdHyper h = a.hyper[it.hyper];
  PsgdCommDev c;
  int e1 = 0;
  if (a.mode >= 5) {
    c = *a.comm;
    e1 = *c.epoch + 1;
  }
  bool ok = true;
  for (int e = threadIdx.x; e < FLAT_PER_BLOCK; e += FLAT_THREADS) {
    const long long i = first + e;
    if (i >= it.numel) break;
    float g;
    if (a.mode == 0) {
      a.flat[it.flat_off + i] = it.grad[i] / a.divisor;
      it.grad[i] = 0.f;
      continue;
    } else if (a.mode == 5) {
      const float v = it.grad[i] / a.divisor;
      it.grad[i] = 0.f;
      for (int p = 0; p < c.world; ++p) psgd_comm_store(psgd_comm_slot(c, p, e1, c.rank) + it.flat_off + i, v, e1);
      continue;
    } else if (a.mode == 1 || a.mode == 2) {
      g = a.flat[it.flat_off + i];
    } else if (a.mode >= 6) {
      g = psgd_comm_reduce(c, e1, it.flat_off + i, ok);
    } else {
      g = it.grad[i] / a.divisor;
      it.grad[i] = 0.f;
    }
    if (a.mode == 2 || a.mode == 4 || a.mode == 7) {
      float p = it.param[i];
      float mo = h.has_momentum ? it.mom[i] : 0.f;
      psgd_sgd_update(g, p, &mo, h);
      it.param[i] = p;
      if (h.has_momentum) it.mom[i] = mo;
    } else {
      it.out[i] = g;
    }
  }
  if (a.mode >= 6) psgd_comm_close_epoch(c, e1);  // the last consumer CTA advances the channel
}

PSGD_API int psgd_flat_block_elems() { return FLAT_PER_BLOCK; }

PSGD_API int psgd_flat_launch(int mode, const void* items, const int* block_item, const int* block_first,
                              int nblocks, const void* hyper, float* flat, float divisor, const void* comm,
                              cudaStream_t stream) {
  if (nblocks <= 0) return 0;
  if (mode >= 5 && comm == nullptr) {
    psgd_set_error("psgd_flat_launch: mode %d needs a communication channel", mode);
    return -1;
  }
  FlatArgs a;
  a.items = (const PsgdFlat*)items;
  a.block_item = block_item;
  a.block_first = block_first;
  a.hyper = (const PsgdHyper*)hyper;
  a.flat = flat;
  a.divisor = divisor;
  a.mode = mode;
  a.comm = (const PsgdCommDev*)comm;
  psgd_flat_kernel<<<nblocks, FLAT_THREADS, 0, stream>>>(a);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
