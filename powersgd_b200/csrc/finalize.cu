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
// General kernel (any K): panels of FIN_KC factor columns are re-staged for every 32-row chunk.
template <int VEC, bool SAME>
__global__ void __launch_bounds__(FIN_THREADS) psgd_finalize_kernel(FinalizeArgs a) {
  const PsgdTile whole = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[whole.mat];
  for (int rc = 0; rc < whole.rows; rc += FIN_ROWS) {
  PsgdTile t = whole;
  t.row0 = whole.row0 + rc;
  t.rows = min(FIN_ROWS, whole.rows - rc);
  __syncthreads();  // the previous chunk is done with the panels
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
  }  // row chunks
}

// Strip kernel (K = half-iterations x rank <= FIN_STRIP_KMAX): a CTA owns a strip of up to
// `tile_rows` rows x 128 columns. All factor panels of the strip are staged in shared memory
// once; the loop over 32-row chunks then runs without barriers, every chunk issuing its global
// loads (gradient, parameter, momentum) before its FMA loop so that their latency overlaps it.
constexpr int FIN_STRIP_KMAX = 32;

template <int VEC, bool SAME>
__global__ void __launch_bounds__(FIN_THREADS, 2) psgd_finalize_strip_kernel(FinalizeArgs a, int tile_rows) {
  extern __shared__ __align__(16) float fin_smem[];
  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  const int r = mt.r, m = mt.m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.nhist * r;
  float* sRl = fin_smem;                         // [K][FIN_COLS]
  float* sLl = sRl + K * FIN_COLS;               // [K][tile_rows]
  float* sRs = SAME ? sRl : sLl + K * tile_rows;
  float* sLs = SAME ? sLl : sRs + K * FIN_COLS;

  for (int h = 0; h < a.nhist; ++h) {
    {
      const long long base = mt.q_off + (long long)t.col0 * r;
      const float* gl = a.rloc[h] + base;
      const float* gs = a.rsum[h] + base;
      for (int e = tid; e < t.cols * r; e += FIN_THREADS) {
        const int lc = e / r, j = e - lc * r;
        // lane-major placement so that each lane's 4 columns are adjacent for the strided layout
        const int pos = (VEC == 4) ? lc : ((lc & 31) * 4 + (lc >> 5));
        sRl[(h * r + j) * FIN_COLS + pos] = gl[e];
        if (!SAME) sRs[(h * r + j) * FIN_COLS + pos] = gs[e];
      }
    }
    {
      const long long base = mt.p_off + (long long)t.row0 * r;
      const float* gl = a.lloc[h] + base;
      const float* gs = a.lsum[h] + base;
      for (int e = tid; e < t.rows * r; e += FIN_THREADS) {
        const int lr = e / r, j = e - lr * r;
        sLl[(h * r + j) * tile_rows + lr] = gl[e];
        if (!SAME) sLs[(h * r + j) * tile_rows + lr] = gs[e];
      }
    }
  }
  __syncthreads();
  const PsgdHyper hy = a.hyper[mt.hyper];
  const bool sgd = a.fused_sgd != 0;
  const bool mom = sgd && hy.has_momentum;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

  for (int rc = 0; rc < t.rows; rc += FIN_ROWS) {
    // ---- global loads of this chunk first ----
    float4 g4[4], p4[4], m4[4];
    bool live[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int lr = rc + warp * 4 + u;
      const long long rowoff = (long long)(t.row0 + lr) * m + t.col0;
      g4[u] = p4[u] = m4[u] = zero4;
      if (VEC == 4) {
        live[u] = lr < t.rows && lane * 4 < t.cols;
        if (live[u]) {
          g4[u] = *reinterpret_cast<const float4*>(mt.grad + rowoff + lane * 4);
          if (sgd) p4[u] = *reinterpret_cast<const float4*>(mt.param + rowoff + lane * 4);
          if (mom) m4[u] = *reinterpret_cast<const float4*>(mt.mom + rowoff + lane * 4);
        }
      } else {
        live[u] = lr < t.rows;
        if (live[u]) {
          float* gv = reinterpret_cast<float*>(&g4[u]);
          float* pv = reinterpret_cast<float*>(&p4[u]);
          float* mv = reinterpret_cast<float*>(&m4[u]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int lc = lane + 32 * c;
            if (lc < t.cols) {
              gv[c] = mt.grad[rowoff + lc];
              if (sgd) pv[c] = mt.param[rowoff + lc];
              if (mom) mv[c] = mt.mom[rowoff + lc];
            }
          }
        }
      }
    }
    // ---- rank-K update from the staged panels ----
    float accE[4][4], accA[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int c = 0; c < 4; ++c) accE[u][c] = accA[u][c] = 0.f;
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
      const float4 ll = *reinterpret_cast<const float4*>(sLl + k * tile_rows + rc + warp * 4);
      const float4 rl = *reinterpret_cast<const float4*>(sRl + k * FIN_COLS + lane * 4);
      const float4 ls = SAME ? ll : *reinterpret_cast<const float4*>(sLs + k * tile_rows + rc + warp * 4);
      const float4 rs = SAME ? rl : *reinterpret_cast<const float4*>(sRs + k * FIN_COLS + lane * 4);
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
    // ---- residual, mean update, optimizer ----
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!live[u]) continue;
      const int lr = rc + warp * 4 + u;
      const long long rowoff = (long long)(t.row0 + lr) * m + t.col0;
      float* gv = reinterpret_cast<float*>(&g4[u]);
      float* pv = reinterpret_cast<float*>(&p4[u]);
      float* mv = reinterpret_cast<float*>(&m4[u]);
      float av[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        gv[c] -= accE[u][c];
        av[c] = (SAME ? accE[u][c] : accA[u][c]) * a.inv_world;
        if (sgd) psgd_sgd_update(av[c], pv[c], &mv[c], hy);
      }
      if (VEC == 4) {
        *reinterpret_cast<float4*>(mt.grad + rowoff + lane * 4) = g4[u];
        if (sgd) {
          *reinterpret_cast<float4*>(mt.param + rowoff + lane * 4) = p4[u];
          if (mom) *reinterpret_cast<float4*>(mt.mom + rowoff + lane * 4) = m4[u];
        } else {
          *reinterpret_cast<float4*>(mt.out + rowoff + lane * 4) = make_float4(av[0], av[1], av[2], av[3]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int lc = lane + 32 * c;
          if (lc >= t.cols) continue;
          mt.grad[rowoff + lc] = gv[c];
          if (sgd) {
            mt.param[rowoff + lc] = pv[c];
            if (mom) mt.mom[rowoff + lc] = mv[c];
          } else {
            mt.out[rowoff + lc] = av[c];
          }
        }
      }
    }
  }
}

template <int VEC, bool SAME>
static int finalize_strip_launch(const FinalizeArgs& a, int ntiles, int tile_rows, int kmax, cudaStream_t stream) {
  const size_t smem = (size_t)(SAME ? 1 : 2) * kmax * (FIN_COLS + tile_rows) * sizeof(float);
  psgd_finalize_strip_kernel<VEC, SAME><<<ntiles, FIN_THREADS, smem, stream>>>(a, tile_rows);
  return 0;
}

// Tallest strip (multiple of 32 rows, at most 256) whose panels fit the shared-memory budget.
PSGD_API int psgd_finalize_strip_rows(int kmax, int same) {
  if (kmax > FIN_STRIP_KMAX) return FIN_ROWS;  // general kernel: strips only save tile overhead
  const int budget = 48 * 1024;                // no opt-in needed, several CTAs per SM stay resident
  int rows = budget / ((same ? 1 : 2) * kmax * (int)sizeof(float)) - FIN_COLS;
  rows = rows / FIN_ROWS * FIN_ROWS;
  return rows > 256 ? 256 : (rows < FIN_ROWS ? FIN_ROWS : rows);
}

// tile_rows: height of the tallest tile in `tiles` (a multiple of 32); max_r: largest rank of a
// matrix in `mats`. With nhist * max_r <= 32 and panels that fit shared memory the strip kernel
// runs, else the general one.
PSGD_API int psgd_finalize_launch(int vec4, const void* mats, const void* tiles, int ntiles, int tile_rows, int max_r,
                                  const void* hyper, int nhist, const float* const* lloc, const float* const* rloc,
                                  const float* const* lsum, const float* const* rsum, float inv_world,
                                  int fused_sgd, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  if (tile_rows <= 0 || tile_rows % FIN_ROWS != 0 || max_r <= 0) {
    psgd_set_error("psgd_finalize_launch: tile_rows=%d must be a positive multiple of %d, max_r=%d positive", tile_rows, FIN_ROWS, max_r);
    return -1;
  }
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
  const int kmax = nhist * max_r;
  const size_t strip_smem = (size_t)(same ? 1 : 2) * kmax * (FIN_COLS + tile_rows) * sizeof(float);
  if (kmax <= FIN_STRIP_KMAX && strip_smem <= 48 * 1024) {
    if (vec4) {
      if (same) { if (finalize_strip_launch<4, true>(a, ntiles, tile_rows, kmax, stream)) return -1; }
      else { if (finalize_strip_launch<4, false>(a, ntiles, tile_rows, kmax, stream)) return -1; }
    } else {
      if (same) { if (finalize_strip_launch<1, true>(a, ntiles, tile_rows, kmax, stream)) return -1; }
      else { if (finalize_strip_launch<1, false>(a, ntiles, tile_rows, kmax, stream)) return -1; }
    }
    PSGD_CUDA_OK(cudaGetLastError());
    return 0;
  }
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
             // 8: accumulate (out += grad; no communication, `flat` unused)
             // large buffers go two-shot (mode 0, then psgd_bulk_allreduce_launch on `flat`, which
             // is the data region of the arena, then one of):
             // 12: wait for the gathered chunks this block reads, then unpack ; 13: same + SGD
  const PsgdCommDev* comm;
  long long n_pad;  // modes 12, 13: length of the arena's data region (whole chunks per rank)
};

constexpr int FLAT_THREADS = 256;
constexpr int FLAT_PER_BLOCK = FLAT_THREADS * 8;

// Modes 12, 13: wait for the chunks of the flat index range [g0, g1) that peers gather into this
// rank's data region. Slices are whole chunks, so chunk `lin` belongs to owner lin / cps; the own
// slice was written by this rank's earlier kernel. A block spans at most two chunks.
__device__ __forceinline__ void flat_wait_gathered(const FlatArgs& a, const PsgdCommDev& c, int e1, long long g0, long long g1) {
  PsgdBulk b;
  b.comm = a.comm;
  b.n_pad = a.n_pad;
  b.cps = (int)(a.n_pad / c.world / PSGD_BULK_CHUNK);
  const int lin0 = (int)(g0 / PSGD_BULK_CHUNK), lin1 = (int)((g1 - 1) / PSGD_BULK_CHUNK);
  if ((int)threadIdx.x <= lin1 - lin0) {
    const int lin = lin0 + threadIdx.x, owner = lin / b.cps;
    if (owner != c.rank) psgd_flag_wait(c, psgd_bulk_flag(c, b, c.rank, 1, owner, lin % b.cps), e1);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(FLAT_THREADS) psgd_flat_kernel(FlatArgs a) {
  const PsgdFlat it = a.items[a.block_item[blockIdx.x]];
  const long long first = a.block_first[blockIdx.x];
  const PsgdHyper h = a.hyper[it.hyper];
  PsgdCommDev c;
  int e1 = 0;
  const bool uses_comm = a.mode >= 5 && a.mode != 8;
  if (uses_comm) {
    c = *a.comm;
    e1 = *c.epoch + 1;
  }
  bool ok = true;
  if (a.mode >= 12)
    flat_wait_gathered(a, c, e1, it.flat_off + first, it.flat_off + min((long long)it.numel, first + (long long)FLAT_PER_BLOCK));
  for (int e = threadIdx.x; e < FLAT_PER_BLOCK; e += FLAT_THREADS) {
    const long long i = first + e;
    if (i >= it.numel) break;
    float g;
    if (a.mode == 8) {
      it.out[i] += it.grad[i];
      continue;
    } else if (a.mode == 0) {
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
    } else if (a.mode >= 12) {
      g = __ldcg(a.flat + it.flat_off + i);  // written by peers: never through L1
    } else if (a.mode >= 6) {
      g = psgd_comm_reduce(c, e1, it.flat_off + i, ok);
    } else {
      g = it.grad[i] / a.divisor;
      it.grad[i] = 0.f;
    }
    if (a.mode == 2 || a.mode == 4 || a.mode == 7 || a.mode == 13) {
      float p = it.param[i];
      float mo = h.has_momentum ? it.mom[i] : 0.f;
      psgd_sgd_update(g, p, &mo, h);
      it.param[i] = p;
      if (h.has_momentum) it.mom[i] = mo;
    } else {
      it.out[i] = g;
    }
  }
  if (uses_comm && a.mode >= 6) psgd_comm_close_epoch(c, e1);  // the last consumer CTA advances the channel
}

// Streaming variant of the modes that move whole buffers (0-4, 12, 13): four elements per access.
// The host selects it when every pointer of every item is 16-byte aligned (flat offsets always
// are: items start at multiples of four floats); the ragged end of an item goes element-wise.
template <int MODE>
__device__ __forceinline__ void flat_one(const FlatArgs& a, const PsgdFlat& it, const PsgdHyper& h, long long i) {
  float g;
  if (MODE == 8) {
    it.out[i] += it.grad[i];
    return;
  } else if (MODE == 0) {
    a.flat[it.flat_off + i] = it.grad[i] / a.divisor;
    it.grad[i] = 0.f;
    return;
  } else if (MODE == 1 || MODE == 2) {
    g = a.flat[it.flat_off + i];
  } else if (MODE >= 12) {
    g = __ldcg(a.flat + it.flat_off + i);
  } else {
    g = it.grad[i] / a.divisor;
    it.grad[i] = 0.f;
  }
  if (MODE == 2 || MODE == 4 || MODE == 13) {
    float p = it.param[i];
    float mo = h.has_momentum ? it.mom[i] : 0.f;
    psgd_sgd_update(g, p, &mo, h);
    it.param[i] = p;
    if (h.has_momentum) it.mom[i] = mo;
  } else {
    it.out[i] = g;
  }
}

template <int MODE>
__global__ void __launch_bounds__(FLAT_THREADS) psgd_flat_vec_kernel(FlatArgs a) {
  const PsgdFlat it = a.items[a.block_item[blockIdx.x]];
  const long long first = a.block_first[blockIdx.x];
  const PsgdHyper h = a.hyper[it.hyper];
  const long long left = min((long long)it.numel - first, (long long)FLAT_PER_BLOCK);
  PsgdCommDev c;
  int e1 = 0;
  if (MODE >= 12) {
    c = *a.comm;
    e1 = *c.epoch + 1;
    flat_wait_gathered(a, c, e1, it.flat_off + first, it.flat_off + first + left);
  }
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int GROUPS = FLAT_PER_BLOCK / 4 / FLAT_THREADS;
#pragma unroll
  for (int k = 0; k < GROUPS; ++k) {
    const int e = (threadIdx.x + k * FLAT_THREADS) * 4;
    if (e >= left) break;
    const long long i = first + e;
    if (e + 4 > left) {
      for (int j = 0; e + j < left; ++j) flat_one<MODE>(a, it, h, i + j);
      break;
    }
    float4 g;
    float4* grad4 = (float4*)(it.grad + i);
    float4* flat4 = (float4*)(a.flat + it.flat_off + i);
    if (MODE == 8) {
      const float4 add = *grad4;
      float4* o4 = (float4*)(it.out + i);
      float4 o = *o4;
      o.x += add.x; o.y += add.y; o.z += add.z; o.w += add.w;
      *o4 = o;
      continue;
    }
    if (MODE == 0 || MODE == 3 || MODE == 4) {
      g = *grad4;
      // the scalar path divides; a multiplication by the reciprocal differs in the last bit for
      // divisors that are not powers of two, so divide here too
      g.x /= a.divisor; g.y /= a.divisor; g.z /= a.divisor; g.w /= a.divisor;
      *grad4 = zero4;
      if (MODE == 0) {
        *flat4 = g;
        continue;
      }
    } else if (MODE >= 12) {
      g = __ldcg(flat4);
    } else {
      g = *flat4;
    }
    if (MODE == 2 || MODE == 4 || MODE == 13) {
      float4* p4 = (float4*)(it.param + i);
      float4 p = *p4;
      if (h.has_momentum) {
        float4* m4 = (float4*)(it.mom + i);
        float4 mo = *m4;
        psgd_sgd_update(g.x, p.x, &mo.x, h);
        psgd_sgd_update(g.y, p.y, &mo.y, h);
        psgd_sgd_update(g.z, p.z, &mo.z, h);
        psgd_sgd_update(g.w, p.w, &mo.w, h);
        *m4 = mo;
      } else {
        float4 mo = zero4;
        psgd_sgd_update(g.x, p.x, &mo.x, h);
        psgd_sgd_update(g.y, p.y, &mo.y, h);
        psgd_sgd_update(g.z, p.z, &mo.z, h);
        psgd_sgd_update(g.w, p.w, &mo.w, h);
      }
      *p4 = p;
    } else {
      *(float4*)(it.out + i) = g;
    }
  }
  if (MODE >= 12) psgd_comm_close_epoch(c, e1);
}

PSGD_API int psgd_flat_block_elems() { return FLAT_PER_BLOCK; }

template <int MODE>
static void flat_vec_launch(const FlatArgs& a, int nblocks, cudaStream_t stream) {
  psgd_flat_vec_kernel<MODE><<<nblocks, FLAT_THREADS, 0, stream>>>(a);
}

// vec != 0 promises 16-byte aligned grad / param / mom / out pointers and flat offsets that are
// multiples of four floats; modes 5-7 (flag-in-data words) always run element-wise.
PSGD_API int psgd_flat_launch(int mode, int vec, const void* items, const int* block_item, const int* block_first,
                              int nblocks, const void* hyper, float* flat, float divisor, const void* comm,
                              long long n_pad, cudaStream_t stream) {
  if (nblocks <= 0) return 0;
  if (mode >= 5 && mode != 8 && comm == nullptr) {
    psgd_set_error("psgd_flat_launch: mode %d needs a communication channel", mode);
    return -1;
  }
  if (!((mode >= 0 && mode <= 8) || mode == 12 || mode == 13)) {
    psgd_set_error("psgd_flat_launch: unknown mode %d", mode);
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
  a.n_pad = n_pad;
  if (vec && !(mode >= 5 && mode <= 7)) {
    switch (mode) {
      case 0: flat_vec_launch<0>(a, nblocks, stream); break;
      case 1: flat_vec_launch<1>(a, nblocks, stream); break;
      case 2: flat_vec_launch<2>(a, nblocks, stream); break;
      case 3: flat_vec_launch<3>(a, nblocks, stream); break;
      case 4: flat_vec_launch<4>(a, nblocks, stream); break;
      case 8: flat_vec_launch<8>(a, nblocks, stream); break;
      case 12: flat_vec_launch<12>(a, nblocks, stream); break;
      default: flat_vec_launch<13>(a, nblocks, stream); break;
    }
  } else {
    psgd_flat_kernel<<<nblocks, FLAT_THREADS, 0, stream>>>(a);
  }
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
