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
#include "psgd_bounds.cuh"
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
  // Multi-GPU, strip kernel only: the summed factor of the LAST half-iteration has not been
  // gathered yet. The panels of lsum[nhist-1] (poll_left != 0) or rsum[nhist-1] are then read
  // from the channel's slots (bounded polls, ranks added in order); the strips that touch column
  // 0 (left factor) or row 0 (right factor) also write the sum to sum_out1 / sum_out2, which are
  // laid out like the factor buffers. Null comm: every panel comes from memory.
  const PsgdCommDev* comm;
  int poll_left;
  float* sum_out1;
  float* sum_out2;
  float sum_scale;   // factor applied to what goes to sum_out2 (1/W keeps the MEAN factor as warm start)
  // bit 0: the residual is M - update (error against the GLOBAL mean product, as the research
  //        harness' rank-k reducer defines its memory) instead of M - (local product);
  // bit 1: the residual is written to the `param` slot of the descriptor (a separate memory
  //        tensor) and the gradient is left untouched. Only without the fused optimizer step.
  int flags;
};

// Column ownership of a lane inside a 128-column block, by access width (see lowrank_ffma.cu).
template <int VEC>
__device__ __forceinline__ int fin_lane_col(int lane, int c) {
  if (VEC == 4) return 4 * lane + c;
  if (VEC == 2) return (c < 2) ? 2 * lane + c : 64 + 2 * lane + (c - 2);
  return lane + 32 * c;
}
// Position of local column lc in a panel row, such that a lane's 4 columns are adjacent.
template <int VEC>
__device__ __forceinline__ int fin_panel_pos(int lc) {
  if (VEC == 4) return lc;
  if (VEC == 2) return ((lc & 63) >> 1) * 4 + (lc & 1) + 2 * (lc >> 6);
  return (lc & 31) * 4 + (lc >> 5);
}
// The lane's 4 elements of a row (block starts at `p`, `cols` valid): load / store.
template <int VEC>
__device__ __forceinline__ void fin_load4(const float* p, int lane, int cols, float* v) {
  if (VEC == 4) {
    if (lane * 4 < cols) *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(p + lane * 4);
  } else if (VEC == 2) {
    if (lane * 2 < cols) *reinterpret_cast<float2*>(v) = *reinterpret_cast<const float2*>(p + lane * 2);
    if (64 + lane * 2 < cols) *reinterpret_cast<float2*>(v + 2) = *reinterpret_cast<const float2*>(p + 64 + lane * 2);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (lane + 32 * c < cols) v[c] = p[lane + 32 * c];
  }
}
template <int VEC>
__device__ __forceinline__ void fin_store4(float* p, int lane, int cols, const float* v) {
  if (VEC == 4) {
    if (lane * 4 < cols) *reinterpret_cast<float4*>(p + lane * 4) = *reinterpret_cast<const float4*>(v);
  } else if (VEC == 2) {
    if (lane * 2 < cols) *reinterpret_cast<float2*>(p + lane * 2) = *reinterpret_cast<const float2*>(v);
    if (64 + lane * 2 < cols) *reinterpret_cast<float2*>(p + 64 + lane * 2) = *reinterpret_cast<const float2*>(v + 2);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (lane + 32 * c < cols) p[lane + 32 * c] = v[c];
  }
}

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
__device__ __forceinline__ void finalize_general_tile(const FinalizeArgs& a, const PsgdTile& whole, const PsgdMat& mt,
                                                      float (*sLl)[FIN_ROWS], float (*sLs)[FIN_ROWS],
                                                      float (*sRl)[FIN_COLS], float (*sRs)[FIN_COLS]) {
  for (int rc = 0; rc < whole.rows; rc += FIN_ROWS) {
  PsgdTile t = whole;
  t.row0 = whole.row0 + rc;
  t.rows = min(FIN_ROWS, whole.rows - rc);
  __syncthreads();  // the previous chunk is done with the panels
  const int r = mt.r, m = mt.m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.nhist * r;

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
      // lane-major placement so that each lane's 4 columns are adjacent
      const int pos = fin_panel_pos<VEC>(lc);
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
  const bool sgd = a.fused_sgd != 0;
  const bool mom = sgd && h.has_momentum;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int lr = warp * 4 + u;
    if (lr >= t.rows) continue;
    const long long rowoff = (long long)(t.row0 + lr) * m + t.col0;
    __align__(16) float gv[4] = {0.f, 0.f, 0.f, 0.f}, pv[4] = {0.f, 0.f, 0.f, 0.f}, mv[4] = {0.f, 0.f, 0.f, 0.f}, av[4];
    if (VEC == 4 && SAME) *reinterpret_cast<float4*>(gv) = gpre[u];
    else fin_load4<VEC>(mt.grad + rowoff, lane, t.cols, gv);
    if (sgd) fin_load4<VEC>(mt.param + rowoff, lane, t.cols, pv);
    if (mom) fin_load4<VEC>(mt.mom + rowoff, lane, t.cols, mv);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      av[c] = accA[u][c] * a.inv_world;
      gv[c] -= (a.flags & 1) ? av[c] : accE[u][c];
      if (sgd) psgd_sgd_update(av[c], pv[c], &mv[c], h);
    }
    fin_store4<VEC>(((a.flags & 2) ? mt.param : mt.grad) + rowoff, lane, t.cols, gv);
    if (sgd) {
      fin_store4<VEC>(mt.param + rowoff, lane, t.cols, pv);
      if (mom) fin_store4<VEC>(mt.mom + rowoff, lane, t.cols, mv);
    } else {
      fin_store4<VEC>(mt.out + rowoff, lane, t.cols, av);
    }
  }
  }  // row chunks
}

template <bool SAME>
__global__ void __launch_bounds__(FIN_THREADS) psgd_finalize_kernel(FinalizeArgs a) {
  __shared__ __align__(16) float sLl[FIN_KC][FIN_ROWS];
  __shared__ __align__(16) float sLs[FIN_KC][FIN_ROWS];
  __shared__ __align__(16) float sRl[FIN_KC][FIN_COLS];
  __shared__ __align__(16) float sRs[FIN_KC][FIN_COLS];
  const PsgdTile whole = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[whole.mat];
  if (whole.vec == 4) finalize_general_tile<4, SAME>(a, whole, mt, sLl, sLs, sRl, sRs);
  else if (whole.vec == 2) finalize_general_tile<2, SAME>(a, whole, mt, sLl, sLs, sRl, sRs);
  else finalize_general_tile<1, SAME>(a, whole, mt, sLl, sLs, sRl, sRs);
}

// Strip kernel (K = half-iterations x rank <= FIN_STRIP_KMAX): a CTA owns a strip of up to
// `tile_rows` rows x 128 columns. All factor panels of the strip are staged in shared memory
// once; the loop over 32-row chunks then runs without barriers, every chunk issuing its global
// loads (gradient, parameter, momentum) before its FMA loop so that their latency overlaps it.
constexpr int FIN_STRIP_KMAX = 32;

// Gather `n` consecutive words starting at slot index `base` of this epoch (sum over ranks in
// rank order) and hand each to `put(i, value)`.
template <class Put>
__device__ __forceinline__ void fin_gather(const PsgdCommDev& c, int e1, long long base, int n, bool& ok, Put put) {
  constexpr int NB = 4;
  for (int i0 = threadIdx.x; i0 < n; i0 += NB * FIN_THREADS) {
    int64_t idx[NB];
    float v[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) idx[j] = (i0 + j * FIN_THREADS < n) ? base + i0 + j * FIN_THREADS : -1;
    psgd_comm_reduce_batch<NB>(c, e1, idx, NB, v, ok);
#pragma unroll
    for (int j = 0; j < NB; ++j)
      if (i0 + j * FIN_THREADS < n) put(i0 + j * FIN_THREADS, v[j]);
  }
}

template <int VEC, bool SAME>
__device__ __forceinline__ void finalize_strip_tile(const FinalizeArgs& a, const PsgdTile& t, const PsgdMat& mt,
                                                    int tile_rows, float* fin_smem) {
  const int r = mt.r, m = mt.m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.nhist * r;
  float* sRl = fin_smem;                         // [K][FIN_COLS]
  float* sLl = sRl + K * FIN_COLS;               // [K][tile_rows]
  float* sRs = SAME ? sRl : sLl + K * tile_rows;
  float* sLs = SAME ? sLl : sRs + K * FIN_COLS;

#ifdef PSGD_BOUNDS_CHECK
  {
    bool ok = true;
    ok &= PSGD_BC(t.row0 >= 0 && t.rows > 0 && t.row0 + t.rows <= mt.n && t.rows <= tile_rows, 3, PSGD_BC_TILE_ROWS, t.row0 + t.rows, mt.n);
    ok &= PSGD_BC(t.col0 >= 0 && t.cols > 0 && t.col0 + t.cols <= mt.m && t.cols <= FIN_COLS, 3, PSGD_BC_TILE_COLS, t.col0 + t.cols, mt.m);
    ok &= PSGD_BC(K >= 1 && K <= FIN_STRIP_KMAX && (SAME ? 1 : 2) * K * (FIN_COLS + tile_rows) * 4 <= 96 * 1024, 3, PSGD_BC_SMEM, K, FIN_STRIP_KMAX);
    const unsigned long long addr = (unsigned long long)mt.grad | (unsigned long long)mt.param | (unsigned long long)mt.mom | (unsigned long long)mt.out;
    ok &= PSGD_BC(t.vec == 1 || (t.vec == 2 && addr % 8 == 0 && mt.m % 2 == 0) || (t.vec == 4 && addr % 16 == 0 && mt.m % 4 == 0),
                  3, PSGD_BC_ALIGNMENT, addr % 16, t.vec);
    ok &= PSGD_BC(!a.fused_sgd || mt.param != nullptr, 3, PSGD_BC_ELEMENT, 0, 0);
    if (!ok) return;
  }
#endif
  const bool gather = !SAME && a.comm != nullptr;
  int e1 = 0;
  bool ok = true;
  if (gather) e1 = *a.comm->epoch + 1;
  for (int h = 0; h < a.nhist; ++h) {
    const bool last = gather && h == a.nhist - 1;
    {
      const long long base = mt.q_off + (long long)t.col0 * r;
      const float* gl = a.rloc[h] + base;
      const float* gs = a.rsum[h] + base;
      const bool poll = last && !a.poll_left;
      for (int e = tid; e < t.cols * r; e += FIN_THREADS) {
        const int lc = e / r, j = e - lc * r;
        const int pos = fin_panel_pos<VEC>(lc);
        sRl[(h * r + j) * FIN_COLS + pos] = gl[e];
        if (!SAME && !poll && gs != gl) sRs[(h * r + j) * FIN_COLS + pos] = gs[e];
      }
      if (poll) {
        const bool writer = t.row0 == 0;
        fin_gather(*a.comm, e1, base, t.cols * r, ok, [&](int e, float v) {
          const int lc = e / r, j = e - lc * r;
          sRs[(h * r + j) * FIN_COLS + fin_panel_pos<VEC>(lc)] = v;
          if (writer) {
            a.sum_out1[base + e] = v;
            if (a.sum_out2) a.sum_out2[base + e] = v * a.sum_scale;
          }
        });
      }
    }
    {
      const long long base = mt.p_off + (long long)t.row0 * r;
      const float* gl = a.lloc[h] + base;
      const float* gs = a.lsum[h] + base;
      const bool poll = last && a.poll_left;
      for (int e = tid; e < t.rows * r; e += FIN_THREADS) {
        const int lr = e / r, j = e - lr * r;
        sLl[(h * r + j) * tile_rows + lr] = gl[e];
        if (!SAME && !poll && gs != gl) sLs[(h * r + j) * tile_rows + lr] = gs[e];
      }
      if (poll) {
        const bool writer = t.col0 == 0;
        fin_gather(*a.comm, e1, base, t.rows * r, ok, [&](int e, float v) {
          const int lr = e / r, j = e - lr * r;
          sLs[(h * r + j) * tile_rows + lr] = v;
          if (writer) {
            a.sum_out1[base + e] = v;
            if (a.sum_out2) a.sum_out2[base + e] = v * a.sum_scale;
          }
        });
      }
    }
  }
  if (gather) psgd_comm_close_epoch(*a.comm, e1);  // (CTA barrier inside) this strip has read its words
  __syncthreads();
  const PsgdHyper hy = a.hyper[mt.hyper];
  const bool sgd = a.fused_sgd != 0;
  const bool mom = sgd && hy.has_momentum;
  const bool global_res = (a.flags & 1) != 0;
  float* const res_base = (a.flags & 2) ? mt.param : mt.grad;

  for (int rc = 0; rc < t.rows; rc += FIN_ROWS) {
    // ---- global loads of this chunk first ----
    __align__(16) float g4[4][4], p4[4][4], m4[4][4];
    bool live[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int lr = rc + warp * 4 + u;
      const long long rowoff = (long long)(t.row0 + lr) * m + t.col0;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) g4[u][c4] = p4[u][c4] = m4[u][c4] = 0.f;
      live[u] = lr < t.rows;
      if (live[u]) {
        fin_load4<VEC>(mt.grad + rowoff, lane, t.cols, g4[u]);
        if (sgd) fin_load4<VEC>(mt.param + rowoff, lane, t.cols, p4[u]);
        if (mom) fin_load4<VEC>(mt.mom + rowoff, lane, t.cols, m4[u]);
      }
    }
    // ---- rank-K update from the staged panels ----
    float accE[4][4], accA[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) accE[u][c4] = accA[u][c4] = 0.f;
    for (int h = 0; h < a.nhist; ++h) {
      // the basis side of a half-iteration is the same array for the local and the summed product:
      // its panel was staged once and is read once
      const bool one_left = SAME || a.lloc[h] == a.lsum[h];
      const bool one_right = SAME || a.rloc[h] == a.rsum[h];
#pragma unroll 4
      for (int j = 0; j < r; ++j) {
        const int k = h * r + j;
        const float4 ll = *reinterpret_cast<const float4*>(sLl + k * tile_rows + rc + warp * 4);
        const float4 rl = *reinterpret_cast<const float4*>(sRl + k * FIN_COLS + lane * 4);
        const float4 ls = one_left ? ll : *reinterpret_cast<const float4*>(sLs + k * tile_rows + rc + warp * 4);
        const float4 rs = one_right ? rl : *reinterpret_cast<const float4*>(sRs + k * FIN_COLS + lane * 4);
        const float lv[4] = {ll.x, ll.y, ll.z, ll.w}, sv[4] = {ls.x, ls.y, ls.z, ls.w};
        const float rlv[4] = {rl.x, rl.y, rl.z, rl.w}, rsv[4] = {rs.x, rs.y, rs.z, rs.w};
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            accE[u][c4] = fmaf(lv[u], rlv[c4], accE[u][c4]);
            if (!SAME) accA[u][c4] = fmaf(sv[u], rsv[c4], accA[u][c4]);
          }
      }
    }
    // ---- residual, mean update, optimizer ----
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!live[u]) continue;
      const int lr = rc + warp * 4 + u;
      const long long rowoff = (long long)(t.row0 + lr) * m + t.col0;
      __align__(16) float av[4];
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        av[c4] = (SAME ? accE[u][c4] : accA[u][c4]) * a.inv_world;
        g4[u][c4] -= global_res ? av[c4] : accE[u][c4];
        if (sgd) psgd_sgd_update(av[c4], p4[u][c4], &m4[u][c4], hy);
      }
      fin_store4<VEC>(res_base + rowoff, lane, t.cols, g4[u]);
      if (sgd) {
        fin_store4<VEC>(mt.param + rowoff, lane, t.cols, p4[u]);
        if (mom) fin_store4<VEC>(mt.mom + rowoff, lane, t.cols, m4[u]);
      } else {
        fin_store4<VEC>(mt.out + rowoff, lane, t.cols, av);
      }
    }
  }
}

template <bool SAME>
__global__ void __launch_bounds__(FIN_THREADS, 2) psgd_finalize_strip_kernel(FinalizeArgs a, int tile_rows) {
  extern __shared__ __align__(16) float fin_smem[];
  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  if (t.vec == 4) finalize_strip_tile<4, SAME>(a, t, mt, tile_rows, fin_smem);
  else if (t.vec == 2) finalize_strip_tile<2, SAME>(a, t, mt, tile_rows, fin_smem);
  else finalize_strip_tile<1, SAME>(a, t, mt, tile_rows, fin_smem);
}

// Shared-memory budgets of a strip CTA: the default carve-out serves the small ranks (several CTAs
// stay resident per SM); when the panels of a 256-row strip do not fit it (K = 32, or K >= 16 with
// separate local and summed factors), the kernel opts in to a budget that still leaves two CTAs
// per SM. Taller strips matter there: every strip re-stages 128 + rows panel entries per K.
constexpr int FIN_SMEM_DEFAULT = 48 * 1024;
constexpr int FIN_SMEM_OPT_IN = 96 * 1024;

template <bool SAME>
static int finalize_strip_launch(const FinalizeArgs& a, int ntiles, int tile_rows, int kmax, cudaStream_t stream) {
  const size_t smem = (size_t)(SAME ? 1 : 2) * kmax * (FIN_COLS + tile_rows) * sizeof(float);
  if (smem > (size_t)FIN_SMEM_DEFAULT) {
    static bool opted_in = false;   // per instantiation
    if (!opted_in) {
      PSGD_CUDA_OK(cudaFuncSetAttribute(psgd_finalize_strip_kernel<SAME>, cudaFuncAttributeMaxDynamicSharedMemorySize, FIN_SMEM_OPT_IN));
      opted_in = true;
    }
  }
  psgd_finalize_strip_kernel<SAME><<<ntiles, FIN_THREADS, smem, stream>>>(a, tile_rows);
  return 0;
}

// Tallest strip (multiple of 32 rows, at most 256) whose panels fit the shared-memory budget.
PSGD_API int psgd_finalize_strip_rows(int kmax, int same) {
  if (kmax > FIN_STRIP_KMAX) return FIN_ROWS;  // general kernel: strips only save tile overhead
  const int per_row = (same ? 1 : 2) * kmax * (int)sizeof(float);
  int rows = FIN_SMEM_DEFAULT / per_row - FIN_COLS;
  if (rows < 256) rows = FIN_SMEM_OPT_IN / per_row - FIN_COLS;
  rows = rows / FIN_ROWS * FIN_ROWS;
  return rows > 256 ? 256 : (rows < FIN_ROWS ? FIN_ROWS : rows);
}

static bool finalize_takes_strip(int nhist, int max_r, int tile_rows, bool same) {
  const int kmax = nhist * max_r;
  const size_t strip_smem = (size_t)(same ? 1 : 2) * kmax * (FIN_COLS + tile_rows) * sizeof(float);
  return kmax <= FIN_STRIP_KMAX && strip_smem <= (size_t)FIN_SMEM_OPT_IN;
}

// Whether psgd_finalize_launch runs the strip kernel for this configuration; only the strip kernel
// can gather the last factor from the channel itself.
PSGD_API int psgd_finalize_uses_strip(int nhist, int max_r, int tile_rows, int same) {
  return finalize_takes_strip(nhist, max_r, tile_rows, same != 0) ? 1 : 0;
}

// tile_rows: height of the tallest tile in `tiles` (a multiple of 32); max_r: largest rank of a
// matrix in `mats`. With nhist * max_r <= 32 and panels that fit shared memory the strip kernel
// runs, else the general one. Every tile carries its matrix's access width (`vec`).
// comm / poll_left / sum_out1 / sum_out2 / flags / sum_scale: see FinalizeArgs (comm null: nothing
// is gathered; flags 0 and sum_scale 1 for the library's own step).
PSGD_API int psgd_finalize_launch(const void* mats, const void* tiles, int ntiles, int tile_rows, int max_r,
                                  const void* hyper, int nhist, const float* const* lloc, const float* const* rloc,
                                  const float* const* lsum, const float* const* rsum, float inv_world,
                                  int fused_sgd, const void* comm, int poll_left, float* sum_out1, float* sum_out2,
                                  int flags, float sum_scale, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  if (tile_rows <= 0 || tile_rows % FIN_ROWS != 0 || max_r <= 0) {
    psgd_set_error("psgd_finalize_launch: tile_rows=%d must be a positive multiple of %d, max_r=%d positive", tile_rows, FIN_ROWS, max_r);
    return -1;
  }
  if (nhist > PSGD_MAX_HIST || nhist < 1) {
    psgd_set_error("psgd_finalize_launch: %d half-iterations outside 1..%d", nhist, PSGD_MAX_HIST);
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
  a.comm = (const PsgdCommDev*)comm;
  a.poll_left = poll_left;
  a.sum_out1 = sum_out1;
  a.sum_out2 = sum_out2;
  a.flags = flags;
  a.sum_scale = sum_scale;
  if (flags != 0 && fused_sgd) {
    psgd_set_error("psgd_finalize_launch: residual flags %d cannot be combined with the fused optimizer step", flags);
    return -1;
  }
  bool same = true;
  for (int i = 0; i < nhist; ++i) same = same && lloc[i] == lsum[i] && rloc[i] == rsum[i];
  const bool strip = finalize_takes_strip(nhist, max_r, tile_rows, same);
  if (comm != nullptr && (!strip || same || sum_out1 == nullptr)) {
    psgd_set_error("psgd_finalize_launch: gathering from a channel needs the strip kernel, distinct summed factors and a destination");
    return -1;
  }
  if (strip) {
    const int kmax = nhist * max_r;
    if (same) finalize_strip_launch<true>(a, ntiles, tile_rows, kmax, stream);
    else finalize_strip_launch<false>(a, ntiles, tile_rows, kmax, stream);
  } else {
    if (same) psgd_finalize_kernel<true><<<ntiles, FIN_THREADS, 0, stream>>>(a);
    else psgd_finalize_kernel<false><<<ntiles, FIN_THREADS, 0, stream>>>(a);
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
             // 9: mixed launch, every item names its own operation (`PsgdFlat::op`): 8, or 5 - the
             //    residual fold of the compressed tensors and the pack + push of the uncompressed
             //    ones leave in one launch
             // large buffers go two-shot (mode 0, then psgd_bulk_allreduce_launch on `flat`, which
             // is the data region of the arena, then one of):
             // 12: wait for the gathered chunks this block reads, then unpack ; 13: same + SGD
  const PsgdCommDev* comm;
  long long n_pad;  // modes 12, 13: length of the arena's data region (whole chunks per rank)
  int keep;         // packing modes: leave the inputs as they are instead of zeroing them
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
#ifdef PSGD_BOUNDS_CHECK
  if (!PSGD_BC(first >= 0 && first < it.numel, 4, PSGD_BC_ELEMENT, first, it.numel)) return;
#endif
  const PsgdHyper h = a.hyper[it.hyper];
  PsgdCommDev c;
  int e1 = 0;
  const int mode = a.mode == 9 ? it.op : a.mode;
  const bool uses_comm = mode >= 5 && mode != 8;
  if (uses_comm) {
    c = *a.comm;
    e1 = *c.epoch + 1;
  }
  bool ok = true;
  if (mode >= 12)
    flat_wait_gathered(a, c, e1, it.flat_off + first, it.flat_off + min((long long)it.numel, first + (long long)FLAT_PER_BLOCK));
  for (int e = threadIdx.x; e < FLAT_PER_BLOCK; e += FLAT_THREADS) {
    const long long i = first + e;
    if (i >= it.numel) break;
    float g;
    if (mode == 8) {
      it.out[i] += it.grad[i];
      continue;
    } else if (mode == 0) {
      a.flat[it.flat_off + i] = it.grad[i] / a.divisor;
      if (!a.keep) it.grad[i] = 0.f;
      continue;
    } else if (mode == 5) {
      const float v = it.grad[i] / a.divisor;
      if (!a.keep) it.grad[i] = 0.f;
      for (int p = 0; p < c.world; ++p) psgd_comm_store(psgd_comm_slot(c, p, e1, c.rank) + it.flat_off + i, v, e1);
      continue;
    } else if (mode == 1 || mode == 2) {
      g = a.flat[it.flat_off + i];
    } else if (mode >= 12) {
      g = __ldcg(a.flat + it.flat_off + i);  // written by peers: never through L1
    } else if (mode >= 6) {
      g = psgd_comm_reduce(c, e1, it.flat_off + i, ok);
    } else {
      g = it.grad[i] / a.divisor;
      if (!a.keep) it.grad[i] = 0.f;
    }
    if (mode == 2 || mode == 4 || mode == 7 || mode == 13) {
      float p = it.param[i];
      float mo = h.has_momentum ? it.mom[i] : 0.f;
      psgd_sgd_update(g, p, &mo, h);
      it.param[i] = p;
      if (h.has_momentum) it.mom[i] = mo;
    } else {
      it.out[i] = g;
    }
  }
  if (uses_comm && mode >= 6) psgd_comm_close_epoch(c, e1);  // the last consumer CTA advances the channel
}

// Streaming variant of the modes that move whole buffers (0-4, 12, 13): four elements per access.
// The host selects it when every pointer of every item is 16-byte aligned (flat offsets always
// are: items start at multiples of four floats); the ragged end of an item goes element-wise.
template <int MODE>
__device__ __forceinline__ void flat_one(const FlatArgs& a, const PsgdFlat& it, const PsgdHyper& h, long long i) {
  float g;
  if (MODE == 8 || MODE == 9) {
    it.out[i] += it.grad[i];
    return;
  } else if (MODE == 0) {
    a.flat[it.flat_off + i] = it.grad[i] / a.divisor;
    if (!a.keep) it.grad[i] = 0.f;
    return;
  } else if (MODE == 1 || MODE == 2) {
    g = a.flat[it.flat_off + i];
  } else if (MODE >= 12) {
    g = __ldcg(a.flat + it.flat_off + i);
  } else {
    g = it.grad[i] / a.divisor;
    if (!a.keep) it.grad[i] = 0.f;
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
  if (MODE == 9 && it.op == 5) {
    // pack + push of an uncompressed tensor: element-wise tagged words (see psgd_flat_kernel)
    const PsgdCommDev& cc = *a.comm;
    const int ep = *cc.epoch + 1;
    for (int e = threadIdx.x; e < left; e += FLAT_THREADS) {
      const long long i = first + e;
      const float v = it.grad[i] / a.divisor;
      if (!a.keep) it.grad[i] = 0.f;
      for (int p = 0; p < cc.world; ++p) psgd_comm_store(psgd_comm_slot(cc, p, ep, cc.rank) + it.flat_off + i, v, ep);
    }
    return;
  }
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
    if (MODE == 8 || MODE == 9) {
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
      if (!a.keep) *grad4 = zero4;
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
// multiples of four floats; modes 5-7 (flag-in-data words) always run element-wise, and so do the
// op-5 items of a mixed launch (mode 9), whose pointers need no alignment.
// keep != 0: the packing modes (0, 3, 4, 5 and the op-5 items of mode 9) leave their inputs untouched.
PSGD_API int psgd_flat_launch(int mode, int vec, const void* items, const int* block_item, const int* block_first,
                              int nblocks, const void* hyper, float* flat, float divisor, const void* comm,
                              long long n_pad, int keep, cudaStream_t stream) {
  if (nblocks <= 0) return 0;
  if (mode >= 5 && mode != 8 && comm == nullptr) {
    psgd_set_error("psgd_flat_launch: mode %d needs a communication channel", mode);
    return -1;
  }
  if (!((mode >= 0 && mode <= 9) || mode == 12 || mode == 13)) {
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
  a.keep = keep;
  if (vec && !(mode >= 5 && mode <= 7)) {
    switch (mode) {
      case 0: flat_vec_launch<0>(a, nblocks, stream); break;
      case 1: flat_vec_launch<1>(a, nblocks, stream); break;
      case 2: flat_vec_launch<2>(a, nblocks, stream); break;
      case 3: flat_vec_launch<3>(a, nblocks, stream); break;
      case 4: flat_vec_launch<4>(a, nblocks, stream); break;
      case 8: flat_vec_launch<8>(a, nblocks, stream); break;
      case 9: flat_vec_launch<9>(a, nblocks, stream); break;
      case 12: flat_vec_launch<12>(a, nblocks, stream); break;
      default: flat_vec_launch<13>(a, nblocks, stream); break;
    }
  } else {
    psgd_flat_kernel<<<nblocks, FLAT_THREADS, 0, stream>>>(a);
  }
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

#ifdef PSGD_BOUNDS_CHECK
PSGD_BOUNDS_EXPORT(psgd_bounds_read_finalize)
#endif
