// Grouped tall-skinny products on the CUDA cores (exact float32 FMA path).
//
//   NT:  Q[m, r] = M^T[m, n] * Phat[n, r]  -  sum_i R_i[m, r] * C_i[r, r]
//   NN:  P[n, r] = M  [n, m] * Qhat[m, r]  -  sum_i L_i[n, r] * C_i[r, r]
//
// One launch covers EVERY compressed matrix of EVERY shape group: the grid walks a tile list
// built once by the host planner. This replaces the reference's per-group `torch.bmm` and the
// first `baddbmm_` (powersgd/powersgd.py:185-202): the deflation M <- M - P Q^T is never
// materialised between half-iterations; the small terms C_i (from the orthonormalisation
// launch) correct the product instead.
//
// At rank r the product does 2r flops per 4 bytes of M, so for r <= 8 float32 FMAs keep up
// with HBM and this path is bandwidth-bound; it is also the path for matrices whose row
// pitch is not a multiple of 16 bytes (27, 650 floats), which TMA cannot address. Every tile
// names the widest global access its matrix allows (16, 8 or 4 bytes: `PsgdTile::vec`), so one
// launch serves all of them.
//
// Tiles that cover the same output rows (NT: row blocks of one column block; NN: column
// blocks of one row block) write partial sums to a scratch arena; the tile that arrives last
// (arrival counter) adds them in a fixed order, so the result does not depend on scheduling.
#include "psgd_bounds.cuh"
#include "psgd_comm.cuh"

constexpr int GEMM_THREADS = 256;
constexpr int GEMM_WARPS = GEMM_THREADS / 32;
constexpr int NT_TILE_COLS = 128;   // columns of M per NT tile
constexpr int NT_MAX_ROWS = 256;    // rows of P-hat staged in smem at a time (128 at RT = 32); a tile may span several such chunks
constexpr int NN_CHUNK_COLS = 128;  // columns consumed per inner iteration of an NN tile

struct GemmArgs {
  const PsgdMat* mats;
  const PsgdTile* tiles;
  const float* in;    // orthonormal factor: P-shaped for NT, Q-shaped for NN
  float* out;         // fresh local factor: Q-shaped for NT, P-shaped for NN
  float* out2;        // optional second copy of it (single worker: the warm-start buffer) or null
  int ncorr;
  const float* corr_fac[PSGD_MAX_HIST];  // earlier local factors on the OUTPUT side
  const float* corr_c[PSGD_MAX_HIST];    // [mat][r*r] cross products
  float* partial;     // scratch for split tiles
  int* tickets;       // arrival counters (all zero between launches)
  // Multi-GPU: the epilogue also pushes every finished factor element, tagged with the next
  // epoch, into slot[rank] of every peer's arena. Null for a single worker.
  const PsgdCommDev* comm;
};

#ifdef PSGD_BOUNDS_CHECK
// Capacities of the buffers behind the raw pointers (floats / counters), set by the host through
// psgd_debug_limits_products() before a checked run; 0 = unknown, not checked.
static __device__ long long g_lim_partial, g_lim_tickets, g_lim_p, g_lim_q;

// Validates one product tile against its matrix, the template rank, the access width it claims and
// the scratch capacities. All threads compute the same verdict; a CTA with a bad tile returns
// before it touches memory.
template <int RT>
__device__ __forceinline__ bool product_tile_ok(const PsgdTile& t, const PsgdMat& mt, int kernel_id, int max_rows,
                                                int max_cols, int tile_elems) {
  bool ok = true;
  ok &= PSGD_BC(t.row0 >= 0 && t.rows > 0 && t.row0 + t.rows <= mt.n && t.rows <= max_rows, kernel_id, PSGD_BC_TILE_ROWS, t.row0 + t.rows, mt.n);
  ok &= PSGD_BC(t.col0 >= 0 && t.cols > 0 && t.col0 + t.cols <= mt.m && t.cols <= max_cols, kernel_id, PSGD_BC_TILE_COLS, t.col0 + t.cols, mt.m);
  ok &= PSGD_BC(mt.r >= 1 && mt.r <= RT, kernel_id, PSGD_BC_RANK, mt.r, RT);
  const unsigned long long addr = (unsigned long long)mt.grad;
  ok &= PSGD_BC(t.vec == 1 || (t.vec == 2 && addr % 8 == 0 && mt.m % 2 == 0) || (t.vec == 4 && addr % 16 == 0 && mt.m % 4 == 0),
                kernel_id, PSGD_BC_ALIGNMENT, addr % 16, t.vec);
  ok &= PSGD_BC(t.nsplit >= 1 && t.split >= 0 && t.split < t.nsplit, kernel_id, PSGD_BC_SCRATCH_SLOT, t.split, t.nsplit);
  if (t.nsplit > 1 && g_lim_partial > 0)
    ok &= PSGD_BC((long long)(t.slot0 + t.nsplit) * tile_elems <= g_lim_partial, kernel_id, PSGD_BC_SCRATCH_SLOT,
                  (long long)(t.slot0 + t.nsplit) * tile_elems, g_lim_partial);
  if (t.nsplit > 1 && g_lim_tickets > 0) ok &= PSGD_BC(t.ticket >= 0 && t.ticket < g_lim_tickets, kernel_id, PSGD_BC_TICKET, t.ticket, g_lim_tickets);
  if (g_lim_p > 0) ok &= PSGD_BC((long long)mt.p_off + (long long)mt.n * mt.r <= g_lim_p, kernel_id, PSGD_BC_FACTOR_INDEX, (long long)mt.p_off + (long long)mt.n * mt.r, g_lim_p);
  if (g_lim_q > 0) ok &= PSGD_BC((long long)mt.q_off + (long long)mt.m * mt.r <= g_lim_q, kernel_id, PSGD_BC_FACTOR_INDEX, (long long)mt.q_off + (long long)mt.m * mt.r, g_lim_q);
  return ok;
}
#endif

template <int RT>
__host__ __device__ constexpr int nt_max_rows() { return RT <= 16 ? NT_MAX_ROWS : NT_MAX_ROWS / 2; }

// A lane owns 4 of the 128 columns of a column block; which ones depends on the access width:
// 4 adjacent (one 16-byte load), 2 + 2 adjacent (two 8-byte loads, 64 columns apart) or 4
// columns 32 apart (scalar loads). Every variant keeps a warp's accesses contiguous.
template <int VEC>
__device__ __forceinline__ int lane_col(int lane, int c) {
  if (VEC == 4) return 4 * lane + c;
  if (VEC == 2) return (c < 2) ? 2 * lane + c : 64 + 2 * lane + (c - 2);
  return lane + 32 * c;
}

// v[0..3] = the lane's four columns of the row at `rowp` (column block starting at c0, valid up
// to cend); zero where the row or the column does not exist.
template <int VEC>
__device__ __forceinline__ void load_lane_cols(const float* __restrict__ rowp, int c0, int cend, int lane, bool rok,
                                               float* v) {
  if (VEC == 4) {
    float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
    if (rok && c0 + 4 * lane < cend) q = __ldg(reinterpret_cast<const float4*>(rowp + c0 + 4 * lane));
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  } else if (VEC == 2) {
    float2 q0 = make_float2(0.f, 0.f), q1 = make_float2(0.f, 0.f);
    if (rok && c0 + 2 * lane < cend) q0 = __ldg(reinterpret_cast<const float2*>(rowp + c0 + 2 * lane));
    if (rok && c0 + 64 + 2 * lane < cend) q1 = __ldg(reinterpret_cast<const float2*>(rowp + c0 + 64 + 2 * lane));
    v[0] = q0.x; v[1] = q0.y; v[2] = q1.x; v[3] = q1.y;
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = (rok && c0 + lane + 32 * c < cend) ? __ldg(rowp + c0 + lane + 32 * c) : 0.f;
  }
}

// Sum of element `e` over the `n` partial tiles of one output block, in split order (fixed, so the
// result does not depend on which tile arrived last). Eight loads are in flight at a time: a tall
// matrix has a hundred partial tiles per block, and one dependent L2 round trip per partial would
// cost the last arriver tens of microseconds.
__device__ __forceinline__ float sum_partials(const float* first, int tile_elems, int n) {
  float s = 0.f;
  int p = 0;
  for (; p + 8 <= n; p += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldcg(first + (long long)(p + j) * tile_elems);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j];
  }
  for (; p < n; ++p) s += __ldcg(first + (long long)p * tile_elems);
  return s;
}

// ------------------------------------------------------------------------------------------
// NT: each lane owns 4 columns, each warp strides over the tile's rows.
// ------------------------------------------------------------------------------------------
template <int RT, int VEC>
__device__ __forceinline__ void gemm_nt_tile(const GemmArgs& a, const PsgdTile& t, const PsgdMat& mt, float* smem) {
  const int r = mt.r, m = mt.m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  float* sP = smem;                        // [rows][RT]
  float* sSum = smem + nt_max_rows<RT>() * RT;   // [128][RT]
  __shared__ int sLast;
#ifdef PSGD_BOUNDS_CHECK
  if (!product_tile_ok<RT>(t, mt, 1, 1 << 30, NT_TILE_COLS, NT_TILE_COLS * RT)) return;
#endif

  float acc[4][RT];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < RT; ++k) acc[c][k] = 0.f;

  const float* __restrict__ M = mt.grad;
  const int cend = t.col0 + t.cols;
  constexpr int MAXR = nt_max_rows<RT>();

  // a tall tile is walked in chunks of MAXR rows (what fits the staging buffer of P-hat); the
  // accumulators live across chunks, so a matrix with tens of thousands of rows needs tens of
  // partial tiles per column block, not hundreds
  for (int rb = 0; rb < t.rows; rb += MAXR) {
    const int rows = min(MAXR, t.rows - rb);
    if (rb) __syncthreads();  // the previous chunk's rows of P-hat are no longer read
    // stage the chunk's rows of P-hat (zero padded to RT columns)
    const float* __restrict__ pin = a.in + mt.p_off + (long long)(t.row0 + rb) * r;
    for (int e = tid; e < rows * RT; e += GEMM_THREADS) {
      const int row = e / RT, k = e % RT;
      sP[e] = (k < r) ? pin[row * r + k] : 0.f;
    }
    __syncthreads();

    for (int i0 = warp; i0 < rows; i0 += GEMM_WARPS * 4) {
      float v[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * GEMM_WARPS;
        const bool rok = i < rows;
        load_lane_cols<VEC>(M + (long long)(t.row0 + rb + (rok ? i : 0)) * m, t.col0, cend, lane, rok, v[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * GEMM_WARPS;
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
  }
  __syncthreads();

  // deterministic cross-warp sum: warps add in index order
  for (int w = 0; w < GEMM_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int lc = lane_col<VEC>(lane, c);
#pragma unroll
        for (int k = 0; k < RT; ++k) {
          if (w == 0) sSum[lc * RT + k] = acc[c][k];
          else sSum[lc * RT + k] += acc[c][k];
        }
      }
    }
    __syncthreads();
  }

  const int tile_elems = NT_TILE_COLS * RT;
  bool owner = true;  // does this CTA write the output rows?
  if (t.nsplit > 1) {
    float* mine = a.partial + (long long)(t.slot0 + t.split) * tile_elems;
    for (int e = tid; e < tile_elems; e += GEMM_THREADS) __stcg(mine + e, sSum[e]);
    __threadfence();
    __syncthreads();
    if (tid == 0) sLast = (psgd_atom_add_acqrel_gpu(a.tickets + t.ticket, 1) == t.nsplit - 1);
    __syncthreads();
    owner = sLast != 0;
    if (owner) {
      __threadfence();
      for (int e = tid; e < tile_elems; e += GEMM_THREADS) sSum[e] = sum_partials(a.partial + (long long)t.slot0 * tile_elems + e, tile_elems, t.nsplit);
      if (tid == 0) a.tickets[t.ticket] = 0;  // ready for the next launch
      __syncthreads();
    }
  }

  // epilogue: subtract the deflation terms, store Q rows locally and push them to the peers
  float* __restrict__ qout = a.out + mt.q_off;
  uint2* push[PSGD_MAX_WORLD];
  int e1 = 0;
  int npush = 0;
  if (a.comm != nullptr && owner) {
    const PsgdCommDev c = *a.comm;
    e1 = *c.epoch + 1;
    npush = c.world;
    for (int p = 0; p < PSGD_MAX_WORLD; ++p) push[p] = p < c.world ? psgd_comm_slot(c, p, e1, c.rank) + mt.q_off : nullptr;
  }
  for (int e = tid; owner && e < t.cols * r; e += GEMM_THREADS) {
    const int lc = e / r, k = e % r;
    const int col = t.col0 + lc;
    float s = sSum[lc * RT + k];
    for (int i = 0; i < a.ncorr; ++i) {
      const float* f = a.corr_fac[i] + mt.q_off + (long long)col * r;
      const float* cm = a.corr_c[i] + (long long)mt.index * PSGD_CMAT_STRIDE;
      float d = 0.f;
      for (int l = 0; l < r; ++l) d = fmaf(f[l], cm[l * r + k], d);
      s -= d;
    }
    qout[(long long)col * r + k] = s;
    if (a.out2) a.out2[mt.q_off + (long long)col * r + k] = s;
    for (int p = 0; p < npush; ++p) psgd_comm_store(push[p] + (long long)col * r + k, s, e1);
  }
}

template <int RT>
__global__ void __launch_bounds__(GEMM_THREADS) psgd_gemm_nt_kernel(GemmArgs a) {
  extern __shared__ float smem[];
  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  if (t.vec == 4) gemm_nt_tile<RT, 4>(a, t, mt, smem);
  else if (t.vec == 2) gemm_nt_tile<RT, 2>(a, t, mt, smem);
  else gemm_nt_tile<RT, 1>(a, t, mt, smem);
}

// ------------------------------------------------------------------------------------------
// NN: each warp owns RPW rows; lanes stride across the columns and shuffle-reduce at the end.
// ------------------------------------------------------------------------------------------
template <int RT, int VEC, int RPW>
__device__ __forceinline__ void gemm_nn_tile(const GemmArgs& a, const PsgdTile& t, const PsgdMat& mt, float* sSum) {
  const int r = mt.r, m = mt.m;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int TILE_ROWS = GEMM_WARPS * RPW;
  __shared__ int sLast;
#ifdef PSGD_BOUNDS_CHECK
  if (!product_tile_ok<RT>(t, mt, 2, TILE_ROWS, 1 << 30, TILE_ROWS * RT)) return;
#endif

  const float* __restrict__ M = mt.grad;
  const float* __restrict__ qin = a.in + mt.q_off;

  float acc[RPW][RT];
#pragma unroll
  for (int u = 0; u < RPW; ++u)
#pragma unroll
    for (int k = 0; k < RT; ++k) acc[u][k] = 0.f;

  const int rbase = warp * RPW;
  const float* rowp[RPW];
  bool rok[RPW];
#pragma unroll
  for (int u = 0; u < RPW; ++u) {
    rok[u] = rbase + u < t.rows;
    rowp[u] = M + (long long)(t.row0 + (rok[u] ? rbase + u : 0)) * m;
  }

  const int cend = t.col0 + t.cols;
  for (int c0 = t.col0; c0 < cend; c0 += NN_CHUNK_COLS) {
    float v[RPW][4];
#pragma unroll
    for (int u = 0; u < RPW; ++u) load_lane_cols<VEC>(rowp[u], c0, cend, lane, rok[u], v[u]);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = c0 + lane_col<VEC>(lane, c);
      if (col < cend) {
        const float* qr = qin + (long long)col * r;
#pragma unroll
        for (int k = 0; k < RT; ++k) {
          const float qk = (k < r) ? __ldg(qr + k) : 0.f;
#pragma unroll
          for (int u = 0; u < RPW; ++u) acc[u][k] = fmaf(v[u][c], qk, acc[u][k]);
        }
      }
    }
  }

#pragma unroll
  for (int u = 0; u < RPW; ++u)
#pragma unroll
    for (int k = 0; k < RT; ++k) {
      const float s = psgd_warp_sum(acc[u][k]);
      if (lane == 0) sSum[(rbase + u) * RT + k] = s;
    }
  __syncthreads();

  constexpr int tile_elems = TILE_ROWS * RT;
  bool owner = true;
  if (t.nsplit > 1) {
    float* mine = a.partial + (long long)(t.slot0 + t.split) * tile_elems;
    for (int e = tid; e < tile_elems; e += GEMM_THREADS) __stcg(mine + e, sSum[e]);
    __threadfence();
    __syncthreads();
    if (tid == 0) sLast = (psgd_atom_add_acqrel_gpu(a.tickets + t.ticket, 1) == t.nsplit - 1);
    __syncthreads();
    owner = sLast != 0;
    if (owner) {
      __threadfence();
      for (int e = tid; e < tile_elems; e += GEMM_THREADS) sSum[e] = sum_partials(a.partial + (long long)t.slot0 * tile_elems + e, tile_elems, t.nsplit);
      if (tid == 0) a.tickets[t.ticket] = 0;
      __syncthreads();
    }
  }

  float* __restrict__ pout = a.out + mt.p_off;
  uint2* push[PSGD_MAX_WORLD];
  int e1 = 0;
  int npush = 0;
  if (a.comm != nullptr && owner) {
    const PsgdCommDev c = *a.comm;
    e1 = *c.epoch + 1;
    npush = c.world;
    for (int p = 0; p < PSGD_MAX_WORLD; ++p) push[p] = p < c.world ? psgd_comm_slot(c, p, e1, c.rank) + mt.p_off : nullptr;
  }
  for (int e = tid; owner && e < t.rows * r; e += GEMM_THREADS) {
    const int lr = e / r, k = e % r;
    const int row = t.row0 + lr;
    float s = sSum[lr * RT + k];
    for (int i = 0; i < a.ncorr; ++i) {
      const float* f = a.corr_fac[i] + mt.p_off + (long long)row * r;
      const float* cm = a.corr_c[i] + (long long)mt.index * PSGD_CMAT_STRIDE;
      float d = 0.f;
      for (int l = 0; l < r; ++l) d = fmaf(f[l], cm[l * r + k], d);
      s -= d;
    }
    pout[(long long)row * r + k] = s;
    if (a.out2) a.out2[mt.p_off + (long long)row * r + k] = s;
    for (int p = 0; p < npush; ++p) psgd_comm_store(push[p] + (long long)row * r + k, s, e1);
  }
}

template <int RT, int RPW>
__global__ void __launch_bounds__(GEMM_THREADS) psgd_gemm_nn_kernel(GemmArgs a) {
  __shared__ float sSum[GEMM_WARPS * RPW * RT];
  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  if (t.vec == 4) gemm_nn_tile<RT, 4, RPW>(a, t, mt, sSum);
  else if (t.vec == 2) gemm_nn_tile<RT, 2, RPW>(a, t, mt, sSum);
  else gemm_nn_tile<RT, 1, RPW>(a, t, mt, sSum);
}

// ------------------------------------------------------------------------------------------
// Host launchers
// ------------------------------------------------------------------------------------------
static void fill_args(GemmArgs& a, const void* mats, const void* tiles, const float* in, float* out, float* out2,
                      int ncorr, const float* const* corr_fac, const float* const* corr_c, float* partial,
                      int* tickets, const void* comm) {
  a.mats = (const PsgdMat*)mats;
  a.tiles = (const PsgdTile*)tiles;
  a.in = in;
  a.out = out;
  a.out2 = out2;
  a.ncorr = ncorr;
  for (int i = 0; i < PSGD_MAX_HIST; ++i) {
    a.corr_fac[i] = i < ncorr ? corr_fac[i] : nullptr;
    a.corr_c[i] = i < ncorr ? corr_c[i] : nullptr;
  }
  a.partial = partial;
  a.tickets = tickets;
  a.comm = (const PsgdCommDev*)comm;
}

template <int RT>
static int launch_nt(const GemmArgs& a, int ntiles, cudaStream_t stream) {
  const size_t smem = (size_t)(nt_max_rows<RT>() * RT + NT_TILE_COLS * RT) * sizeof(float);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    PSGD_CUDA_OK(cudaFuncSetAttribute(psgd_gemm_nt_kernel<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  psgd_gemm_nt_kernel<RT><<<ntiles, GEMM_THREADS, smem, stream>>>(a);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int RT>
static int launch_nn(const GemmArgs& a, int ntiles, cudaStream_t stream) {
  constexpr int RPW = RT <= 8 ? 4 : (RT == 16 ? 2 : 1);
  psgd_gemm_nn_kernel<RT, RPW><<<ntiles, GEMM_THREADS, 0, stream>>>(a);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

#define PSGD_DISPATCH_RT(FN)                                   \
  if (max_r <= 1) return FN<1>(a, ntiles, stream);             \
  if (max_r <= 2) return FN<2>(a, ntiles, stream);             \
  if (max_r <= 4) return FN<4>(a, ntiles, stream);             \
  if (max_r <= 8) return FN<8>(a, ntiles, stream);             \
  if (max_r <= 16) return FN<16>(a, ntiles, stream);           \
  return FN<32>(a, ntiles, stream);

// Rows handled by one NN tile for the template rank that `max_r` selects (the planner needs it).
PSGD_API int psgd_gemm_nn_tile_rows(int max_r) {
  const int rt = max_r <= 1 ? 1 : max_r <= 2 ? 2 : max_r <= 4 ? 4 : max_r <= 8 ? 8 : max_r <= 16 ? 16 : 32;
  return GEMM_WARPS * (rt <= 8 ? 4 : (rt == 16 ? 2 : 1));
}
PSGD_API int psgd_gemm_nt_max_rows(int max_r) { return max_r <= 16 ? NT_MAX_ROWS : NT_MAX_ROWS / 2; }
PSGD_API int psgd_gemm_template_rank(int max_r) {
  return max_r <= 1 ? 1 : max_r <= 2 ? 2 : max_r <= 4 ? 4 : max_r <= 8 ? 8 : max_r <= 16 ? 16 : 32;
}

// `transposed` != 0: NT (Q = M^T P); else NN (P = M Q). Every tile carries the access width of
// its matrix (`vec`: 4 needs a 16-byte aligned base and m % 4 == 0; 2 an 8-byte aligned base and
// an even m). `out2`, when not null, receives a second copy of the fresh factor.
PSGD_API int psgd_gemm_ffma_launch(int transposed, int max_r, const void* mats, const void* tiles, int ntiles,
                                   const float* in, float* out, float* out2, int ncorr,
                                   const float* const* corr_fac, const float* const* corr_c, float* partial,
                                   int* tickets, const void* comm, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  if (max_r > PSGD_MAX_RANK || ncorr > PSGD_MAX_HIST) {
    psgd_set_error("psgd_gemm_ffma_launch: rank %d or history %d beyond the compiled maximum", max_r, ncorr);
    return -1;
  }
  GemmArgs a;
  fill_args(a, mats, tiles, in, out, out2, ncorr, corr_fac, corr_c, partial, tickets, comm);
  if (transposed) { PSGD_DISPATCH_RT(launch_nt) }
  PSGD_DISPATCH_RT(launch_nn)
}

#ifdef PSGD_BOUNDS_CHECK
PSGD_BOUNDS_EXPORT(psgd_bounds_read_products)
// Capacities (floats / counters) of the partial-sum arena, the ticket table and the P- and Q-shaped
// factor buffers of the launches that follow; 0 leaves a capacity unchecked.
PSGD_API int psgd_debug_limits_products(long long partial_floats, long long tickets, long long p_floats, long long q_floats) {
  PSGD_CUDA_OK(cudaMemcpyToSymbol(g_lim_partial, &partial_floats, sizeof(long long)));
  PSGD_CUDA_OK(cudaMemcpyToSymbol(g_lim_tickets, &tickets, sizeof(long long)));
  PSGD_CUDA_OK(cudaMemcpyToSymbol(g_lim_p, &p_floats, sizeof(long long)));
  PSGD_CUDA_OK(cudaMemcpyToSymbol(g_lim_q, &q_floats, sizeof(long long)));
  return 0;
}
#endif
