// Batched orthonormalisation of tall factor matrices, spread over the whole GPU.
//
// Replaces the reference's per-group `torch.linalg.qr` / joint-norm division
// (powersgd/orthogonalization.py:4-8) and the research harness' column-serial Gram-Schmidt
// (paper-code/gradient_reducers.py:945-956) with a Gram-matrix formulation that walks the
// tall matrix exactly twice, whatever the rank:
//
//   G = X^T X        accumulated in float64, fixed summation order (bit-reproducible)
//   G = R^T R        Cholesky in float64 by one warp; R^-1 by back substitution
//   X <- X R^-1      rounded to float32 once
//
// With a float64 Gram matrix one pass is as orthonormal as float32 can express for any X
// that float32 can represent (error ~ 1e-16 * cond(X)^2 + 6e-8). A pivot below 1e-12 of its
// column's squared norm means the column is noise at float32 input precision; it is replaced
// by a canonical basis vector (what Householder QR yields for a zero column), so a factor
// that collapsed to zero (an all-zero gradient) recovers on the next step.
//
// Rank-1 units keep the reference's quirk: ONE Frobenius norm over the whole shape group
// (all B matrices jointly), floored at 1e-16, divides every entry.
//
// Two launches. The first cuts every unit into row chunks, one CTA each: partial Gram matrices
// (and partial cross products F_i^T X against earlier factors of the same side) go to scratch;
// the CTA that arrives last at the unit's ticket adds the partials in chunk order, factorises,
// and publishes R^-1 plus the cross products C_i = (F_i^T X) R^-1 = F_i^T X_hat that the product
// kernels use to deflate algebraically. The second launch applies R^-1 to every row chunk. A long
// factor (an embedding with 50 000 rows, rank 16) thus takes microseconds instead of the
// hundreds that one CTA per unit needed.
//
// Multi-GPU: the factor to orthonormalise is the SUM over workers of what the previous product
// launch pushed into this rank's slot arena. The first launch is then also the consumer of that
// in-kernel all-reduce (powersgd/powersgd.py:205-209 in the reference is a blocking library
// call): while staging its chunk every CTA polls the tagged words of the W slots, adds them in
// rank order, and writes the sum to the factor buffer and to the copy the decompression reads.
#include "psgd_bounds.cuh"
#include "psgd_comm.cuh"

typedef struct {
  int32_t x_off;      // float offset of the unit inside the factor buffer
  int32_t sub_len;    // rows of one sub-matrix
  int32_t nsub;       // sub-matrices in the unit (> 1 only for rank-1 groups)
  int32_t r;          // columns
  int32_t first_mat;  // descriptor index of sub-matrix 0 (sub-matrices are consecutive)
  int32_t chunk0;     // index of the unit's first chunk (chunks of a unit are consecutive)
  int32_t nchunks;
  int32_t pad;
} PsgdOrthUnit;  // 32 bytes

typedef struct {
  int32_t unit;
  int32_t sub;    // sub-matrix the chunk lies in (chunks never straddle sub-matrices)
  int32_t row0;   // first row, counted from the start of the unit
  int32_t rows;
} PsgdOrthChunk;  // 16 bytes

struct OrthArgs {
  const PsgdOrthUnit* units;
  const PsgdOrthChunk* chunks;
  float* x;                          // factor buffer, orthonormalised in place
  float* copy_to;                    // optional second destination (same layout) or null
  int nprev;                         // earlier same-side factor buffers
  const float* prev[PSGD_MAX_HIST];  // each laid out like x
  float* cmat[PSGD_MAX_HIST];        // out: [mat][r*r] blocks with stride PSGD_CMAT_STRIDE
  double* part;                      // scratch: [chunk][1 + nprev][RT*RT] partial sums
  double* rinv;                      // scratch: [unit][RT*RT]  R^-1 (rank 1: [0] = the divisor)
  int* dead;                         // scratch: [unit][RT]     column status (see sDead)
  int* tickets;                      // [unit], zero between launches
  const PsgdCommDev* comm;           // not null: x is first gathered from the channel's slots (see above)
  float* sum_out;                    // with comm: second destination of the gathered sum (laid out like x)
};

constexpr int ORTH_THREADS = 256;
constexpr int ORTH_CHUNK_FLOATS = 2048;  // rows per chunk = 2048 / RT (8 KiB of the factor). The chunk
                                         // is staged in shared memory as float64: conversions issue at
                                         // a fraction of the FMA rate, so each value is converted once
                                         // and not once per pair it takes part in

// Sum over the rows of a chunk of a[row][j] * b[row][k] for every pair (j, k), in float64 and in
// a fixed order: row groups stride through the chunk, then the groups are added in order.
// Result: out[j * RT + k] (global scratch), written by the threads with tid < RT * RT.
template <int RT>
__device__ __forceinline__ void chunk_pairs(const double* sa, const double* sb, int rows, double* red, double* out, int tid) {
  constexpr int NP = RT * RT;
  constexpr int PP = NP > ORTH_THREADS ? NP / ORTH_THREADS : 1;     // pairs per thread
  constexpr int NG = NP >= ORTH_THREADS ? 1 : ORTH_THREADS / NP;    // row groups
  const int g = NP >= ORTH_THREADS ? 0 : tid / NP;
  double acc[PP];
#pragma unroll
  for (int q = 0; q < PP; ++q) acc[q] = 0.0;
  const int p0 = NP >= ORTH_THREADS ? tid : tid % NP;
#pragma unroll 4
  for (int row = g; row < rows; row += NG) {
#pragma unroll
    for (int q = 0; q < PP; ++q) {
      const int p = p0 + q * ORTH_THREADS;
      acc[q] = fma(sa[row * RT + p / RT], sb[row * RT + p % RT], acc[q]);
    }
  }
  if (NG == 1) {
#pragma unroll
    for (int q = 0; q < PP; ++q) out[p0 + q * ORTH_THREADS] = acc[q];
  } else {
    red[tid] = acc[0];
    __syncthreads();
    if (tid < NP) {
      double s = 0.0;
      for (int gg = 0; gg < NG; ++gg) s += red[gg * NP + tid];
      out[tid] = s;
    }
    __syncthreads();
  }
}

template <int RT>
__global__ void __launch_bounds__(ORTH_THREADS) psgd_orth_gram_kernel(OrthArgs a) {
  constexpr int NP = RT * RT;
  const PsgdOrthChunk ch = a.chunks[blockIdx.x];
  const PsgdOrthUnit u = a.units[ch.unit];
  const int r = u.r;
  const int tid = threadIdx.x;
  const float* __restrict__ x = a.x + u.x_off;
#ifdef PSGD_BOUNDS_CHECK
  {
    bool ok = true;
    ok &= PSGD_BC(r >= 1 && r <= RT, 5, PSGD_BC_RANK, r, RT);
    ok &= PSGD_BC(ch.row0 >= 0 && ch.rows > 0 && (long long)ch.row0 + ch.rows <= (long long)u.sub_len * u.nsub && ch.rows * RT <= ORTH_CHUNK_FLOATS,
                  5, PSGD_BC_CHUNK, (long long)ch.row0 + ch.rows, (long long)u.sub_len * u.nsub);
    ok &= PSGD_BC((int)blockIdx.x >= u.chunk0 && (int)blockIdx.x < u.chunk0 + u.nchunks, 5, PSGD_BC_CHUNK, blockIdx.x, u.chunk0 + u.nchunks);
    if (!ok) return;
  }
#endif

  __shared__ __align__(16) double sx[ORTH_CHUNK_FLOATS];
  __shared__ __align__(16) double sf[ORTH_CHUNK_FLOATS];
  __shared__ double red[ORTH_THREADS];
  __shared__ double sG[NP];
  __shared__ int sDead[RT];      // -1: alive; >= 0: row of the substituted basis vector; -2: dropped
  __shared__ int s_last;
  // used by the finishing CTA only, after the staging buffers are dead
  static_assert(NP <= ORTH_CHUNK_FLOATS, "R must fit a staging buffer");
  double* sR = sf;      // upper-triangular Cholesky factor
  double* sRinv = sx;
  __shared__ double sDiagInv[RT];                  // 1 / R[c][c]: float64 divisions and square roots
                                                   // are long dependent instruction chains, so each
                                                   // column pays for one and multiplies afterwards

  // ---- partial sums of this chunk ---------------------------------------------------------
  const int stride = 1 + a.nprev;
  double* my_part = a.part + (long long)blockIdx.x * stride * NP;
  if (a.comm != nullptr) {
    // gather: this chunk is a contiguous run of rows * r words in every slot
    const PsgdCommDev& c = *a.comm;
    const int e1 = *c.epoch + 1;
    const long long base = (long long)u.x_off + (long long)ch.row0 * r;
    float* __restrict__ xw = a.x + base;
    float* __restrict__ sw = a.sum_out + base;
    const int n = ch.rows * r;
    for (int e = tid; e < ch.rows * RT; e += ORTH_THREADS)
      if (e % RT >= r) sx[e] = 0.0;
    bool ok = true;
    constexpr int NB = 4;
    for (int i0 = tid; i0 < n; i0 += NB * ORTH_THREADS) {
      int64_t idx[NB];
      float v[NB];
#pragma unroll
      for (int j = 0; j < NB; ++j) idx[j] = (i0 + j * ORTH_THREADS < n) ? base + i0 + j * ORTH_THREADS : -1;
      psgd_comm_reduce_batch<NB>(c, e1, idx, NB, v, ok);
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const int i = i0 + j * ORTH_THREADS;
        if (i < n) {
          xw[i] = v[j];
          sw[i] = v[j];
          sx[(i / r) * RT + i % r] = (double)v[j];
        }
      }
    }
    psgd_comm_close_epoch(c, e1);  // (CTA barrier inside) every word of this chunk has been read
  } else {
    for (int e = tid; e < ch.rows * RT; e += ORTH_THREADS) {
      const int row = e / RT, c = e % RT;
      sx[e] = c < r ? (double)x[(long long)(ch.row0 + row) * r + c] : 0.0;
    }
  }
  __syncthreads();
  chunk_pairs<RT>(sx, sx, ch.rows, red, my_part, tid);
  for (int p = 0; p < a.nprev; ++p) {
    const float* __restrict__ f = a.prev[p] + u.x_off;
    __syncthreads();
    for (int e = tid; e < ch.rows * RT; e += ORTH_THREADS) {
      const int row = e / RT, c = e % RT;
      sf[e] = c < r ? (double)f[(long long)(ch.row0 + row) * r + c] : 0.0;
    }
    __syncthreads();
    chunk_pairs<RT>(sf, sx, ch.rows, red, my_part + (long long)(1 + p) * NP, tid);
  }

  // ---- the chunk that arrives last finishes the unit ----------------------------------------
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = (psgd_atom_add_acqrel_gpu(a.tickets + ch.unit, 1) == u.nchunks - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const double* unit_part = a.part + (long long)u.chunk0 * stride * NP;
  if (tid < NP) {
    double s = 0.0;
    for (int c = 0; c < u.nchunks; ++c) s += __ldcg(unit_part + (long long)c * stride * NP + tid);
    sG[tid] = s;
  }
  __syncthreads();
  double* rinv_out = a.rinv + (long long)ch.unit * NP;
  int* dead_out = a.dead + (long long)ch.unit * RT;
  const long long len = (long long)u.sub_len * u.nsub;

  if (RT == 1 || r == 1) {
    // joint Frobenius norm of the whole unit, float32 semantics of the division
    const float d = fmaxf((float)sqrt(sG[0]), 1e-16f);
    if (tid == 0) {
      rinv_out[0] = (double)d;
      dead_out[0] = -1;
    }
    // cross products per sub-matrix: (sum of f * x over the sub-matrix) / d
    for (int e = tid; e < a.nprev * u.nsub; e += ORTH_THREADS) {
      const int p = e / u.nsub, s = e % u.nsub;
      double t = 0.0;
      for (int c = 0; c < u.nchunks; ++c)
        if (a.chunks[u.chunk0 + c].sub == s) t += __ldcg(unit_part + ((long long)c * stride + 1 + p) * NP);
      a.cmat[p][(long long)(u.first_mat + s) * PSGD_CMAT_STRIDE] = (float)(t / (double)d);
    }
  } else {
    // ---- Cholesky (one warp) with canonical-vector substitution -------------------------
    if (tid < 32) {
      const int lane = tid;
      if (lane < RT) sDead[lane] = -1;
      for (int e = lane; e < NP; e += 32) { sR[e] = 0.0; sRinv[e] = 0.0; }
      __syncwarp();
      for (int c = 0; c < r; ++c) {
        // pivot of column c
        int attempt = 0;
        double piv = 0.0, inv_piv = 0.0;
        while (true) {
          double s = sG[c * RT + c];
          for (int i = 0; i < c; ++i) s -= sR[i * RT + c] * sR[i * RT + c];
          const double ref = sG[c * RT + c];
          const bool ok = (ref > 0.0) && (s > 1e-12 * ref);
          if (ok) { inv_piv = rsqrt(s); piv = s * inv_piv; break; }
          if (attempt == 2) { piv = 0.0; break; }
          // substitute column c by the basis vector e_row; its Gram entries are matrix entries
          const long long row = (attempt == 0 ? c : c + r) % len;
          ++attempt;
          __syncwarp();
          if (lane < r) {
            double g;
            if (lane == c) g = 1.0;
            else if (sDead[lane] >= 0) g = (sDead[lane] == (int)row) ? 1.0 : 0.0;
            else if (sDead[lane] == -2) g = 0.0;
            else g = (double)x[row * r + lane];
            sG[c * RT + lane] = g;
            sG[lane * RT + c] = g;
          }
          if (lane == 0) sDead[c] = (int)row;
          __syncwarp();
          // entries above the diagonal of column c were built from the old column: redo them
          if (lane == 0) {
            for (int i = 0; i < c; ++i) {
              if (sDead[i] == -2) { sR[i * RT + c] = 0.0; continue; }
              double t = sG[i * RT + c];
              for (int l = 0; l < i; ++l) t -= sR[l * RT + i] * sR[l * RT + c];
              sR[i * RT + c] = t * sDiagInv[i];
            }
          }
          __syncwarp();
        }
        __syncwarp();
        if (piv == 0.0) {
          // could not be completed: drop the column (its output is zero)
          if (lane == 0) {
            sDead[c] = -2;
            sR[c * RT + c] = 1.0;
            sDiagInv[c] = 1.0;
            for (int i = 0; i < c; ++i) sR[i * RT + c] = 0.0;
          }
          __syncwarp();
          continue;  // row c of R stays zero right of the diagonal
        }
        if (lane == 0) {
          sR[c * RT + c] = piv;
          sDiagInv[c] = inv_piv;
        }
        // row c of R, right of the diagonal: one lane per column
        for (int k = c + 1 + lane; k < r; k += 32) {
          double t = sG[c * RT + k];
          for (int i = 0; i < c; ++i) t -= sR[i * RT + c] * sR[i * RT + k];
          sR[c * RT + k] = t * inv_piv;
        }
        __syncwarp();
      }
      // inverse of the upper-triangular R, one lane per column
      for (int c = lane; c < r; c += 32) {
        for (int i = c; i >= 0; --i) {
          double t = (i == c) ? 1.0 : 0.0;
          for (int k = i + 1; k <= c; ++k) t -= sR[i * RT + k] * sRinv[k * RT + c];
          sRinv[i * RT + c] = t * sDiagInv[i];
        }
        if (sDead[c] == -2)
          for (int i = 0; i <= c; ++i) sRinv[i * RT + c] = 0.0;
      }
    }
    __syncthreads();
    if (tid < NP) rinv_out[tid] = sRinv[tid];
    if (tid < RT) dead_out[tid] = sDead[tid];
    // ---- cross products: C_p = (F_p^T X') R^-1, X' = X with the substituted columns ----------
    for (int p = 0; p < a.nprev; ++p) {
      const float* __restrict__ f = a.prev[p] + u.x_off;
      __syncthreads();
      if (tid < NP) {
        const int j = tid / RT, k = tid % RT;
        double s = 0.0;
        if (j < r && k < r) {
          const int d = sDead[k];
          if (d == -1) {
            for (int c = 0; c < u.nchunks; ++c) s += __ldcg(unit_part + ((long long)c * stride + 1 + p) * NP + tid);
          } else if (d >= 0) {
            s = (double)f[(long long)d * r + j];  // column k of X' is the basis vector e_d
          }
        }
        sG[tid] = s;
      }
      __syncthreads();
      if (tid < NP) {
        const int j = tid / RT, k = tid % RT;
        if (j < r && k < r) {
          double o = 0.0;
          for (int l = 0; l <= k; ++l) o = fma(sG[j * RT + l], sRinv[l * RT + k], o);
          a.cmat[p][(long long)u.first_mat * PSGD_CMAT_STRIDE + j * r + k] = (float)o;
        }
      }
    }
  }
  if (tid == 0) a.tickets[ch.unit] = 0;  // ready for the next launch
}

// Second launch: X <- X' R^-1 (rank 1: X / d) on every row chunk, optionally mirrored to copy_to.
template <int RT>
__global__ void __launch_bounds__(ORTH_THREADS) psgd_orth_apply_kernel(OrthArgs a) {
  constexpr int NP = RT * RT;
  const PsgdOrthChunk ch = a.chunks[blockIdx.x];
  const PsgdOrthUnit u = a.units[ch.unit];
  const int r = u.r;
  const int tid = threadIdx.x;
  float* __restrict__ x = a.x + u.x_off;
  float* __restrict__ x2 = a.copy_to ? a.copy_to + u.x_off : nullptr;
  __shared__ double sRinv[NP];
  __shared__ int sDead[RT];
  if (tid < NP) sRinv[tid] = a.rinv[(long long)ch.unit * NP + tid];
  if (tid < RT) sDead[tid] = a.dead[(long long)ch.unit * RT + tid];
  __syncthreads();

  if (RT == 1 || r == 1) {
    const float d = (float)sRinv[0];
    for (int i = tid; i < ch.rows; i += ORTH_THREADS) {
      const float v = x[ch.row0 + i] / d;
      x[ch.row0 + i] = v;
      if (x2) x2[ch.row0 + i] = v;
    }
    return;
  }
  for (int lr = tid; lr < ch.rows; lr += ORTH_THREADS) {
    const long long row = ch.row0 + lr;
    float* xr = x + row * r;
    double xin[RT];
#pragma unroll
    for (int k = 0; k < RT; ++k) {
      double v = 0.0;
      if (k < r) {
        const int d = sDead[k];
        v = (d == -1) ? (double)xr[k] : ((d >= 0 && d == (int)row) ? 1.0 : 0.0);
      }
      xin[k] = v;
    }
#pragma unroll
    for (int c = 0; c < RT; ++c) {
      if (c < r) {
        double o = 0.0;
#pragma unroll
        for (int k = 0; k <= c; ++k) o = fma(xin[k], sRinv[k * RT + c], o);
        const float of = (float)o;
        xr[c] = of;
        if (x2) x2[row * r + c] = of;
      }
    }
  }
}

template <int RT>
static void orth_launch_rt(const OrthArgs& a, int nchunks, cudaStream_t stream) {
  psgd_orth_gram_kernel<RT><<<nchunks, ORTH_THREADS, 0, stream>>>(a);
  psgd_orth_apply_kernel<RT><<<nchunks, ORTH_THREADS, 0, stream>>>(a);
}

// Template rank used for factors of rank max_r, and the rows of one chunk at that rank.
PSGD_API int psgd_orth_template_rank(int max_r) {
  return max_r <= 1 ? 1 : max_r <= 2 ? 2 : max_r <= 4 ? 4 : max_r <= 8 ? 8 : max_r <= 16 ? 16 : 32;
}
PSGD_API int psgd_orth_chunk_rows(int max_r) { return ORTH_CHUNK_FLOATS / psgd_orth_template_rank(max_r); }
// Scratch per chunk (doubles) for `nprev` earlier factors; per unit: RT*RT doubles and RT ints.
PSGD_API int psgd_orth_part_doubles(int max_r, int nprev) {
  const int rt = psgd_orth_template_rank(max_r);
  return (1 + nprev) * rt * rt;
}

// units / chunks: device tables; all units of one call share the template rank RT >= max r.
// part: nchunks * psgd_orth_part_doubles(max_r, nprev) doubles; rinv: nunits * RT*RT doubles;
// dead: nunits * RT ints; tickets: nunits ints, zero (the kernel leaves them zero).
// comm / sum_out: see OrthArgs (null for a single worker or when x already holds the factor).
PSGD_API int psgd_orth_launch(const void* units, int nunits, const void* chunks, int nchunks, int max_r, float* x,
                              float* copy_to, int nprev, const float* const* prev, float* const* cmat,
                              double* part, double* rinv, int* dead, int* tickets, const void* comm,
                              float* sum_out, cudaStream_t stream) {
  if (nunits <= 0 || nchunks <= 0) return 0;
  if (max_r > PSGD_MAX_RANK || nprev > PSGD_MAX_HIST) {
    psgd_set_error("psgd_orth_launch: rank %d or history %d beyond the compiled maximum", max_r, nprev);
    return -1;
  }
  OrthArgs a;
  a.units = (const PsgdOrthUnit*)units;
  a.chunks = (const PsgdOrthChunk*)chunks;
  a.x = x;
  a.copy_to = copy_to;
  a.nprev = nprev;
  for (int i = 0; i < PSGD_MAX_HIST; ++i) {
    a.prev[i] = i < nprev ? prev[i] : nullptr;
    a.cmat[i] = i < nprev ? cmat[i] : nullptr;
  }
  a.part = part;
  a.rinv = rinv;
  a.dead = dead;
  a.tickets = tickets;
  a.comm = (const PsgdCommDev*)comm;
  a.sum_out = sum_out;
  if (comm != nullptr && sum_out == nullptr) {
    psgd_set_error("psgd_orth_launch: a channel was given without a destination for the gathered sum");
    return -1;
  }
  switch (psgd_orth_template_rank(max_r)) {
    case 1: orth_launch_rt<1>(a, nchunks, stream); break;
    case 2: orth_launch_rt<2>(a, nchunks, stream); break;
    case 4: orth_launch_rt<4>(a, nchunks, stream); break;
    case 8: orth_launch_rt<8>(a, nchunks, stream); break;
    case 16: orth_launch_rt<16>(a, nchunks, stream); break;
    default: orth_launch_rt<32>(a, nchunks, stream); break;
  }
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

#ifdef PSGD_BOUNDS_CHECK
PSGD_BOUNDS_EXPORT(psgd_bounds_read_orth)
#endif
