// Batched orthonormalisation of tall factor matrices (one CTA per unit).
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
// The same launch also produces the small cross products C_i = F_i^T X_hat against earlier
// factors of the same side; the product kernels use them to deflate algebraically.
#include "psgd_common.cuh"

typedef struct {
  int32_t x_off;      // float offset of the unit inside the factor buffer
  int32_t sub_len;    // rows of one sub-matrix
  int32_t nsub;       // sub-matrices in the unit (> 1 only for rank-1 groups)
  int32_t r;          // columns
  int32_t first_mat;  // descriptor index of sub-matrix 0 (sub-matrices are consecutive)
  int32_t pad[3];
} PsgdOrthUnit;  // 32 bytes

struct OrthArgs {
  const PsgdOrthUnit* units;
  float* x;                          // factor buffer, orthonormalised in place
  float* copy_to;                    // optional second destination (same layout) or null
  int nprev;                         // earlier same-side factor buffers
  const float* prev[PSGD_MAX_HIST];  // each laid out like x
  float* cmat[PSGD_MAX_HIST];        // out: [mat][r*r] blocks with stride PSGD_CMAT_STRIDE
};

constexpr int ORTH_THREADS = 512;
constexpr int ORTH_WARPS = ORTH_THREADS / 32;

// Deterministic CTA-wide sum of per-thread rows acc[RT] that belong to column `j`
// (thread layout: j = tid % RT, row lane = tid / RT). Result in sm[j*RT + k].
template <int RT>
__device__ __forceinline__ void cta_reduce_rows(double (&acc)[RT], double* sm, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int k = 0; k < RT; ++k) {
#pragma unroll
    for (int o = 16; o >= RT; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
  }
  for (int w = 0; w < ORTH_WARPS; ++w) {
    if (warp == w && lane < RT) {
#pragma unroll
      for (int k = 0; k < RT; ++k) {
        if (w == 0) sm[lane * RT + k] = acc[k];
        else sm[lane * RT + k] += acc[k];
      }
    }
    __syncthreads();
  }
}

template <int RT>
__global__ void __launch_bounds__(ORTH_THREADS) psgd_orth_kernel(OrthArgs a) {
  const PsgdOrthUnit u = a.units[blockIdx.x];
  const int r = u.r;
  const int tid = threadIdx.x;
  const long long len = (long long)u.sub_len * u.nsub;
  float* __restrict__ x = a.x + u.x_off;
  float* __restrict__ x2 = a.copy_to ? a.copy_to + u.x_off : nullptr;

  __shared__ double sG[RT * RT];
  __shared__ double sR[RT * RT];     // upper-triangular Cholesky factor, then its inverse
  __shared__ double sRinv[RT * RT];
  __shared__ int sDead[RT];          // -1: alive; >= 0: row of the substituted basis vector; -2: dropped
  __shared__ float sScale;

  const int j = tid % RT;            // column owned by this thread in the Gram phases
  const int rl = tid / RT;           // row lane
  constexpr int NRL = ORTH_THREADS / RT;

  // ---- Gram matrix -----------------------------------------------------------------------
  {
    double acc[RT];
#pragma unroll
    for (int k = 0; k < RT; ++k) acc[k] = 0.0;
    if (j < r) {
#pragma unroll 4
      for (long long row = rl; row < len; row += NRL) {
        const float* xr = x + row * r;
        const double xj = (double)xr[j];
#pragma unroll
        for (int k = 0; k < RT; ++k)
          if (k < r) acc[k] = fma(xj, (double)xr[k], acc[k]);
      }
    }
    cta_reduce_rows<RT>(acc, sG, tid);
  }

  if (RT == 1 || r == 1) {
    // joint Frobenius norm of the whole unit, float32 semantics of the division
    if (tid == 0) {
      float nrm = (float)sqrt(sG[0]);
      sScale = fmaxf(nrm, 1e-16f);
    }
    __syncthreads();
    const float d = sScale;
    for (long long i = tid; i < len; i += ORTH_THREADS) {
      float v = x[i] / d;
      x[i] = v;
      if (x2) x2[i] = v;
    }
  } else {
    // ---- Cholesky (one warp) with canonical-vector substitution -------------------------
    if (tid < 32) {
      const int lane = tid;
      if (lane < RT) sDead[lane] = -1;
      for (int e = lane; e < RT * RT; e += 32) { sR[e] = 0.0; sRinv[e] = 0.0; }
      __syncwarp();
      for (int c = 0; c < r; ++c) {
        // pivot of column c
        int attempt = 0;
        double piv = 0.0;
        while (true) {
          double s = sG[c * RT + c];
          for (int i = 0; i < c; ++i) s -= sR[i * RT + c] * sR[i * RT + c];
          const double ref = sG[c * RT + c];
          const bool ok = (ref > 0.0) && (s > 1e-12 * ref);
          if (ok) { piv = sqrt(s); break; }
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
              sR[i * RT + c] = t / sR[i * RT + i];
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
            for (int i = 0; i < c; ++i) sR[i * RT + c] = 0.0;
          }
          __syncwarp();
          continue;  // row c of R stays zero right of the diagonal
        }
        if (lane == 0) sR[c * RT + c] = piv;
        // row c of R, right of the diagonal: one lane per column
        for (int k = c + 1 + lane; k < r; k += 32) {
          double t = sG[c * RT + k];
          for (int i = 0; i < c; ++i) t -= sR[i * RT + c] * sR[i * RT + k];
          sR[c * RT + k] = t / piv;
        }
        __syncwarp();
      }
      // inverse of the upper-triangular R, one lane per column
      for (int c = lane; c < r; c += 32) {
        for (int i = c; i >= 0; --i) {
          double t = (i == c) ? 1.0 : 0.0;
          for (int k = i + 1; k <= c; ++k) t -= sR[i * RT + k] * sRinv[k * RT + c];
          sRinv[i * RT + c] = t / sR[i * RT + i];
        }
        if (sDead[c] == -2)
          for (int i = 0; i <= c; ++i) sRinv[i * RT + c] = 0.0;
      }
    }
    __syncthreads();

    // ---- X <- X' R^-1 --------------------------------------------------------------------
#pragma unroll 2
    for (long long row = tid; row < len; row += ORTH_THREADS) {
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

  // ---- cross products against earlier same-side factors ---------------------------------
  if (a.nprev > 0) {
    __syncthreads();  // make this CTA's writes to x visible to all its threads
    for (int p = 0; p < a.nprev; ++p) {
      const float* __restrict__ f = a.prev[p] + u.x_off;
      for (int s = 0; s < u.nsub; ++s) {
        double acc[RT];
#pragma unroll
        for (int k = 0; k < RT; ++k) acc[k] = 0.0;
        if (j < r) {
          const long long lo = (long long)s * u.sub_len, hi = lo + u.sub_len;
#pragma unroll 4
          for (long long row = lo + rl; row < hi; row += NRL) {
            const double fj = (double)f[row * r + j];
            const float* xr = x + row * r;
#pragma unroll
            for (int k = 0; k < RT; ++k)
              if (k < r) acc[k] = fma(fj, (double)xr[k], acc[k]);
          }
        }
        cta_reduce_rows<RT>(acc, sG, tid);
        float* c_out = a.cmat[p] + (long long)(u.first_mat + s) * PSGD_CMAT_STRIDE;
        for (int e = tid; e < r * r; e += ORTH_THREADS) c_out[e] = (float)sG[(e / r) * RT + (e % r)];
        __syncthreads();
      }
    }
  }
}

// Launch one CTA per unit; all units of one call share the template rank RT >= max r.
PSGD_API int psgd_orth_launch(const void* units, int nunits, int max_r, float* x, float* copy_to, int nprev,
                              const float* const* prev, float* const* cmat, cudaStream_t stream) {
  if (nunits <= 0) return 0;
  if (max_r > PSGD_MAX_RANK || nprev > PSGD_MAX_HIST) {
    psgd_set_error("psgd_orth_launch: rank %d or history %d beyond the compiled maximum", max_r, nprev);
    return -1;
  }
  OrthArgs a;
  a.units = (const PsgdOrthUnit*)units;
  a.x = x;
  a.copy_to = copy_to;
  a.nprev = nprev;
  for (int i = 0; i < PSGD_MAX_HIST; ++i) {
    a.prev[i] = i < nprev ? prev[i] : nullptr;
    a.cmat[i] = i < nprev ? cmat[i] : nullptr;
  }
  if (max_r <= 1) psgd_orth_kernel<1><<<nunits, ORTH_THREADS, 0, stream>>>(a);
  else if (max_r <= 2) psgd_orth_kernel<2><<<nunits, ORTH_THREADS, 0, stream>>>(a);
  else if (max_r <= 4) psgd_orth_kernel<4><<<nunits, ORTH_THREADS, 0, stream>>>(a);
  else if (max_r <= 8) psgd_orth_kernel<8><<<nunits, ORTH_THREADS, 0, stream>>>(a);
  else if (max_r <= 16) psgd_orth_kernel<16><<<nunits, ORTH_THREADS, 0, stream>>>(a);
  else psgd_orth_kernel<32><<<nunits, ORTH_THREADS, 0, stream>>>(a);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
