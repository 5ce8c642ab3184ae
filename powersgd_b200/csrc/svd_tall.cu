// Batched thin SVD of tall-skinny matrices (c <= 32 columns), one CTA per matrix.
//
// The ATOMO and SVD reducers of the research harness factorise reshaped gradient tensors whose
// 2-D views are tall and narrow (a [64,64,3,3] kernel becomes 2048 x 18); the reference ships
// them to the CPU for LAPACK because the GPU SVD it had was slower
// (paper-code/gradient_reducers.py:1019-1029). For that shape class the SVD is cheap on the GPU:
//     G = X^T X            float64, fixed summation order (as in the orthonormalisation kernel)
//     G = V diag(s^2) V^T  cyclic Jacobi on the c x c matrix by one warp, float64
//     U = X V diag(1/s)    one more pass over X
// Singular values come out sorted in descending order; columns whose singular value is below
// 1e-7 of the largest get a zero left vector (they carry no energy at float32 precision).
#include "psgd_common.cuh"

namespace {

constexpr int SV_THREADS = 512;
constexpr int SV_MAXC = 32;

typedef struct {
  int64_t x_off;   // float offset of X (row-major [n, c]) in the input buffer
  int64_t u_off;   // float offset of U ([n, c]) in the U buffer
  int32_t s_off;   // float offset of s ([c]) in the S buffer
  int32_t v_off;   // float offset of V ([c, c], row-major: V[i][j] = component i of right vector j)
  int32_t n, c;
} PsgdSvdItem;  // 32 bytes

__global__ void __launch_bounds__(SV_THREADS) psgd_svd_tall_kernel(const PsgdSvdItem* items, const float* __restrict__ xin,
                                                                    float* __restrict__ u, float* __restrict__ s_out,
                                                                    float* __restrict__ v_out, int sweeps) {
  const PsgdSvdItem it = items[blockIdx.x];
  const int n = it.n, c = it.c, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* __restrict__ x = xin + it.x_off;
  __shared__ double G[SV_MAXC][SV_MAXC + 1];
  __shared__ double V[SV_MAXC][SV_MAXC + 1];
  __shared__ double part[SV_THREADS / 32][SV_MAXC];
  __shared__ double sval[SV_MAXC];
  __shared__ int order[SV_MAXC];

  // ---- Gram matrix: thread (row lane, column j) accumulates row j of G -----------------------
  const int j = tid % SV_MAXC, rl = tid / SV_MAXC;
  constexpr int NRL = SV_THREADS / SV_MAXC;  // 16 row lanes = one per warp
  double acc[SV_MAXC];
#pragma unroll
  for (int k = 0; k < SV_MAXC; ++k) acc[k] = 0.0;
  if (j < c) {
    for (int row = rl; row < n; row += NRL) {
      const float* xr = x + (long long)row * c;
      const double xj = (double)xr[j];
#pragma unroll
      for (int k = 0; k < SV_MAXC; ++k)
        if (k < c) acc[k] = fma(xj, (double)xr[k], acc[k]);
    }
  }
  // one warp holds one row lane (32 columns): add the 16 warps in index order
  for (int k = 0; k < SV_MAXC; ++k) {
    part[warp][lane] = acc[k];
    __syncthreads();
    if (warp == 0) {
      double t = 0.0;
      for (int w = 0; w < SV_THREADS / 32; ++w) t += part[w][lane];
      G[lane][k] = t;
      V[lane][k] = lane == k ? 1.0 : 0.0;
    }
    __syncthreads();
  }

  // ---- cyclic Jacobi on G (symmetric c x c), lanes own rows / columns ------------------------
  if (warp == 0) {
    for (int sweep = 0; sweep < sweeps; ++sweep) {
      double off = 0.0;
      for (int p = 0; p < c - 1; ++p)
        for (int q = p + 1; q < c; ++q) {
          const double gpq = G[p][q];
          off += gpq * gpq;
          if (fabs(gpq) > 1e-300) {
            const double theta = (G[q][q] - G[p][p]) / (2.0 * gpq);
            const double t = (theta >= 0.0 ? 1.0 : -1.0) / (fabs(theta) + sqrt(theta * theta + 1.0));
            const double cs = 1.0 / sqrt(t * t + 1.0), sn = t * cs;
            __syncwarp();
            if (lane < c) {  // columns p, q of G and V
              const double gkp = G[lane][p], gkq = G[lane][q];
              G[lane][p] = cs * gkp - sn * gkq;
              G[lane][q] = sn * gkp + cs * gkq;
              const double vkp = V[lane][p], vkq = V[lane][q];
              V[lane][p] = cs * vkp - sn * vkq;
              V[lane][q] = sn * vkp + cs * vkq;
            }
            __syncwarp();
            if (lane < c) {  // rows p, q of G
              const double gpk = G[p][lane], gqk = G[q][lane];
              G[p][lane] = cs * gpk - sn * gqk;
              G[q][lane] = sn * gpk + cs * gqk;
            }
            __syncwarp();
          }
        }
      if (off < 1e-30 * (1e-300 + fabs(G[0][0]) * fabs(G[0][0]))) break;
    }
    // sort by descending eigenvalue (selection sort by lane 0: c <= 32)
    if (lane == 0) {
      for (int i = 0; i < c; ++i) order[i] = i;
      for (int i = 0; i < c; ++i) {
        int best = i;
        for (int k = i + 1; k < c; ++k)
          if (G[order[k]][order[k]] > G[order[best]][order[best]]) best = k;
        const int tmp = order[i]; order[i] = order[best]; order[best] = tmp;
      }
      for (int i = 0; i < c; ++i) sval[i] = sqrt(fmax(G[order[i]][order[i]], 0.0));
    }
    __syncwarp();
    if (lane < c) {
      s_out[it.s_off + lane] = (float)sval[lane];
      for (int i = 0; i < c; ++i) v_out[it.v_off + i * c + lane] = (float)V[i][order[lane]];
    }
  }
  __syncthreads();

  // ---- U = X V / s ---------------------------------------------------------------------------
  const double floor_s = 1e-7 * sval[0];
  for (int row = tid; row < n; row += SV_THREADS) {
    const float* xr = x + (long long)row * c;
    float* ur = u + it.u_off + (long long)row * c;
    for (int col = 0; col < c; ++col) {
      const int src = order[col];
      double t = 0.0;
      for (int k = 0; k < c; ++k) t = fma((double)xr[k], V[k][src], t);
      ur[col] = sval[col] > floor_s && sval[col] > 0.0 ? (float)(t / sval[col]) : 0.f;
    }
  }
}

}  // namespace

PSGD_API int psgd_svd_tall_max_cols() { return SV_MAXC; }

// items: device array of `count` descriptors (see PsgdSvdItem); every matrix has c <= 32 <= n.
PSGD_API int psgd_svd_tall_launch(const void* items, int count, const float* x, float* u, float* s, float* v,
                                  cudaStream_t stream) {
  if (count <= 0) return 0;
  psgd_svd_tall_kernel<<<count, SV_THREADS, 0, stream>>>((const PsgdSvdItem*)items, x, u, s, v, 30);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
