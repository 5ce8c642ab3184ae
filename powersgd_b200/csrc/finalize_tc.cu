// Decompression + error feedback (+ SGD) with the rank-K update on the tensor cores.
//
// Same contract as psgd_finalize_kernel (finalize.cu): for a 128 x 64 tile of one gradient matrix
//     residual  M   <- M - sum_t Lloc_t Rloc_t^T          update  A = (1/W) sum_t Lsum_t Rsum_t^T
// followed by `out <- A` or the SGD step. Here the two rank-K products (K = T * r) are tcgen05
// MMAs: the factor panels are staged in shared memory as K-major, 128-byte-swizzled operands and
// the 128 x 64 accumulators live in TMEM, so the CUDA cores only stream the tile: TMA load of M,
// one TMEM read per row, coalesced stores. FP32 accuracy comes from splitting along K:
//     A' = [a_hi | a_lo | a_hi]    B' = [b_hi | b_hi | b_lo]    (hi = TF32 part, lo = remainder)
// so that one TF32 MMA chain over K' = 3K computes a_hi b_hi + a_lo b_hi + a_hi b_lo.
//
// Roles (160 threads): warp 4 allocates TMEM, issues the TMA loads of the M tile and, once the
// 128 staging threads have arrived, the MMAs; warps 0-3 stage the panels, then each thread owns
// one tile row for the TMEM -> shared-memory step, then the warps write rows out coalesced.
// All mbarrier waits are bounded (status word + abort flag), as in lowrank_tc.cu.
#include <cuda.h>

#include "psgd_comm.cuh"

namespace {

constexpr int FT_THREADS = 160;
constexpr int FT_ROWS = 128;
constexpr int FT_COLS = 64;
constexpr int FT_MAX_KP = 128;                      // padded 3K; 4 slabs of 32
constexpr int FT_TILE_BYTES = FT_ROWS * FT_COLS * 4;  // 32 KiB
constexpr uint64_t FT_WAIT_LIMIT_NS = 2000000000ull;

struct FinTcArgs {
  const PsgdMat* mats;
  const PsgdTile* tiles;
  const CUtensorMap* maps;     // [2 * mat]: box 32 x 32, SWIZZLE_128B
  const PsgdHyper* hyper;
  int nhist;
  const float* lloc[PSGD_MAX_HIST];
  const float* rloc[PSGD_MAX_HIST];
  const float* lsum[PSGD_MAX_HIST];
  const float* rsum[PSGD_MAX_HIST];
  float inv_world;
  int fused_sgd;
  int* status;
};

__device__ __forceinline__ uint32_t ft_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool ft_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(ft_smem(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ft_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (ft_try_wait(bar, parity)) return true;
  const uint64_t t0 = psgd_globaltimer_ns();
  while (!ft_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (psgd_globaltimer_ns() - t0 > FT_WAIT_LIMIT_NS) {
      *abort_flag = 1;
      if (status) {
        // plain store: the word may live in mapped pinned host memory, which the host reads
        *((volatile int*)status) = (int)PSGD_TIMEOUT_MBARRIER;
        __threadfence_system();
      }
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ uint64_t ft_desc(uint32_t saddr) {  // K-major, 128-byte swizzle, 8-row groups 1 KiB apart
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ float ft_hi(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

// byte offset of element (row, kk) inside a K-major swizzled panel with `rows` rows per 32-float slab
__device__ __forceinline__ uint32_t ft_panel_off(int rows, int row, int kk) {
  return (uint32_t)(kk >> 5) * (uint32_t)(rows * 128) + (uint32_t)row * 128u +
         ((uint32_t)((((kk & 31) >> 2) ^ (row & 7))) << 4) + (uint32_t)(kk & 3) * 4u;
}
// byte offset of element (row, col) of the 128 x 64 tile stored as two 32-column swizzled slabs
__device__ __forceinline__ uint32_t ft_tile_off(int row, int col) {
  return (uint32_t)(col >> 5) * (FT_ROWS * 128) + (uint32_t)row * 128u +
         ((uint32_t)((((col & 31) >> 2) ^ (row & 7))) << 4) + (uint32_t)(col & 3) * 4u;
}

__device__ __forceinline__ void ft_tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float ft_sgd(float g, float& p, float& mo, const PsgdHyper& h) {
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) g = fmaf(h.weight_decay, p, g);
  if (h.has_momentum) {
    const float b = fmaf(h.momentum, mo, h.one_minus_dampening * g);
    mo = b;
    g = h.nesterov ? fmaf(h.momentum, b, g) : b;
  }
  p = fmaf(-h.lr, g, p);
  return p;
}

template <bool SAME>
__global__ void __launch_bounds__(FT_THREADS) psgd_finalize_tc_kernel(const __grid_constant__ FinTcArgs a, int nslab) {
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(FT_COLS >> 3) << 17) |
                             ((uint32_t)(FT_ROWS >> 4) << 24);
  constexpr int TMEM_COLS = SAME ? 64 : 128;
  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  const CUtensorMap* map = a.maps + 2 * t.mat;
  const int r = mt.r, m = mt.m;
  const int K = a.nhist * r;
  const int Kp = nslab * 32;  // >= 3K, zero padded
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ __align__(1024) uint8_t ft_smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)ft_smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sM = base;                            // gradient tile, then residual
  uint8_t* sU = sM + FT_TILE_BYTES;              // update tile
  uint8_t* sAl = sU + FT_TILE_BYTES;             // A' from Lloc   [nslab][128][128 B]
  uint8_t* sBl = sAl + nslab * 16384;            // B' from Rloc   [nslab][ 64][128 B]
  uint8_t* sAs = sBl + nslab * 8192;             // (not SAME) A' from Lsum
  uint8_t* sBs = sAs + nslab * 16384;            // (not SAME) B' from Rsum
  __shared__ __align__(8) uint64_t bar_m, bar_panels, bar_mma;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ft_smem(&bar_m)), "r"(1));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ft_smem(&bar_panels)), "r"(128));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ft_smem(&bar_mma)), "r"(1));
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ft_smem(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  volatile int* abort_flag = &s_abort;

  if (warp == 4) {
    if (lane == 0) {
      // gradient tile: 2 column slabs x 4 row boxes of 32 x 32 floats
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ft_smem(&bar_m)), "r"(FT_TILE_BYTES) : "memory");
#pragma unroll
      for (int cs = 0; cs < 2; ++cs)
#pragma unroll
        for (int rb = 0; rb < 4; ++rb)
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
              ::"r"(ft_smem(sM + cs * (FT_ROWS * 128) + rb * 4096)), "l"(map), "r"(ft_smem(&bar_m)),
                "r"(t.col0 + 32 * cs), "r"(t.row0 + 32 * rb) : "memory");
      if (ft_wait(&bar_panels, 0, abort_flag, a.status)) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t al = ft_smem(sAl), bl = ft_smem(sBl), as = ft_smem(sAs), bs = ft_smem(sBs);
        for (int ks = 0; ks < Kp / 8; ++ks) {
          const uint32_t ao = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
          const uint32_t bo = (uint32_t)(ks >> 2) * 8192u + (uint32_t)(ks & 3) * 32u;
          const uint32_t acc = ks != 0 ? 1u : 0u;
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
              ::"r"(tmem), "l"(ft_desc(al + ao)), "l"(ft_desc(bl + bo)), "r"(IDESC), "r"(acc) : "memory");
          if (!SAME)
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                ::"r"(tmem + 64), "l"(ft_desc(as + ao)), "l"(ft_desc(bs + bo)), "r"(IDESC), "r"(acc) : "memory");
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ft_smem(&bar_mma)) : "memory");
    }
  } else {
    // ---- stage the factor panels (split along K) ----
    auto stage = [&](uint8_t* panel, int prow, int valid, const float* const* fac, long long off0, bool is_a) {
      for (int e = tid; e < prow * K; e += 128) {
        const int row = e / K, k = e % K;
        float v = 0.f;
        if (row < valid) v = __ldg(fac[k / r] + off0 + (long long)row * r + (k % r));
        const float hi = ft_hi(v), lo = v - hi;
        *reinterpret_cast<float*>(panel + ft_panel_off(prow, row, k)) = hi;
        *reinterpret_cast<float*>(panel + ft_panel_off(prow, row, K + k)) = is_a ? lo : hi;
        *reinterpret_cast<float*>(panel + ft_panel_off(prow, row, 2 * K + k)) = is_a ? hi : lo;
      }
      const int pad = Kp - 3 * K;
      for (int e = tid; e < prow * pad; e += 128)
        *reinterpret_cast<float*>(panel + ft_panel_off(prow, e / pad, 3 * K + e % pad)) = 0.f;
    };
    const long long poff = mt.p_off + (long long)t.row0 * r, qoff = mt.q_off + (long long)t.col0 * r;
    stage(sAl, FT_ROWS, t.rows, a.lloc, poff, true);
    stage(sBl, FT_COLS, t.cols, a.rloc, qoff, false);
    if (!SAME) {
      stage(sAs, FT_ROWS, t.rows, a.lsum, poff, true);
      stage(sBs, FT_COLS, t.cols, a.rsum, qoff, false);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ft_smem(&bar_panels)) : "memory");

    // ---- one tile row per thread: residual = M - E into sM, update into sU ----
    const bool ok = ft_wait(&bar_mma, 0, abort_flag, a.status) && ft_wait(&bar_m, 0, abort_flag, a.status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
      for (int j = 0; j < FT_COLS / 16; ++j) {
        float e[16], u[16];
        ft_tmem_ld16(trow + 16 * j, e);
        if (!SAME) ft_tmem_ld16(trow + 64 + 16 * j, u);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off = ft_tile_off(tid, 16 * j + 4 * q);
          float4 g = *reinterpret_cast<float4*>(sM + off);
          g.x -= e[4 * q]; g.y -= e[4 * q + 1]; g.z -= e[4 * q + 2]; g.w -= e[4 * q + 3];
          *reinterpret_cast<float4*>(sM + off) = g;
          const float* src = SAME ? e : u;
          *reinterpret_cast<float4*>(sU + off) = make_float4(src[4 * q] * a.inv_world, src[4 * q + 1] * a.inv_world,
                                                             src[4 * q + 2] * a.inv_world, src[4 * q + 3] * a.inv_world);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
  if (s_abort) {
    const uint64_t t0 = psgd_globaltimer_ns();
    while (psgd_globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    return;
  }

  // ---- coalesced write-out: a warp writes one row (64 floats) per instruction ----
  if (warp < 4) {
    const PsgdHyper h = a.hyper[mt.hyper];
    const int c = 2 * lane;
    if (c < t.cols) {
      for (int lr = warp; lr < t.rows; lr += 4) {
        const uint32_t off = ft_tile_off(lr, c);
        const float2 res = *reinterpret_cast<const float2*>(sM + off);
        const float2 upd = *reinterpret_cast<const float2*>(sU + off);
        const long long g = (long long)(t.row0 + lr) * m + t.col0 + c;
        *reinterpret_cast<float2*>(mt.grad + g) = res;
        if (a.fused_sgd) {
          float2 p = *reinterpret_cast<const float2*>(mt.param + g);
          float2 mo = make_float2(0.f, 0.f);
          if (h.has_momentum) mo = *reinterpret_cast<const float2*>(mt.mom + g);
          ft_sgd(upd.x, p.x, mo.x, h);
          ft_sgd(upd.y, p.y, mo.y, h);
          *reinterpret_cast<float2*>(mt.param + g) = p;
          if (h.has_momentum) *reinterpret_cast<float2*>(mt.mom + g) = mo;
        } else {
          *reinterpret_cast<float2*>(mt.out + g) = upd;
        }
      }
    }
  }
}

}  // namespace

// Largest total factor width K = (half-iterations x rank) this kernel takes: 3K must fit 128.
PSGD_API int psgd_finalize_tc_max_k() { return FT_MAX_KP / 3; }

// Tiles are 128 rows x 64 columns (PsgdTile row0/rows/col0/cols); every matrix in the list needs a
// tensor map (see psgd_tma_encode_matrix) and 16-byte aligned grad / param / mom / out pointers.
PSGD_API int psgd_finalize_tc_launch(const void* mats, const void* tiles, int ntiles, const void* maps, const void* hyper,
                                     int nhist, int rank, const float* const* lloc, const float* const* rloc,
                                     const float* const* lsum, const float* const* rsum, float inv_world, int fused_sgd,
                                     int* status, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  const int K = nhist * rank;
  if (nhist > PSGD_MAX_HIST || 3 * K > FT_MAX_KP) {
    psgd_set_error("psgd_finalize_tc_launch: %d half-iterations x rank %d exceeds K = %d", nhist, rank, FT_MAX_KP / 3);
    return -1;
  }
  FinTcArgs a;
  a.mats = (const PsgdMat*)mats;
  a.tiles = (const PsgdTile*)tiles;
  a.maps = (const CUtensorMap*)maps;
  a.hyper = (const PsgdHyper*)hyper;
  a.nhist = nhist;
  bool same = true;
  for (int i = 0; i < PSGD_MAX_HIST; ++i) {
    a.lloc[i] = i < nhist ? lloc[i] : nullptr;
    a.rloc[i] = i < nhist ? rloc[i] : nullptr;
    a.lsum[i] = i < nhist ? lsum[i] : nullptr;
    a.rsum[i] = i < nhist ? rsum[i] : nullptr;
    if (i < nhist) same = same && lloc[i] == lsum[i] && rloc[i] == rsum[i];
  }
  a.inv_world = inv_world;
  a.fused_sgd = fused_sgd;
  a.status = status;
  const int nslab = (3 * K + 31) / 32;
  const size_t smem = 1024 + 2 * (size_t)FT_TILE_BYTES + (size_t)nslab * (16384 + 8192) * (same ? 1 : 2);
  if (same) {
    PSGD_CUDA_OK(cudaFuncSetAttribute(psgd_finalize_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    psgd_finalize_tc_kernel<true><<<ntiles, FT_THREADS, smem, stream>>>(a, nslab);
  } else {
    PSGD_CUDA_OK(cudaFuncSetAttribute(psgd_finalize_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    psgd_finalize_tc_kernel<false><<<ntiles, FT_THREADS, smem, stream>>>(a, nslab);
  }
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}
