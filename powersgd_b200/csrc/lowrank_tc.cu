// Grouped tall-skinny products on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   NT:  Q[m, r] = M^T P_hat  - corrections          D[128 columns of M, N] += A^T-tile * B
//   NN:  P[n, r] = M   Q_hat  - corrections          D[128 rows    of M, N] += A-tile   * B
//
// Same contract, tile descriptors, deterministic split reduction, algebraic-deflation epilogue
// and peer push as the CUDA-core kernels in lowrank_ffma.cu; this path takes over for matrices
// that TMA can address (16-byte aligned base, row pitch a multiple of 16 bytes) and that are
// large enough to be HBM bound.
//
// Data flow per CTA (192 threads, one output tile of 128 x r, K walked in slabs of 32):
//   warp 4   one lane issues TMA loads of the gradient tile (4 boxes of 32 x 32 floats with
//            128-byte swizzle) into a 3-stage shared-memory ring; completion on an mbarrier.
//   warps 0-3  split precision: write A_lo = A - tf32(A) beside the landed tile and stage the
//            32 x r slab of the small factor as [B_hi | B_lo] (K-major, 128-byte swizzle), then
//            fence.proxy.async and arrive on the stage's "ready" mbarrier.
//   warp 5   one lane issues tcgen05.mma kind::tf32 (M = 128, N = 2 r_pad, K = 8): A from shared
//            memory (MN-major for NT, K-major for NN), accumulator in TMEM, FP32 accumulate;
//            tcgen05.commit releases the stage and, at the end, signals the epilogue.
//   warps 0-3  epilogue: tcgen05.ld the 128 x N accumulator (one TMEM lane per thread), add the
//            hi and lo halves, then partial-sum / correction / store / peer-push as in the FFMA
//            path.
// (A_hi + A_lo)(B_hi + B_lo) with every term a TF32 product accumulated in FP32 reproduces the
// FP32 product to ~1e-6 relative, which the 1e-5 parity target needs; `split = 0` runs plain
// TF32 (one MMA per K step) for users who accept 1e-3.
//
// Every mbarrier wait is bounded: when the limit expires the CTA sets an abort flag and a global
// status word, all roles fall through, TMEM is released and the kernel returns.
#include <cuda.h>
#include <string.h>

#include "psgd_comm.cuh"

namespace {

constexpr int TC_THREADS = 320;     // warps 0-3: converters + epilogue, 4: TMA, 5: MMA, 6-9: converters
constexpr int TC_NCONV = 256;       // converter threads: the conversion pass, not the memory system,
                                    // paced the pipeline with four warps
constexpr int TC_BK = 32;           // K elements (floats) per stage
constexpr int TC_TILE = 128;        // output rows of the accumulator (UMMA M)
constexpr int TC_A_BYTES = TC_TILE * TC_BK * 4;   // 16 KiB
constexpr int TC_STAGES = 4;      // landing ring of the gradient tile (TMA -> shared memory)
constexpr int TC_OP_STAGES = 2;   // ring of the operands the converters write (A_lo, factor slab):
                                  // shallower than the landing ring, two CTAs still fit one SM
constexpr int TC_SEG = 16;        // stages (512 K rows) accumulated in TMEM before the sum moves to registers:
                                  // the tensor core adds into its FP32 accumulator with truncation, a bias
                                  // that grows with the length of the chain (measured against the FP64
                                  // product: 5e-7 relative for 512 rows, 1e-5 for 2048, 6e-5 for 6272). Two
                                  // accumulators alternate, so the MMA stream never waits for the hand-over.
constexpr int TC_DRAIN_LAG = 2;   // stages converted into the next segment before the finished one is read
constexpr uint64_t TC_WAIT_LIMIT_NS = 2000000000ull;  // 2 s

struct TcArgs {
  const PsgdMat* mats;
  const PsgdTile* tiles;
  const CUtensorMap* maps;   // two per matrix, box 32 columns x 32 rows: [2*mat] SWIZZLE_128B (NN),
                             // [2*mat + 1] SWIZZLE_128B_ATOM_32B (NT, MN-major A operand)
  const float* in;
  float* out;
  int ncorr;
  const float* corr_fac[PSGD_MAX_HIST];
  const float* corr_c[PSGD_MAX_HIST];
  float* partial;
  int* tickets;
  const PsgdCommDev* comm;
  float* out2;               // optional second copy of the fresh factor or null
  int* status;               // word (device or mapped host memory) set on a wait that ran out
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false (and raises the abort flag) when the limit expires or another
// role already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = psgd_globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (psgd_globaltimer_ns() - t0 > TC_WAIT_LIMIT_NS) {
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

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor, version 1 (Blackwell). layout_type 2 = 128-byte swizzle with
// 16-byte atoms (K-major operands); 1 = 128-byte swizzle with 32-byte atoms, the only swizzled
// layout the tensor core accepts for MN-major 32-bit (TF32) operands.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type = 2) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version
  d |= (uint64_t)layout_type << 61;
  return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ float tf32_hi(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

template <int N>
__device__ __forceinline__ void tmem_load_row(uint32_t taddr, float* v);
template <>
__device__ __forceinline__ void tmem_load_row<16>(uint32_t taddr, float* v) {
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
template <>
__device__ __forceinline__ void tmem_load_row<32>(uint32_t taddr, float* v) {
  tmem_load_row<16>(taddr, v);
  tmem_load_row<16>(taddr + 16, v + 16);
}
template <>
__device__ __forceinline__ void tmem_load_row<64>(uint32_t taddr, float* v) {
  tmem_load_row<32>(taddr, v);
  tmem_load_row<32>(taddr + 32, v + 32);
}

// RP: factor rank padded to 8 / 16 / 32. N of the MMA is max(16, (SPLIT ? 2 : 1) * RP).
template <bool TRANSPOSED, int RP, bool SPLIT>
__global__ void __launch_bounds__(TC_THREADS, 2) psgd_gemm_tc_kernel(const __grid_constant__ TcArgs a) {
  constexpr int N2 = ((SPLIT ? 2 : 1) * RP) < 16 ? 16 : ((SPLIT ? 2 : 1) * RP);
  constexpr int B_BYTES = N2 * 128;
  constexpr int TMEM_COLS = 2 * N2 < 32 ? 32 : 2 * N2;   // two accumulators of N2 columns
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((TRANSPOSED ? 1u : 0u) << 15) |
                             ((uint32_t)(N2 >> 3) << 17) | ((uint32_t)(TC_TILE >> 4) << 24);

  const PsgdTile t = a.tiles[blockIdx.x];
  const PsgdMat mt = a.mats[t.mat];
  const CUtensorMap* map = a.maps + 2 * t.mat + (TRANSPOSED ? 1 : 0);
  const int r = mt.r;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;                                            // [STAGES][16 KiB]
  uint8_t* sAlo = sA + TC_STAGES * TC_A_BYTES;                   // [OP_STAGES][16 KiB] (SPLIT only)
  uint8_t* sB = sAlo + (SPLIT ? TC_OP_STAGES * TC_A_BYTES : 0);  // [OP_STAGES][B_BYTES]
  // full: tile landed (TMA -> converters); ready: A_lo and factor slab written (converters -> MMA);
  // empty: landing slot consumed (MMA -> TMA); op_empty: operand slot consumed (MMA -> converters)
  // seg: the MMAs of a segment are complete (MMA -> converters); drained: its accumulator was read
  __shared__ __align__(8) uint64_t bar_full[TC_STAGES], bar_empty[TC_STAGES], bar_ready[TC_OP_STAGES], bar_op_empty[TC_OP_STAGES];
  __shared__ __align__(8) uint64_t bar_seg[2], bar_drained[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort, s_last;

  // K range of this tile and the global coordinates of its first box
  const int k_begin = TRANSPOSED ? t.row0 : t.col0;
  const int k_len = TRANSPOSED ? t.rows : t.cols;
  const int k_limit = TRANSPOSED ? mt.n : mt.m;     // factor rows beyond this are zero
  const int nk = (k_len + TC_BK - 1) / TC_BK;
  const int out0 = TRANSPOSED ? t.col0 : t.row0;     // first output row of the accumulator
  const int out_len = TRANSPOSED ? t.cols : t.rows;  // valid accumulator rows (<= 128)

  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int s = 0; s < TC_OP_STAGES; ++s) {
      mbar_init(&bar_ready[s], TC_NCONV);
      mbar_init(&bar_op_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bar_seg[b], 1);
      mbar_init(&bar_drained[b], 128);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  volatile int* abort_flag = &s_abort;
  // warps 0-3: running FP32 sum of the finished segments of accumulator row (warp * 32 + lane)
  float sum[N2];
#pragma unroll
  for (int i = 0; i < N2; ++i) sum[i] = 0.f;
  const int nseg = (nk + TC_SEG - 1) / TC_SEG;
  int next_drain = 0;
  bool drain_ok = true;
  auto drain = [&](int g) {
    // segment g used accumulator (g & 1) for the (g >> 1)-th time
    if (drain_ok) drain_ok = mbar_wait(&bar_seg[g & 1], (g >> 1) & 1, abort_flag, a.status);
    if (drain_ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float d[N2];
      tmem_load_row<N2>(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)((g & 1) * N2), d);
#pragma unroll
      for (int i = 0; i < N2; ++i) sum[i] += d[i];
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    mbar_arrive(&bar_drained[g & 1]);
  };

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % TC_STAGES;
        const uint32_t ph = (kb / TC_STAGES) & 1;
        if (!mbar_wait(&bar_empty[s], ph ^ 1, abort_flag, a.status)) break;
        mbar_expect_tx(&bar_full[s], TC_A_BYTES);
        uint8_t* dst = sA + s * TC_A_BYTES;
        const int k0 = k_begin + kb * TC_BK;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // NT: 4 column groups of 32 at the same 32 rows; NN: 4 row groups of 32 at the same 32 columns
          const int x = TRANSPOSED ? out0 + 32 * j : k0;
          const int y = TRANSPOSED ? k0 : out0 + 32 * j;
          tma_load_2d(dst + j * 4096, map, x, y, &bar_full[s]);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < nk && ok; ++kb) {
        const int s = kb % TC_STAGES, so = kb % TC_OP_STAGES;
        const int g = kb / TC_SEG;
        const bool seg_first = kb % TC_SEG == 0;
        // accumulator (g & 1) was last used by segment g - 2: wait until the converters have read it
        if (seg_first && g >= 2) ok = mbar_wait(&bar_drained[g & 1], ((g >> 1) - 1) & 1, abort_flag, a.status);
        if (!ok) break;
        ok = mbar_wait(&bar_ready[so], (kb / TC_OP_STAGES) & 1, abort_flag, a.status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + (uint32_t)((g & 1) * N2);
        const uint32_t aaddr = smem_u32(sA + s * TC_A_BYTES);
        const uint32_t laddr = smem_u32(sAlo + so * TC_A_BYTES);
        const uint32_t baddr = smem_u32(sB + so * B_BYTES);
#pragma unroll
        for (int ks = 0; ks < TC_BK / 8; ++ks) {
          // NT (MN-major A): a slab holds 32 K rows of 128 bytes (32 columns); 8 K rows = two
          //   512-byte swizzle atoms (stride 512), the four 32-column slabs are 4 KiB apart.
          // NN (K-major A): 8 K floats = 32 bytes further along each 128-byte row, row groups 1 KiB apart.
          const uint64_t da = TRANSPOSED ? umma_desc(aaddr + ks * 1024, 4096, 512, 1) : umma_desc(aaddr + ks * 32, 16, 1024);
          const uint64_t db = umma_desc(baddr + ks * 32, 16, 1024);
          umma_tf32(acc, da, db, IDESC, (seg_first && ks == 0) ? 0u : 1u);
          if (SPLIT) {
            const uint64_t dl = TRANSPOSED ? umma_desc(laddr + ks * 1024, 4096, 512, 1) : umma_desc(laddr + ks * 32, 16, 1024);
            umma_tf32(acc, dl, db, IDESC, 1u);
          }
        }
        umma_commit(&bar_empty[s]);      // frees the landing slot once these MMAs have read it
        umma_commit(&bar_op_empty[so]);  // and the operand slot
        if (kb % TC_SEG == TC_SEG - 1 || kb == nk - 1) umma_commit(&bar_seg[g & 1]);  // segment complete
      }
    }
  } else {
    // ---------------- converters (then epilogue) ----------------
    const int ctid = warp < 4 ? tid : tid - 64;   // index among the converter threads
    const float* __restrict__ fac = a.in + (TRANSPOSED ? mt.p_off : mt.q_off);
    // each thread stages RP / 4 factor values per stage; they are fetched one stage ahead so
    // that their L2 latency hides behind the wait for the gradient tile
    constexpr int PER_THREAD = TC_BK * RP / TC_NCONV;
    float pre[PER_THREAD];
    auto fetch = [&](int kb) {
      const int k0 = k_begin + kb * TC_BK;
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i) {
        const int e = ctid + i * TC_NCONV;
        const int k = e / RP, n = e % RP;
        float v = 0.f;
        if (kb < nk && n < r && k0 + k < k_limit && kb * TC_BK + k < k_len) v = __ldg(fac + (long long)(k0 + k) * r + n);
        pre[i] = v;
      }
    };
    fetch(0);
    for (int kb = 0; kb < nk; ++kb) {
      const int s = kb % TC_STAGES, so = kb % TC_OP_STAGES;
      const uint32_t ph = (kb / TC_STAGES) & 1;
      float cur[PER_THREAD];
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i) cur[i] = pre[i];
      fetch(kb + 1);
      if (!mbar_wait(&bar_full[s], ph, abort_flag, a.status)) break;
      if (!mbar_wait(&bar_op_empty[so], ((kb / TC_OP_STAGES) & 1) ^ 1, abort_flag, a.status)) break;
      if (SPLIT) {
        const float4* src = reinterpret_cast<const float4*>(sA + s * TC_A_BYTES);
        float4* dst = reinterpret_cast<float4*>(sAlo + so * TC_A_BYTES);
#pragma unroll
        for (int i = 0; i < TC_A_BYTES / 16 / TC_NCONV; ++i) {
          const float4 v = src[ctid + i * TC_NCONV];
          dst[ctid + i * TC_NCONV] = make_float4(v.x - tf32_hi(v.x), v.y - tf32_hi(v.y), v.z - tf32_hi(v.z), v.w - tf32_hi(v.w));
        }
      }
      // factor slab: B[n][k] for k in this stage, K-major rows of 128 bytes with 128-byte swizzle
      uint8_t* bt = sB + so * B_BYTES;
#pragma unroll
      for (int i = 0; i < PER_THREAD; ++i) {
        const int e = ctid + i * TC_NCONV;
        const int k = e / RP, n = e % RP;
        const float v = cur[i];
        const float hi = tf32_hi(v);
        const uint32_t off = (uint32_t)(((k >> 2) ^ (n & 7)) << 4) + (uint32_t)(k & 3) * 4u;
        *reinterpret_cast<float*>(bt + n * 128 + off) = hi;
        if (SPLIT) *reinterpret_cast<float*>(bt + (n + RP) * 128 + off) = v - hi;   // (n + RP) & 7 == n & 7
      }
      if ((SPLIT ? 2 : 1) * RP < N2) {
        // pad rows of B (only when RP = 8 without split): zero
        for (int e = ctid; e < (N2 - (SPLIT ? 2 : 1) * RP) * 32; e += TC_NCONV)
          reinterpret_cast<float*>(bt + (SPLIT ? 2 : 1) * RP * 128)[e] = 0.f;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&bar_ready[so]);
      // a finished segment is read a couple of stages later, when its MMAs are certainly done
      while (warp < 4 && next_drain < nseg - 1 && kb >= (next_drain + 1) * TC_SEG - 1 + TC_DRAIN_LAG) drain(next_drain++);
    }
    while (warp < 4 && next_drain < nseg) drain(next_drain++);
  }

  // ---------------- epilogue ----------------
  float* sSum = reinterpret_cast<float*>(base);  // [128][RP], aliases stage 0 once the MMAs are done
  if (warp < 4) {
    // all segments are in registers (the last drain waited for the last MMAs, so no stage of
    // shared memory is read any more and sSum may alias it)
#pragma unroll
    for (int n = 0; n < RP; ++n) sSum[tid * RP + n] = SPLIT ? sum[n] + sum[n + RP] : sum[n];
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_abort) {
    // a wait ran out: give copies that may still be in flight time to land before this CTA's
    // shared memory is handed to another one
    const uint64_t t0 = psgd_globaltimer_ns();
    while (psgd_globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }

  constexpr int tile_elems = TC_TILE * RP;
  bool owner = true;
  if (t.nsplit > 1) {
    float* mine = a.partial + (long long)(t.slot0 + t.split) * tile_elems;
    for (int e = tid; e < tile_elems; e += TC_THREADS) __stcg(mine + e, sSum[e]);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (psgd_atom_add_acqrel_gpu(a.tickets + t.ticket, 1) == t.nsplit - 1);
    __syncthreads();
    owner = s_last != 0;
    if (owner) {
      __threadfence();
      for (int e = tid; e < tile_elems; e += TC_THREADS) {
        float s = 0.f;
        for (int p = 0; p < t.nsplit; ++p) s += __ldcg(a.partial + (long long)(t.slot0 + p) * tile_elems + e);
        sSum[e] = s;
      }
      if (tid == 0) a.tickets[t.ticket] = 0;
      __syncthreads();
    }
  }

  const long long out_off = TRANSPOSED ? mt.q_off : mt.p_off;
  float* __restrict__ fout = a.out + out_off;
  uint2* push[PSGD_MAX_WORLD];
  int npush = 0, e1 = 0;
  if (a.comm != nullptr && owner) {
    const PsgdCommDev c = *a.comm;
    e1 = *c.epoch + 1;
    npush = c.world;
    for (int p = 0; p < PSGD_MAX_WORLD; ++p) push[p] = p < c.world ? psgd_comm_slot(c, p, e1, c.rank) + out_off : nullptr;
  }
  for (int e = tid; owner && e < out_len * r; e += TC_THREADS) {
    const int lr = e / r, k = e % r;
    const long long row = out0 + lr;
    float s = sSum[lr * RP + k];
    for (int i = 0; i < a.ncorr; ++i) {
      const float* f = a.corr_fac[i] + out_off + row * r;
      const float* cm = a.corr_c[i] + (long long)mt.index * PSGD_CMAT_STRIDE;
      float dsum = 0.f;
      for (int l = 0; l < r; ++l) dsum = fmaf(f[l], cm[l * r + k], dsum);
      s -= dsum;
    }
    fout[row * r + k] = s;
    if (a.out2) a.out2[out_off + row * r + k] = s;
    for (int p = 0; p < npush; ++p) psgd_comm_store(push[p] + row * r + k, s, e1);
  }
}

template <bool TRANSPOSED, int RP, bool SPLIT>
int launch_tc(const TcArgs& a, int ntiles, cudaStream_t stream) {
  constexpr int N2 = ((SPLIT ? 2 : 1) * RP) < 16 ? 16 : ((SPLIT ? 2 : 1) * RP);
  const size_t smem = 1024 + (size_t)TC_STAGES * TC_A_BYTES + (size_t)TC_OP_STAGES * ((SPLIT ? TC_A_BYTES : 0) + N2 * 128);
  static bool configured = false;
  if (!configured) {
    PSGD_CUDA_OK(cudaFuncSetAttribute(psgd_gemm_tc_kernel<TRANSPOSED, RP, SPLIT>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  psgd_gemm_tc_kernel<TRANSPOSED, RP, SPLIT><<<ntiles, TC_THREADS, smem, stream>>>(a);
  PSGD_CUDA_OK(cudaGetLastError());
  return 0;
}

template <bool TRANSPOSED, bool SPLIT>
int dispatch_rank(const TcArgs& a, int max_r, int ntiles, cudaStream_t stream) {
  if (max_r <= 8) return launch_tc<TRANSPOSED, 8, SPLIT>(a, ntiles, stream);
  if (max_r <= 16) return launch_tc<TRANSPOSED, 16, SPLIT>(a, ntiles, stream);
  return launch_tc<TRANSPOSED, 32, SPLIT>(a, ntiles, stream);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

}  // namespace

// Rank padding the tensor-core kernels use for `max_r` (slot size of a split tile is 128 * this).
PSGD_API int psgd_gemm_tc_rank_pad(int max_r) { return max_r <= 8 ? 8 : max_r <= 16 ? 16 : 32; }

// Writes TWO 128-byte tensor maps for a row-major float32 matrix [n, m] (box 32 x 32, zero fill
// outside) into host memory at `out`: first with the 16-byte-atom 128-byte swizzle (tiles used
// as K-major operands), then with the 32-byte-atom variant (tiles used as MN-major operands).
// The matrix must be 16-byte aligned with m % 4 == 0.
PSGD_API int psgd_tma_encode_matrix(void* out, const float* base, int n, int m) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    psgd_set_error("cuTensorMapEncodeTiled is not available from this driver");
    return -1;
  }
  if (((uintptr_t)base & 15u) != 0 || (m % 4) != 0) {
    psgd_set_error("psgd_tma_encode_matrix: base %p / row pitch %d floats not 16-byte aligned", (const void*)base, m);
    return -1;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)m, (cuuint64_t)n};
  const cuuint64_t strides[1] = {(cuuint64_t)m * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUtensorMapSwizzle modes[2] = {CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B};
  for (int i = 0; i < 2; ++i) {
    CUtensorMap map;
    const CUresult rc = fn(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, modes[i], CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      psgd_set_error("cuTensorMapEncodeTiled (swizzle mode %d) failed with CUresult %d for a %d x %d matrix", i,
                     (int)rc, n, m);
      return -1;
    }
    memcpy((char*)out + i * sizeof(map), &map, sizeof(map));
  }
  return 0;
}

// Same contract as psgd_gemm_ffma_launch; `maps` is a device array of tensor maps indexed like
// `mats`; `split` selects split-precision TF32 (FP32-accurate) or plain TF32.
PSGD_API int psgd_gemm_tc_launch(int transposed, int split, int max_r, const void* mats, const void* tiles, int ntiles,
                                 const void* maps, const float* in, float* out, float* out2, int ncorr,
                                 const float* const* corr_fac, const float* const* corr_c, float* partial,
                                 int* tickets, const void* comm, int* status, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  if (max_r > PSGD_MAX_RANK || ncorr > PSGD_MAX_HIST) {
    psgd_set_error("psgd_gemm_tc_launch: rank %d or history %d beyond the compiled maximum", max_r, ncorr);
    return -1;
  }
  TcArgs a;
  a.mats = (const PsgdMat*)mats;
  a.tiles = (const PsgdTile*)tiles;
  a.maps = (const CUtensorMap*)maps;
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
  a.status = status;
  if (transposed) return split ? dispatch_rank<true, true>(a, max_r, ntiles, stream) : dispatch_rank<true, false>(a, max_r, ntiles, stream);
  return split ? dispatch_rank<false, true>(a, max_r, ntiles, stream) : dispatch_rank<false, false>(a, max_r, ntiles, stream);
}
