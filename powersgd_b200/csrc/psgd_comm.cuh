// In-kernel collectives over NVLink peer memory: device-side context and primitives.
//
// Every rank owns one "slot arena", allocated with cudaMalloc and mapped into every peer through
// CUDA IPC. The protocol is flag-in-data (what NCCL calls LL): every float travels as an aligned
// 8-byte word {value, epoch}. A collective on a channel is
//   1. producers STORE their contribution into slot[my_rank] of EVERY peer's arena, one 8-byte
//      store per element (posted writes; nothing is loaded across NVLink, no fences, no flags),
//   2. consumers poll each word of their OWN arena until its tag equals the epoch, then add the
//      W slots in RANK ORDER, so every rank computes the same bits.
// An aligned 8-byte store is single-copy atomic, so a word whose tag matches carries its value;
// no memory fence is needed on either side and the latency is one NVLink hop.
// Arenas are double buffered by epoch parity: a rank can only start pushing for epoch e+2 after
// it consumed e+1, which needs every peer's e+1 data, which a peer sends only after it finished
// consuming e. Epochs start at 1 and arenas at zero, so a stale word never matches.
// No wait is unbounded: when the limit expires the kernel records a status word that the host
// can read through mapped pinned memory, stops waiting and lets the launch drain.
#pragma once
#include "psgd_common.cuh"

#define PSGD_MAX_WORLD 8

typedef struct {
  int32_t world, rank;
  uint2* slots[PSGD_MAX_WORLD];   // peer p's arena: [2][world][cap] words {value bits, epoch}
  int32_t* epoch;                 // local: last completed epoch of this channel
  int32_t* arrive;                // local: [4] arrival counters of consumer launches
  int32_t* abort_flag;            // local device word: non-zero once a wait on this channel ran out
  int32_t* status;                // mapped pinned host word: 0 ok, else PsgdStatus (written once, on a
                                  // timeout; never read by kernels - a read is a PCIe round trip)
  int64_t cap;                    // words per slot
  uint64_t timeout_ns;
} PsgdCommDev;

__device__ __forceinline__ uint2* psgd_comm_slot(const PsgdCommDev& c, int peer, int epoch, int src_rank) {
  return c.slots[peer] + ((int64_t)(epoch & 1) * c.world + src_rank) * c.cap;
}

__device__ __forceinline__ void psgd_comm_store(uint2* p, float v, int epoch) {
  asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"((uint32_t)epoch) : "memory");
}

__device__ __forceinline__ uint2 psgd_comm_peek(const uint2* p) {
  uint2 w;
  asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
  return w;
}

// Value of a word of the own arena once its tag shows `epoch`. `ok` turns false (and stays false)
// when the wait was abandoned: limit hit now, or already hit by an earlier wait of this launch.
__device__ __forceinline__ float psgd_comm_load(const PsgdCommDev& c, const uint2* p, int epoch, bool& ok) {
  uint2 w = psgd_comm_peek(p);
  if ((int)w.y == epoch) return __uint_as_float(w.x);
  if (!ok) return 0.f;
  const uint64_t t0 = psgd_globaltimer_ns();
  int spins = 0;
  while (true) {
    w = psgd_comm_peek(p);
    if ((int)w.y == epoch) return __uint_as_float(w.x);
    if ((++spins & 15) == 0) __nanosleep(32);   // keep thousands of pollers from saturating L2
    if ((spins & 255) == 0) {
      if (*((volatile int*)c.abort_flag) != 0) { ok = false; return 0.f; }
      if (psgd_globaltimer_ns() - t0 > c.timeout_ns) {
        *((volatile int*)c.abort_flag) = 1;
        *((volatile int*)c.status) = PSGD_TIMEOUT_PEER_BARRIER;
        __threadfence_system();
        ok = false;
        return 0.f;
      }
    }
  }
}

// Sum over ranks, in rank order, of element i of this epoch's slots of the own arena.
__device__ __forceinline__ float psgd_comm_reduce(const PsgdCommDev& c, int epoch, int64_t i, bool& ok) {
  float s = 0.f;
  for (int r = 0; r < c.world; ++r) s += psgd_comm_load(c, psgd_comm_slot(c, c.rank, epoch, r) + i, epoch, ok);
  return s;
}

// Sum over ranks, in rank order, of N elements (indices idx[j], j < n <= N; idx[j] < 0 skips) of
// this epoch's slots of the own arena. All N peeks of one rank's slot are issued before any tag
// is looked at, so a thread with several elements pays one load latency per rank, not per word.
template <int N>
__device__ __forceinline__ void psgd_comm_reduce_batch(const PsgdCommDev& c, int epoch, const int64_t* idx, int n,
                                                       float* out, bool& ok) {
#pragma unroll
  for (int j = 0; j < N; ++j) out[j] = 0.f;
  for (int r = 0; r < c.world; ++r) {
    const uint2* slot = psgd_comm_slot(c, c.rank, epoch, r);
    uint2 w[N];
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (j < n && idx[j] >= 0) w[j] = psgd_comm_peek(slot + idx[j]);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      if (j < n && idx[j] >= 0) {
        const float v = ((int)w[j].y == epoch) ? __uint_as_float(w[j].x) : psgd_comm_load(c, slot + idx[j], epoch, ok);
        out[j] += v;
      }
    }
  }
}

// Consumer launches close the epoch: the CTA that arrives last advances the channel.
__device__ __forceinline__ void psgd_comm_close_epoch(const PsgdCommDev& c, int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (psgd_atom_add_acqrel_gpu(c.arrive + 1, 1) == (int)gridDim.x - 1) {
      c.arrive[1] = 0;
      *c.epoch = epoch;
    }
  }
}

// ---- bulk protocol (large messages) ---------------------------------------------------------
// The flag-in-data words double the bytes on the wire. Messages of megabytes travel as plain
// floats instead, in chunks; the CTA that wrote a chunk fences once (thread 0, after a CTA
// barrier) and then publishes the epoch in one flag per chunk. With a thousand CTAs in flight the
// fence latency (a round trip over the link) overlaps other CTAs' stores. Flags only grow, so
// they are never reset; chunk data is read with L1-bypassing loads after the acquire.
__device__ __forceinline__ void psgd_flag_publish(int32_t* flag, int epoch) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
}

__device__ __forceinline__ int psgd_flag_peek(const int32_t* flag) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}

// Bounded wait until *flag == epoch. False when the wait was abandoned (now or earlier).
__device__ __forceinline__ bool psgd_flag_wait(const PsgdCommDev& c, const int32_t* flag, int epoch) {
  if (psgd_flag_peek(flag) == epoch) return true;
  const uint64_t t0 = psgd_globaltimer_ns();
  int spins = 0;
  while (true) {
    if (psgd_flag_peek(flag) == epoch) return true;
    __nanosleep(64);
    if ((++spins & 63) == 0) {
      if (*((volatile int*)c.abort_flag) != 0) return false;
      if (psgd_globaltimer_ns() - t0 > c.timeout_ns) {
        *((volatile int*)c.abort_flag) = 1;
        *((volatile int*)c.status) = PSGD_TIMEOUT_PEER_BARRIER;
        __threadfence_system();
        return false;
      }
    }
  }
}

constexpr int PSGD_BULK_CHUNK = 4096;  // floats per chunk; slices are padded to whole chunks

// Where the parts of a bulk all-reduce live inside every rank's arena (byte offsets are multiples
// of 256): the flat data itself, the landing area of the reduce-scatter, and the two flag tables.
typedef struct {
  const PsgdCommDev* comm;
  long long n_pad;      // floats, a multiple of world * PSGD_BULK_CHUNK
  int cps;              // chunks per slice = n_pad / world / PSGD_BULK_CHUNK
} PsgdBulk;

__device__ __forceinline__ float* psgd_bulk_data(const PsgdCommDev& c, int peer) { return (float*)c.slots[peer]; }
__device__ __forceinline__ float* psgd_bulk_stage(const PsgdCommDev& c, const PsgdBulk& b, int peer) {
  return (float*)c.slots[peer] + b.n_pad;
}
// which = 0: "rank src pushed chunk q of my slice"; 1: "owner src wrote chunk q of its slice here"
__device__ __forceinline__ int32_t* psgd_bulk_flag(const PsgdCommDev& c, const PsgdBulk& b, int peer, int which, int src, int q) {
  return (int32_t*)((float*)c.slots[peer] + 2 * b.n_pad) + ((long long)which * c.world + src) * b.cps + q;
}

