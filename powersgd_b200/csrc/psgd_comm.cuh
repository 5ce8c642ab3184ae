// In-kernel collectives over NVLink peer memory: device-side context and primitives.
//
// Every rank owns one "slot arena" and one flag pad, allocated with cudaMalloc and mapped into
// every peer through CUDA IPC. A collective on a channel is:
//   1. producers STORE their contribution into slot[my_rank] of EVERY peer's arena (pushes are
//      posted writes; nothing is ever loaded across NVLink on the critical path),
//   2. the last producer CTA of the launch publishes `epoch` into flag[my_rank] of every peer
//      (st.release.sys after a system-scope fence),
//   3. consumers spin (ld.acquire.sys, bounded by %globaltimer) until all W flags show the
//      epoch, then add the W slots in RANK ORDER, so every rank computes the same bits.
// Arenas are double buffered by epoch parity: a rank can only start pushing for epoch e+2
// after it saw every peer's flag for e+1, which a peer raises after it finished consuming e.
// No wait is unbounded: when the limit expires the kernel records a status word that the host
// can read through mapped pinned memory, stops waiting and lets the launch drain.
#pragma once
#include "psgd_common.cuh"

#define PSGD_MAX_WORLD 8

typedef struct {
  int32_t world, rank;
  float* slots[PSGD_MAX_WORLD];   // peer p's arena: [2][world][cap] floats
  int32_t* flags[PSGD_MAX_WORLD]; // peer p's flag pad: [world] ints, flag[r] = last epoch published by r
  int32_t* epoch;                 // local: last completed epoch of this channel
  int32_t* arrive;                // local: [4] arrival counters (producer launch, consumer launch, spare)
  int32_t* status;                // mapped pinned host word: 0 ok, else PsgdStatus
  int64_t cap;                    // floats per slot
  uint64_t timeout_ns;
} PsgdCommDev;

__device__ __forceinline__ float* psgd_comm_slot(const PsgdCommDev& c, int peer, int epoch, int src_rank) {
  return c.slots[peer] + ((int64_t)(epoch & 1) * c.world + src_rank) * c.cap;
}

// Called by ONE thread of the CTA that arrived last: publish `epoch` to every peer.
__device__ __forceinline__ void psgd_comm_publish(const PsgdCommDev& c, int epoch) {
  __threadfence_system();
  for (int p = 0; p < c.world; ++p) psgd_st_release_sys(c.flags[p] + c.rank, epoch);
}

// Every thread of the CTA may call this; threads t < world poll one flag each. Returns false
// when the wait was abandoned (limit hit now or by an earlier wait).
__device__ __forceinline__ bool psgd_comm_wait_all(const PsgdCommDev& c, int epoch) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < c.world) {
    const int* f = c.flags[c.rank] + threadIdx.x;
    if (psgd_ld_acquire_sys(f) - epoch < 0) {
      const uint64_t t0 = psgd_globaltimer_ns();
      bool ok = true;
      while (psgd_ld_acquire_sys(f) - epoch < 0) {
        if (*((volatile int*)c.status) != 0) { ok = false; break; }
        if (psgd_globaltimer_ns() - t0 > c.timeout_ns) {
          *((volatile int*)c.status) = PSGD_TIMEOUT_PEER_BARRIER;
          __threadfence_system();
          ok = false;
          break;
        }
        __nanosleep(64);
      }
      if (!ok) s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}
