// Debug build of the native library: `python -m powersgd_b200.csrc.build --debug` compiles every
// translation unit with -DPSGD_BOUNDS_CHECK into libpsgd_b200_debug.so. In that build the kernels
// validate what the host planner handed them - tile extents against matrix extents, scratch slots
// against scratch capacities, pointer alignment against the access width a tile claims, chunk
// ranges against factor lengths - and guard their global accesses. A violation never traps and never
// touches memory: the first one is recorded (kernel id, what failed, the offending value) in a
// status block that the host reads with psgd_bounds_status(), and the access is skipped.
// (compute-sanitizer is not available where this library is developed; this is its stand-in.)
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// what failed
enum PsgdBoundsWhat : int {
  PSGD_BC_TILE_ROWS = 1,      // tile row range outside the matrix
  PSGD_BC_TILE_COLS = 2,      // tile column range outside the matrix
  PSGD_BC_ALIGNMENT = 3,      // pointer or pitch not aligned to the tile's access width
  PSGD_BC_SCRATCH_SLOT = 4,   // partial-sum slot outside the scratch arena
  PSGD_BC_TICKET = 5,         // arrival counter outside its table
  PSGD_BC_FACTOR_INDEX = 6,   // factor element outside the factor buffer
  PSGD_BC_RANK = 7,           // matrix rank above the compiled template rank
  PSGD_BC_SMEM = 8,           // shared-memory panel index outside the allocation
  PSGD_BC_ELEMENT = 9,        // element index outside a flat item
  PSGD_BC_CHUNK = 10,         // orthonormalisation chunk outside its unit
};

#ifdef PSGD_BOUNDS_CHECK
// One block per translation unit (static linkage): [0] number of violations, [1] kernel id of the
// first, [2] what, [3] value low, [4] value high, [5] limit low, [6] limit high.
static __device__ int g_psgd_bounds[8];

__device__ __forceinline__ void psgd_bounds_fail(int kernel_id, int what, long long value, long long limit) {
  if (atomicAdd(&g_psgd_bounds[0], 1) == 0) {
    g_psgd_bounds[1] = kernel_id;
    g_psgd_bounds[2] = what;
    g_psgd_bounds[3] = (int)(value & 0xffffffffll);
    g_psgd_bounds[4] = (int)(value >> 32);
    g_psgd_bounds[5] = (int)(limit & 0xffffffffll);
    g_psgd_bounds[6] = (int)(limit >> 32);
  }
}
// true when `cond` holds; records the violation and returns false otherwise
#define PSGD_BC(cond, kernel_id, what, value, limit) ((cond) ? true : (psgd_bounds_fail((kernel_id), (what), (long long)(value), (long long)(limit)), false))
#define PSGD_BC_ENABLED 1

// Host side: every translation unit exports its block through this helper.
#define PSGD_BOUNDS_EXPORT(name)                                                              \
  extern "C" __attribute__((visibility("default"))) int name(int* out, int reset) {           \
    cudaError_t e = cudaMemcpyFromSymbol(out, g_psgd_bounds, sizeof(int) * 8);                \
    if (e != cudaSuccess) return (int)e;                                                      \
    if (reset) {                                                                              \
      int zeros[8] = {0};                                                                     \
      e = cudaMemcpyToSymbol(g_psgd_bounds, zeros, sizeof(zeros));                            \
    }                                                                                         \
    return (int)e;                                                                            \
  }
#else
#define PSGD_BC(cond, kernel_id, what, value, limit) (true)
#define PSGD_BC_ENABLED 0
#define PSGD_BOUNDS_EXPORT(name)
#endif
