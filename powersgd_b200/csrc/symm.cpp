// Symmetric-memory runtime: allocation, CUDA-IPC export / import, mapped status words and the
// device-side channel descriptors used by the in-kernel collectives (psgd_comm.cuh).
//
// The Python layer exchanges the 64-byte IPC handles over the existing torch.distributed
// process group (one all-gather at construction); after that no library collective is on the
// data path. One process per GPU; all ranks live on one NVSwitch domain.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "psgd_comm.cuh"

PSGD_API int psgd_symm_alloc(size_t bytes, void** out) {
  PSGD_CUDA_OK(cudaMalloc(out, bytes));
  PSGD_CUDA_OK(cudaMemset(*out, 0, bytes));
  PSGD_CUDA_OK(cudaDeviceSynchronize());
  return 0;
}

PSGD_API int psgd_symm_free(void* ptr) {
  PSGD_CUDA_OK(cudaFree(ptr));
  return 0;
}

PSGD_API int psgd_symm_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

PSGD_API int psgd_symm_export(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  PSGD_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

PSGD_API int psgd_symm_import(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  PSGD_CUDA_OK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

PSGD_API int psgd_symm_unmap(void* ptr) {
  PSGD_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return 0;
}

// A status word in pinned host memory that kernels write through its device mapping.
PSGD_API int psgd_status_alloc(int** host_ptr, int** dev_ptr) {
  PSGD_CUDA_OK(cudaHostAlloc((void**)host_ptr, 64, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(*host_ptr, 0, 64);
  PSGD_CUDA_OK(cudaHostGetDevicePointer((void**)dev_ptr, *host_ptr, 0));
  return 0;
}

PSGD_API int psgd_status_free(int* host_ptr) {
  PSGD_CUDA_OK(cudaFreeHost(host_ptr));
  return 0;
}

PSGD_API int psgd_comm_desc_bytes() { return (int)sizeof(PsgdCommDev); }

// Fills a host-side PsgdCommDev (the caller uploads it). `slots` holds `world` arena pointers
// indexed by rank (own allocation at index `rank`); an arena has 2 * world * cap 8-byte words.
PSGD_API int psgd_comm_fill(void* desc_out, int world, int rank, void* const* slots, int* words, int* status_dev,
                            long long cap, double timeout_ms) {
  if (world < 1 || world > PSGD_MAX_WORLD || rank < 0 || rank >= world) {
    psgd_set_error("psgd_comm_fill: world %d / rank %d out of range (max %d ranks)", world, rank, PSGD_MAX_WORLD);
    return -1;
  }
  PsgdCommDev d;
  memset(&d, 0, sizeof(d));
  d.world = world;
  d.rank = rank;
  for (int p = 0; p < world; ++p) {
    d.slots[p] = (uint2*)slots[p];
  }
  d.epoch = words;           // 16 zeroed device ints: [0] epoch, [4..7] arrival counters, [8] abort flag
  d.arrive = words + 4;
  d.abort_flag = words + 8;
  d.status = status_dev;
  d.cap = cap;
  d.timeout_ns = (uint64_t)(timeout_ms * 1e6);
  memcpy(desc_out, &d, sizeof(d));
  return 0;
}
