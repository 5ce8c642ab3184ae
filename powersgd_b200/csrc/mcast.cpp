// NVLink multicast memory: the part of the symmetric-memory runtime behind the in-switch
// all-reduce (nvls.cu).
//
// One multicast object spans the W GPUs of the job. Rank 0 creates it and exports a POSIX file
// descriptor, which the Python layer hands to the other ranks over a Unix-domain socket
// (SCM_RIGHTS); every rank adds its device, allocates physical memory with the virtual-memory
// API, binds it to the object and maps two address ranges: its own replica (ordinary loads and
// stores, what the pack / unpack kernels use) and the multicast range (what `multimem.*`
// instructions address: one address, all replicas). The reference reaches the same hardware
// through NCCL's NVLS transport (powersgd/powersgd.py:22-31 -> torch.distributed.all_reduce).
//
// The driver entry points are looked up at run time, so the library loads on machines without a
// driver. Every function returns 0 or an error code with a message for psgd_last_error().
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <unistd.h>

#include "psgd_common.cuh"

namespace {

struct McApi {
  CUresult (*DeviceGet)(CUdevice*, int);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*GetErrorString)(CUresult, const char**);
  bool ok;
};

bool mc_lookup(const char* name, void** fn) {
  cudaDriverEntryPointQueryResult q;
  *fn = nullptr;
  return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn != nullptr;
}

const McApi* mc_api() {
  static McApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    bool ok = true;
    ok &= mc_lookup("cuDeviceGet", (void**)&api.DeviceGet);
    ok &= mc_lookup("cuDeviceGetAttribute", (void**)&api.DeviceGetAttribute);
    ok &= mc_lookup("cuMulticastCreate", (void**)&api.MulticastCreate);
    ok &= mc_lookup("cuMulticastGetGranularity", (void**)&api.MulticastGetGranularity);
    ok &= mc_lookup("cuMulticastAddDevice", (void**)&api.MulticastAddDevice);
    ok &= mc_lookup("cuMulticastBindMem", (void**)&api.MulticastBindMem);
    ok &= mc_lookup("cuMulticastUnbind", (void**)&api.MulticastUnbind);
    ok &= mc_lookup("cuMemCreate", (void**)&api.MemCreate);
    ok &= mc_lookup("cuMemRelease", (void**)&api.MemRelease);
    ok &= mc_lookup("cuMemGetAllocationGranularity", (void**)&api.MemGetAllocationGranularity);
    ok &= mc_lookup("cuMemAddressReserve", (void**)&api.MemAddressReserve);
    ok &= mc_lookup("cuMemAddressFree", (void**)&api.MemAddressFree);
    ok &= mc_lookup("cuMemMap", (void**)&api.MemMap);
    ok &= mc_lookup("cuMemUnmap", (void**)&api.MemUnmap);
    ok &= mc_lookup("cuMemSetAccess", (void**)&api.MemSetAccess);
    ok &= mc_lookup("cuMemExportToShareableHandle", (void**)&api.MemExportToShareableHandle);
    ok &= mc_lookup("cuMemImportFromShareableHandle", (void**)&api.MemImportFromShareableHandle);
    ok &= mc_lookup("cuGetErrorString", (void**)&api.GetErrorString);
    api.ok = ok;
  }
  return &api;
}

int mc_fail(const McApi* api, const char* what, CUresult r) {
  const char* msg = nullptr;
  if (api->GetErrorString) api->GetErrorString(r, &msg);
  psgd_set_error("%s -> %s (%d)", what, msg ? msg : "unknown driver error", (int)r);
  return (int)r == 0 ? -1 : (int)r;
}

#define PSGD_CU_OK(api, expr)                              \
  do {                                                     \
    CUresult _r = (expr);                                  \
    if (_r != CUDA_SUCCESS) return mc_fail(api, #expr, _r); \
  } while (0)

CUmulticastObjectProp mc_prop(int world, size_t bytes) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = (unsigned)world;
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

CUmemAllocationProp mem_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

}  // namespace

// What one rank holds of a multicast buffer.
struct PsgdMcBuffer {
  unsigned long long mc_handle;   // the multicast object (imported or created)
  unsigned long long mem_handle;  // this rank's physical memory
  unsigned long long local_ptr;   // this rank's replica
  unsigned long long mc_ptr;      // the multicast range
  unsigned long long bytes;       // mapped size (rounded up)
  int device;
  int bound;
};

PSGD_API int psgd_mc_buffer_bytes() { return (int)sizeof(PsgdMcBuffer); }

// 1 when the current device and driver offer NVLink multicast, 0 when not, < 0 on error.
PSGD_API int psgd_mc_supported() {
  const McApi* api = mc_api();
  if (!api->ok) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaFree(0) != cudaSuccess) return 0;  // a context for the driver calls below
  CUdevice cu;
  if (api->DeviceGet(&cu, dev) != CUDA_SUCCESS) return 0;
  int yes = 0;
  if (api->DeviceGetAttribute(&yes, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu) != CUDA_SUCCESS) return 0;
  return yes ? 1 : 0;
}

// Size that a buffer of `bytes` must be rounded up to (a multiple of the multicast and of the
// allocation granularity).
PSGD_API int psgd_mc_round_up(int world, unsigned long long bytes, unsigned long long* out) {
  const McApi* api = mc_api();
  if (!api->ok) { psgd_set_error("psgd_mc_round_up: driver without the multicast API"); return -1; }
  int dev = 0;
  PSGD_CUDA_OK(cudaGetDevice(&dev));
  PSGD_CUDA_OK(cudaFree(0));
  size_t g_mc = 0, g_mem = 0;
  CUmulticastObjectProp mp = mc_prop(world, (size_t)bytes);
  PSGD_CU_OK(api, api->MulticastGetGranularity(&g_mc, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  CUmemAllocationProp ap = mem_prop(dev);
  PSGD_CU_OK(api, api->MemGetAllocationGranularity(&g_mem, &ap, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
  size_t g = g_mc > g_mem ? g_mc : g_mem;
  if (g == 0 || g % g_mem != 0 || g % g_mc != 0) g = g_mc * g_mem;  // not multiples of one another: take a common one
  *out = ((bytes + g - 1) / g) * g;
  return 0;
}

// Rank 0: creates the object for `world` devices and `bytes` (already rounded) and exports a file
// descriptor for the peers. The caller closes the descriptor once every peer has received it.
PSGD_API int psgd_mc_create(int world, unsigned long long bytes, PsgdMcBuffer* buf, int* fd_out) {
  const McApi* api = mc_api();
  if (!api->ok) { psgd_set_error("psgd_mc_create: driver without the multicast API"); return -1; }
  memset(buf, 0, sizeof(*buf));
  PSGD_CUDA_OK(cudaGetDevice(&buf->device));
  PSGD_CUDA_OK(cudaFree(0));
  CUmulticastObjectProp mp = mc_prop(world, (size_t)bytes);
  CUmemGenericAllocationHandle h;
  PSGD_CU_OK(api, api->MulticastCreate(&h, &mp));
  int fd = -1;
  CUresult r = api->MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    api->MemRelease(h);
    return mc_fail(api, "cuMemExportToShareableHandle(multicast object)", r);
  }
  buf->mc_handle = (unsigned long long)h;
  buf->bytes = bytes;
  *fd_out = fd;
  return 0;
}

// Other ranks: import the object from the descriptor received from rank 0 (closed here).
PSGD_API int psgd_mc_import(int fd, unsigned long long bytes, PsgdMcBuffer* buf) {
  const McApi* api = mc_api();
  if (!api->ok) { psgd_set_error("psgd_mc_import: driver without the multicast API"); return -1; }
  memset(buf, 0, sizeof(*buf));
  PSGD_CUDA_OK(cudaGetDevice(&buf->device));
  PSGD_CUDA_OK(cudaFree(0));
  CUmemGenericAllocationHandle h;
  CUresult r = api->MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  if (r != CUDA_SUCCESS) return mc_fail(api, "cuMemImportFromShareableHandle(multicast object)", r);
  buf->mc_handle = (unsigned long long)h;
  buf->bytes = bytes;
  return 0;
}

// Every rank, after the object exists everywhere: register this device with the object. All ranks
// must have done this before any rank binds memory (the caller puts a barrier between the two).
PSGD_API int psgd_mc_add_device(PsgdMcBuffer* buf) {
  const McApi* api = mc_api();
  CUdevice cu;
  PSGD_CU_OK(api, api->DeviceGet(&cu, buf->device));
  PSGD_CU_OK(api, api->MulticastAddDevice((CUmemGenericAllocationHandle)buf->mc_handle, cu));
  return 0;
}

// Every rank: allocate this rank's replica, bind it at offset 0 of the object, map the replica and
// the multicast range, zero the replica.
PSGD_API int psgd_mc_bind(PsgdMcBuffer* buf) {
  const McApi* api = mc_api();
  const size_t bytes = (size_t)buf->bytes;
  CUmemAllocationProp ap = mem_prop(buf->device);
  CUmemGenericAllocationHandle mem;
  PSGD_CU_OK(api, api->MemCreate(&mem, bytes, &ap, 0));
  buf->mem_handle = (unsigned long long)mem;
  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = buf->device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUdeviceptr local = 0, mc = 0;
  PSGD_CU_OK(api, api->MemAddressReserve(&local, bytes, 0, 0, 0));
  buf->local_ptr = (unsigned long long)local;
  PSGD_CU_OK(api, api->MemMap(local, bytes, 0, mem, 0));
  PSGD_CU_OK(api, api->MemSetAccess(local, bytes, &access, 1));
  PSGD_CU_OK(api, api->MulticastBindMem((CUmemGenericAllocationHandle)buf->mc_handle, 0, mem, 0, bytes, 0));
  buf->bound = 1;
  PSGD_CU_OK(api, api->MemAddressReserve(&mc, bytes, 0, 0, 0));
  buf->mc_ptr = (unsigned long long)mc;
  PSGD_CU_OK(api, api->MemMap(mc, bytes, 0, (CUmemGenericAllocationHandle)buf->mc_handle, 0));
  PSGD_CU_OK(api, api->MemSetAccess(mc, bytes, &access, 1));
  PSGD_CUDA_OK(cudaMemset((void*)(uintptr_t)local, 0, bytes));
  PSGD_CUDA_OK(cudaDeviceSynchronize());
  return 0;
}

// Every rank, with no kernel in flight anywhere that addresses the buffer: unmap, unbind, release.
// Tolerates a buffer that was only partly set up.
PSGD_API int psgd_mc_release(PsgdMcBuffer* buf) {
  const McApi* api = mc_api();
  if (!api->ok) return 0;
  const size_t bytes = (size_t)buf->bytes;
  int rc = 0;
  if (buf->mc_ptr) {
    if (api->MemUnmap((CUdeviceptr)buf->mc_ptr, bytes) != CUDA_SUCCESS) rc = -1;
    api->MemAddressFree((CUdeviceptr)buf->mc_ptr, bytes);
    buf->mc_ptr = 0;
  }
  if (buf->bound) {
    CUdevice cu;
    if (api->DeviceGet(&cu, buf->device) == CUDA_SUCCESS)
      api->MulticastUnbind((CUmemGenericAllocationHandle)buf->mc_handle, cu, 0, bytes);
    buf->bound = 0;
  }
  if (buf->local_ptr) {
    if (api->MemUnmap((CUdeviceptr)buf->local_ptr, bytes) != CUDA_SUCCESS) rc = -1;
    api->MemAddressFree((CUdeviceptr)buf->local_ptr, bytes);
    buf->local_ptr = 0;
  }
  if (buf->mem_handle) {
    api->MemRelease((CUmemGenericAllocationHandle)buf->mem_handle);
    buf->mem_handle = 0;
  }
  if (buf->mc_handle) {
    api->MemRelease((CUmemGenericAllocationHandle)buf->mc_handle);
    buf->mc_handle = 0;
  }
  if (rc != 0) psgd_set_error("psgd_mc_release: unmapping failed");
  return rc;
}
