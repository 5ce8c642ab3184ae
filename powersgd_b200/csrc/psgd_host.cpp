// Host-side odds and ends of the native library: last-error string, version, device query.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#define PSGD_API extern "C" __attribute__((visibility("default")))

static thread_local char g_last_error[1024] = "";

void psgd_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

PSGD_API const char* psgd_last_error() { return g_last_error; }

PSGD_API int psgd_version() { return 100; }

// Fills sm_count / major / minor of the CURRENT device. Returns a CUDA error code.
PSGD_API int psgd_device_info(int* sm_count, int* cc_major, int* cc_minor, int* max_smem_optin) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { psgd_set_error("cudaGetDevice: %s", cudaGetErrorString(e)); return (int)e; }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) { psgd_set_error("cudaGetDeviceProperties: %s", cudaGetErrorString(e)); return (int)e; }
  *sm_count = prop.multiProcessorCount;
  *cc_major = prop.major;
  *cc_minor = prop.minor;
  *max_smem_optin = (int)prop.sharedMemPerBlockOptin;
  return 0;
}

#ifdef PSGD_BOUNDS_CHECK
extern "C" int psgd_bounds_read_products(int* out, int reset);
extern "C" int psgd_bounds_read_finalize(int* out, int reset);
extern "C" int psgd_bounds_read_orth(int* out, int reset);
// Debug build only. out[0..23]: the status blocks of the product, decompression / flat and
// orthonormalisation translation units (8 ints each: violations, kernel id of the first, what,
// value lo / hi, limit lo / hi, unused). Returns the total number of violations, or -1 on error.
PSGD_API int psgd_bounds_status(int* out, int reset) {
  if (psgd_bounds_read_products(out, reset) != 0 || psgd_bounds_read_finalize(out + 8, reset) != 0 ||
      psgd_bounds_read_orth(out + 16, reset) != 0) {
    psgd_set_error("psgd_bounds_status: reading a status block failed");
    return -1;
  }
  return out[0] + out[8] + out[16];
}
#endif
