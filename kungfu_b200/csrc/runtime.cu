// Library-wide state: the last CUDA error text, version, device checks.
#include "common.cuh"
#include <string.h>
#include <stdio.h>

static char g_last_error[512] = "";

extern "C" int kf_record_cuda_error(cudaError_t e) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return (int)e;
}

extern "C" void kf_record_message(const char* msg) { snprintf(g_last_error, sizeof(g_last_error), "%s", msg); }

KF_API const char* kf_last_cuda_error() { return g_last_error; }

static int g_pdl = 0;
extern "C" int kf_pdl_enabled() { return g_pdl; }
// Switch programmatic dependent launch on (1) or off (0) for every kernel launched afterwards.
KF_API void kf_set_pdl(int on) { g_pdl = on ? 1 : 0; }

KF_API int kf_abi_version() { return 1; }

// Compute capability of the current device as major*10+minor, or -1.
KF_API int kf_device_arch() {
  int dev = 0, major = 0, minor = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
  return major * 10 + minor;
}

// Number of SMs of the current device (asked once per device; 148 on a B200).  The planners size their grids by it.
extern "C" int kf_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
