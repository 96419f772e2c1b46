// Shared helpers for the sm_100a kernels: element types, conversions, reductions, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define KF_API extern "C" __attribute__((visibility("default")))

// element type codes shared with the Python side
enum KfDtype { KF_F32 = 0, KF_BF16 = 1 };

// error codes returned by every entry point (0 = launched)
enum KfStatus {
  KF_OK = 0,
  KF_ERR_DTYPE = 1,        // combination of element types this kernel has no instance for
  KF_ERR_SIZE = 2,         // a size the kernel refuses (documented per entry point)
  KF_ERR_LAUNCH = 3,       // the CUDA runtime refused the launch; see kf_last_cuda_error
  KF_ERR_ALIGN = 4,        // a pointer or stride breaks an alignment rule
  KF_ERR_SETUP = 5,        // one-time set-up failed (driver entry point, attribute)
};

extern "C" int kf_record_cuda_error(cudaError_t e);
extern "C" void kf_record_message(const char* msg);

#define KF_CHECK_LAUNCH()                                   \
  do {                                                      \
    cudaError_t _e = cudaGetLastError();                    \
    if (_e != cudaSuccess) { kf_record_cuda_error(_e); return KF_ERR_LAUNCH; } \
  } while (0)

// Programmatic dependent launch.  Every kernel of this library may be launched before its predecessor in the
// stream has finished (kf_launch below sets the attribute); a kernel therefore calls kf_pdl_wait() before it
// touches global memory that the predecessor may write or read, and kf_pdl_trigger() as early as it can so that the
// next kernel's blocks can take free resources and run their own prologue (the tensor-core product prefetches
// weights there).  Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void kf_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void kf_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// A kernel that reads global memory before kf_pdl_wait() passes every pointer to what earlier kernels of the stream
// wrote through this, after the wait.  Loads through a const __restrict__ parameter count as invariant for the whole
// kernel, and the compiler may then schedule them together with the loads that stand before the wait (it did, in a
// norm kernel, and read rows that the product before it had not finished).  The empty statement makes the pointer's
// value depend on something that is ordered after the wait, so no load through it can move above it.
template <typename T>
__device__ __forceinline__ T* kf_produced(T* p) {
  asm volatile("" : "+l"(p)::"memory");
  return p;
}

extern "C" int kf_pdl_enabled();
extern "C" int kf_sm_count();           // SMs of the current device

// Launch with the programmatic-dependent-launch attribute when it is switched on (kf_set_pdl).
template <typename... KArgs, typename... Args>
static inline cudaError_t kf_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kf_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float kf_load(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float kf_load(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void kf_store(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void kf_store(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float kf_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float kf_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float kf_block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = kf_warp_sum(v);
  __syncthreads();                       // red may still be read from an earlier call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = kf_warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// activations of the gated feed-forward
enum KfAct { KF_ACT_GELU_TANH = 0, KF_ACT_GELU_ERF = 1, KF_ACT_SILU = 2 };

__device__ __forceinline__ float kf_act(float x, int act) {
  if (act == KF_ACT_GELU_TANH) {
    const float c = 0.7978845608028654f;                  // sqrt(2/pi)
    return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
  } else if (act == KF_ACT_GELU_ERF) {
    return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  }
  return x / (1.f + expf(-x));
}

__device__ __forceinline__ float kf_softcap(float x, float cap) { return cap > 0.f ? cap * tanhf(x / cap) : x; }

static inline int kf_ceil_div(long a, long b) { return (int)((a + b - 1) / b); }
