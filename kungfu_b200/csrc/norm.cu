// Root-mean-square norms over the 32-bit residual stream.
//   rmsnorm:      out[r, :] = x[row(r), :] * rsqrt(mean(x^2) + eps) * g,  g = w or 1 + w
//   add_rmsnorm:  x += rmsnorm(a; w1);  optionally out2 = rmsnorm(x; w2)  (post-norm + residual + next pre-norm)
// Reference: crates/kf-backend-cuda/src/kernels/norm.cu:4-27.  Sums and the scale are 32-bit.
#include "common.cuh"

template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, float eps, int plus_one,
                               TO* __restrict__ out, const int* __restrict__ rows, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = kf_load(w, i) + (plus_one ? 1.f : 0.f);
    kf_store(o, i, xr[i] * inv * g);
  }
}

// Single-pass variants: the row (up to NPT * blockDim elements) stays in registers between the sum of squares and
// the scaling, so every input is read once.
// One block per row, the row in registers.  The gains do not depend on earlier kernels and are requested before the grid
// dependency is waited for; `x` and `rows` come from earlier kernels and go through kf_produced() after the wait.
template <typename TW, typename TO, int NPT>
__global__ void rmsnorm_reg_kernel(const float* x, const TW* __restrict__ w, float eps, int plus_one,
                                   TO* __restrict__ out, const int* rows, int H) {
  kf_pdl_trigger();
  __shared__ float red[33];
  const int r = blockIdx.x;
  float v[NPT], g[NPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    g[k] = i < H ? kf_load(w, i) + (plus_one ? 1.f : 0.f) : 0.f;
  }
  kf_pdl_wait();
  x = kf_produced(x), rows = kf_produced(rows);
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = i < H ? xr[i] : 0.f;
  }
#pragma unroll
  for (int k = 0; k < NPT; ++k) ss += v[k] * v[k];
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < H) kf_store(o, i, v[k] * inv * g[k]);
  }
}

template <typename TW1, typename TW2, typename TO, int NPT, int MAXT>
__global__ void __launch_bounds__(MAXT) add_rmsnorm_reg_kernel(const float* a, const TW1* __restrict__ w1, float eps1, int plus1,
                                       float* x, const TW2* __restrict__ w2, float eps2, int plus2,
                                       TO* __restrict__ out2, int H) {
  kf_pdl_trigger();
  __shared__ float red[33];
  const int r = blockIdx.x;
  float v[NPT], xv[NPT], g1[NPT], g2[NPT];
  float ss = 0.f;
  // The gains do not depend on earlier kernels: they are requested before the grid dependency is waited for (2.56 ->
  // 2.44 ms per decode step at 26 layers); then both rows at once, before the first sum.
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    g1[k] = i < H ? kf_load(w1, i) + (plus1 ? 1.f : 0.f) : 0.f;
    g2[k] = (i < H && out2 != nullptr) ? kf_load(w2, i) + (plus2 ? 1.f : 0.f) : 0.f;
  }
  kf_pdl_wait();
  a = kf_produced(a), x = kf_produced(x);
  const float* ar = a + (size_t)r * H;
  float* xr = x + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = i < H ? ar[i] : 0.f;
    xv[k] = i < H ? xr[i] : 0.f;
  }
#pragma unroll
  for (int k = 0; k < NPT; ++k) ss += v[k] * v[k];
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps1);
  float ss2 = 0.f;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < H) {
      v[k] = xv[k] + v[k] * inv * g1[k];
      xr[i] = v[k];
      ss2 += v[k] * v[k];
    } else {
      v[k] = 0.f;
    }
  }
  if (out2 == nullptr) return;
  ss2 = kf_block_sum(ss2, red);
  const float inv2 = 1.f / sqrtf(ss2 / (float)H + eps2);
  TO* o = out2 + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < H) kf_store(o, i, v[k] * inv2 * g2[k]);
  }
}

// Many rows (prompt portions): one warp per row, the row in registers as float4, no block barrier.
// Needs H % 4 == 0 and H <= 128 * NV4.
template <typename TW>
__device__ __forceinline__ float4 kf_gain4(const TW* w, int i, int plus_one) {
  const float p = plus_one ? 1.f : 0.f;
  return make_float4(kf_load(w, i) + p, kf_load(w, i + 1) + p, kf_load(w, i + 2) + p, kf_load(w, i + 3) + p);
}
__device__ __forceinline__ void kf_store4(float* o, int i, float4 v) { *reinterpret_cast<float4*>(o + i) = v; }
__device__ __forceinline__ void kf_store4(__nv_bfloat16* o, int i, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(o + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename TW1, typename TW2, typename TO, int NV4>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(const float* __restrict__ a, const TW1* __restrict__ w1, float eps1, int plus1,
                        float* __restrict__ x, const TW2* __restrict__ w2, float eps2, int plus2,
                        TO* __restrict__ out2, int T, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= T) return;
  const float* ar = a + (size_t)r * H;
  float* xr = x + (size_t)r * H;
  float4 v[NV4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV4; ++k) {
    const int i = (lane + 32 * k) * 4;
    v[k] = i < H ? *reinterpret_cast<const float4*>(ar + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  ss = kf_warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)H + eps1);
  float ss2 = 0.f;
#pragma unroll
  for (int k = 0; k < NV4; ++k) {
    const int i = (lane + 32 * k) * 4;
    if (i < H) {
      const float4 g = kf_gain4(w1, i, plus1);
      const float4 xo = *reinterpret_cast<const float4*>(xr + i);
      v[k] = make_float4(xo.x + v[k].x * inv * g.x, xo.y + v[k].y * inv * g.y, xo.z + v[k].z * inv * g.z, xo.w + v[k].w * inv * g.w);
      *reinterpret_cast<float4*>(xr + i) = v[k];
      ss2 += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  if (out2 == nullptr) return;
  ss2 = kf_warp_sum(ss2);
  const float inv2 = 1.f / sqrtf(ss2 / (float)H + eps2);
  TO* o = out2 + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < NV4; ++k) {
    const int i = (lane + 32 * k) * 4;
    if (i < H) {
      const float4 g = kf_gain4(w2, i, plus2);
      kf_store4(o, i, make_float4(v[k].x * inv2 * g.x, v[k].y * inv2 * g.y, v[k].z * inv2 * g.z, v[k].w * inv2 * g.w));
    }
  }
}

template <typename TW>
static int launch_rmsnorm(const float* x, const TW* w, float eps, int plus_one, void* out, int out_dtype,
                          const int* rows, int n, int H, cudaStream_t stream) {
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (H <= 16 * threads) {
    const int npt = kf_ceil_div(H, threads);
#define KF_GO(TO, NPT) kf_launch(rmsnorm_reg_kernel<TW, TO, NPT>, dim3(n), dim3(threads), 0, stream, x, w, eps, plus_one, (TO*)out, rows, H)
#define KF_PICK(TO)                                                            \
    if (npt <= 2) KF_GO(TO, 2); else if (npt <= 4) KF_GO(TO, 4); else if (npt <= 8) KF_GO(TO, 8); else KF_GO(TO, 16)
    if (out_dtype == KF_F32) { KF_PICK(float); }
    else if (out_dtype == KF_BF16) { KF_PICK(__nv_bfloat16); }
    else return KF_ERR_DTYPE;
#undef KF_PICK
#undef KF_GO
    KF_CHECK_LAUNCH();
    return KF_OK;
  }
  if (out_dtype == KF_F32)
    kf_launch(rmsnorm_kernel<TW, float>, dim3(n), dim3(threads), 0, stream, x, w, eps, plus_one, (float*)out, rows, H);
  else if (out_dtype == KF_BF16)
    kf_launch(rmsnorm_kernel<TW, __nv_bfloat16>, dim3(n), dim3(threads), 0, stream, x, w, eps, plus_one, (__nv_bfloat16*)out, rows, H);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

KF_API int kf_rmsnorm(const float* x, const void* w, int w_dtype, float eps, int plus_one, void* out, int out_dtype,
                      const int* rows, int n, int H, cudaStream_t stream) {
  if (n <= 0) return KF_OK;
  if (w_dtype == KF_F32) return launch_rmsnorm<float>(x, (const float*)w, eps, plus_one, out, out_dtype, rows, n, H, stream);
  if (w_dtype == KF_BF16) return launch_rmsnorm<__nv_bfloat16>(x, (const __nv_bfloat16*)w, eps, plus_one, out, out_dtype, rows, n, H, stream);
  return KF_ERR_DTYPE;
}

template <typename TW1, typename TW2, typename TO>
__global__ void add_rmsnorm_kernel(const float* __restrict__ a, const TW1* __restrict__ w1, float eps1, int plus1,
                                   float* __restrict__ x, const TW2* __restrict__ w2, float eps2, int plus2,
                                   TO* __restrict__ out2, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* ar = a + (size_t)r * H;
  float* xr = x + (size_t)r * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) { const float v = ar[i]; ss += v * v; }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps1);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = kf_load(w1, i) + (plus1 ? 1.f : 0.f);
    const float v = xr[i] + ar[i] * inv * g;
    xr[i] = v;
    ss2 += v * v;
  }
  if (out2 == nullptr) return;
  ss2 = kf_block_sum(ss2, red);
  const float inv2 = 1.f / sqrtf(ss2 / (float)H + eps2);
  TO* o = out2 + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {     // each thread re-reads only what it wrote
    const float g = kf_load(w2, i) + (plus2 ? 1.f : 0.f);
    kf_store(o, i, xr[i] * inv2 * g);
  }
}

// Many rows, two warps per row: every lane requests all of its part of both rows at once (the branch row and the
// residual row, up to 2 x NV 16-byte loads in flight), so a row costs about three trips to memory instead of one per
// 128 elements; the two warps meet through shared memory for the two sums.  Needs H % 4 == 0 and H <= 256 * NV.
template <typename TW1, typename TW2, typename TO, int NV>
__global__ void __launch_bounds__(256, 2)
add_rmsnorm_split_kernel(const float* __restrict__ a, const TW1* __restrict__ w1, float eps1, int plus1,
                         float* __restrict__ x, const TW2* __restrict__ w2, float eps2, int plus2,
                         TO* __restrict__ out2, int T, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[2][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (warp >> 1), half = warp & 1;
  const bool valid = r < T;
  const float* ar = a + (size_t)(valid ? r : 0) * H;
  float* xr = x + (size_t)(valid ? r : 0) * H;
  float4 v[NV], xo[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (lane + 32 * (half + 2 * k)) * 4;
    const bool in = valid && i < H;
    v[k] = in ? *reinterpret_cast<const float4*>(ar + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    xo[k] = in ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  ss = kf_warp_sum(ss);
  if (lane == 0) red[0][warp] = ss;
  __syncthreads();
  ss = red[0][warp & ~1] + red[0][warp | 1];
  const float inv = 1.f / sqrtf(ss / (float)H + eps1);
  float ss2 = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (lane + 32 * (half + 2 * k)) * 4;
    if (valid && i < H) {
      const float4 g = kf_gain4(w1, i, plus1);
      v[k] = make_float4(xo[k].x + v[k].x * inv * g.x, xo[k].y + v[k].y * inv * g.y, xo[k].z + v[k].z * inv * g.z,
                         xo[k].w + v[k].w * inv * g.w);
      *reinterpret_cast<float4*>(xr + i) = v[k];
      ss2 += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  if (out2 == nullptr) return;                                    // uniform over the block
  ss2 = kf_warp_sum(ss2);
  if (lane == 0) red[1][warp] = ss2;
  __syncthreads();
  ss2 = red[1][warp & ~1] + red[1][warp | 1];
  const float inv2 = 1.f / sqrtf(ss2 / (float)H + eps2);
  TO* o = out2 + (size_t)(valid ? r : 0) * H;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (lane + 32 * (half + 2 * k)) * 4;
    if (valid && i < H) {
      const float4 g = kf_gain4(w2, i, plus2);
      kf_store4(o, i, make_float4(v[k].x * inv2 * g.x, v[k].y * inv2 * g.y, v[k].z * inv2 * g.z, v[k].w * inv2 * g.w));
    }
  }
}

template <typename TW1, typename TW2>
static int launch_add_rmsnorm(const float* a, const TW1* w1, float eps1, int plus1, float* x, const TW2* w2, float eps2,
                              int plus2, void* out2, int out2_dtype, int T, int H, cudaStream_t stream) {
  // four values per element live in registers in the one-block-per-row kernel: at most 8 elements per thread
  const int threads = H > 4096 ? 1024 : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
  const bool aligned = H % 4 == 0 && (((uintptr_t)a | (uintptr_t)x | (uintptr_t)out2) & 15) == 0;
  if (T >= 256 && aligned && H <= 256 * 20 && H >= 256) {         // many rows: two warps per row, all loads at once
    const int nv = kf_ceil_div(H, 256);
#define KF_GO(TO, NV) kf_launch(add_rmsnorm_split_kernel<TW1, TW2, TO, NV>, dim3(kf_ceil_div(T, 4)), dim3(256), 0, stream, a, w1, eps1, plus1, x, w2, eps2, plus2, (TO*)out2, T, H)
#define KF_PICK(TO)                                                                         \
    if (nv <= 4) KF_GO(TO, 4); else if (nv <= 9) KF_GO(TO, 9); else if (nv <= 14) KF_GO(TO, 14); else KF_GO(TO, 20)
    if (out2 == nullptr || out2_dtype == KF_F32) { KF_PICK(float); }
    else if (out2_dtype == KF_BF16) { KF_PICK(__nv_bfloat16); }
    else return KF_ERR_DTYPE;
#undef KF_PICK
#undef KF_GO
    KF_CHECK_LAUNCH();
    return KF_OK;
  }
  if (T >= 256 && aligned && H <= 128 * 40 && H >= 128) {        // many rows: a warp per row
    const int nv4 = kf_ceil_div(H, 128);
#define KF_GO(TO, NV4) kf_launch(add_rmsnorm_warp_kernel<TW1, TW2, TO, NV4>, dim3(kf_ceil_div(T, 8)), dim3(256), 0, stream, a, w1, eps1, plus1, x, w2, eps2, plus2, (TO*)out2, T, H)
#define KF_PICK(TO)                                                                         \
    if (nv4 <= 8) KF_GO(TO, 8); else if (nv4 <= 16) KF_GO(TO, 16); else if (nv4 <= 24) KF_GO(TO, 24); \
    else if (nv4 <= 32) KF_GO(TO, 32); else KF_GO(TO, 40)
    if (out2 == nullptr || out2_dtype == KF_F32) { KF_PICK(float); }
    else if (out2_dtype == KF_BF16) { KF_PICK(__nv_bfloat16); }
    else return KF_ERR_DTYPE;
#undef KF_PICK
#undef KF_GO
    KF_CHECK_LAUNCH();
    return KF_OK;
  }
  if (H <= 8 * threads) {
    const int npt = kf_ceil_div(H, threads);
#define KF_GO(TO, NPT, MAXT) kf_launch(add_rmsnorm_reg_kernel<TW1, TW2, TO, NPT, MAXT>, dim3(T), dim3(threads), 0, stream, a, w1, eps1, plus1, x, w2, eps2, plus2, (TO*)out2, H)
#define KF_PICK(TO)                                                            \
    if (threads > 512) { if (npt <= 5) KF_GO(TO, 5, 1024); else KF_GO(TO, 8, 1024); } else if (npt <= 2) KF_GO(TO, 2, 512); else if (npt <= 4) KF_GO(TO, 4, 512); else KF_GO(TO, 8, 512)
    if (out2 == nullptr || out2_dtype == KF_F32) { KF_PICK(float); }
    else if (out2_dtype == KF_BF16) { KF_PICK(__nv_bfloat16); }
    else return KF_ERR_DTYPE;
#undef KF_PICK
#undef KF_GO
    KF_CHECK_LAUNCH();
    return KF_OK;
  }
  if (out2 == nullptr || out2_dtype == KF_F32)
    kf_launch(add_rmsnorm_kernel<TW1, TW2, float>, dim3(T), dim3(threads), 0, stream, a, w1, eps1, plus1, x, w2, eps2, plus2, (float*)out2, H);
  else if (out2_dtype == KF_BF16)
    kf_launch(add_rmsnorm_kernel<TW1, TW2, __nv_bfloat16>, dim3(T), dim3(threads), 0, stream, a, w1, eps1, plus1, x, w2, eps2, plus2, (__nv_bfloat16*)out2, H);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

KF_API int kf_add_rmsnorm(const float* a, const void* w1, int w1_dtype, float eps1, int plus1, float* x,
                          const void* w2, int w2_dtype, float eps2, int plus2, void* out2, int out2_dtype,
                          int T, int H, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (out2 == nullptr) { w2 = w1; w2_dtype = w1_dtype; }
  if (w1_dtype == KF_F32 && w2_dtype == KF_F32)
    return launch_add_rmsnorm<float, float>(a, (const float*)w1, eps1, plus1, x, (const float*)w2, eps2, plus2, out2, out2_dtype, T, H, stream);
  if (w1_dtype == KF_BF16 && w2_dtype == KF_BF16)
    return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(a, (const __nv_bfloat16*)w1, eps1, plus1, x, (const __nv_bfloat16*)w2, eps2, plus2, out2, out2_dtype, T, H, stream);
  if (w1_dtype == KF_F32 && w2_dtype == KF_BF16)
    return launch_add_rmsnorm<float, __nv_bfloat16>(a, (const float*)w1, eps1, plus1, x, (const __nv_bfloat16*)w2, eps2, plus2, out2, out2_dtype, T, H, stream);
  if (w1_dtype == KF_BF16 && w2_dtype == KF_F32)
    return launch_add_rmsnorm<__nv_bfloat16, float>(a, (const __nv_bfloat16*)w1, eps1, plus1, x, (const float*)w2, eps2, plus2, out2, out2_dtype, T, H, stream);
  return KF_ERR_DTYPE;
}
