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
template <typename TW, typename TO, int NPT>
__global__ void rmsnorm_reg_kernel(const float* __restrict__ x, const TW* __restrict__ w, float eps, int plus_one,
                                   TO* __restrict__ out, const int* __restrict__ rows, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
  float v[NPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = i < H ? xr[i] : 0.f;
    ss += v[k] * v[k];
  }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < H) kf_store(o, i, v[k] * inv * (kf_load(w, i) + (plus_one ? 1.f : 0.f)));
  }
}

template <typename TW1, typename TW2, typename TO, int NPT>
__global__ void add_rmsnorm_reg_kernel(const float* __restrict__ a, const TW1* __restrict__ w1, float eps1, int plus1,
                                       float* __restrict__ x, const TW2* __restrict__ w2, float eps2, int plus2,
                                       TO* __restrict__ out2, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* ar = a + (size_t)r * H;
  float* xr = x + (size_t)r * H;
  float v[NPT];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = i < H ? ar[i] : 0.f;
    ss += v[k] * v[k];
  }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps1);
  float ss2 = 0.f;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < H) {
      v[k] = xr[i] + v[k] * inv * (kf_load(w1, i) + (plus1 ? 1.f : 0.f));
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
    if (i < H) kf_store(o, i, v[k] * inv2 * (kf_load(w2, i) + (plus2 ? 1.f : 0.f)));
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

template <typename TW1, typename TW2>
static int launch_add_rmsnorm(const float* a, const TW1* w1, float eps1, int plus1, float* x, const TW2* w2, float eps2,
                              int plus2, void* out2, int out2_dtype, int T, int H, cudaStream_t stream) {
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (H <= 16 * threads) {
    const int npt = kf_ceil_div(H, threads);
#define KF_GO(TO, NPT) kf_launch(add_rmsnorm_reg_kernel<TW1, TW2, TO, NPT>, dim3(T), dim3(threads), 0, stream, a, w1, eps1, plus1, x, w2, eps2, plus2, (TO*)out2, H)
#define KF_PICK(TO)                                                            \
    if (npt <= 2) KF_GO(TO, 2); else if (npt <= 4) KF_GO(TO, 4); else if (npt <= 8) KF_GO(TO, 8); else KF_GO(TO, 16)
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
