// Embedding gather, rotary tables, gated activation, residual add.
#include "common.cuh"

// x[t, :] = table[token[t], :] * scale.  A token id outside [0, V) writes zeros and sets *bad.
// Reference: gather then scale, crates/kf-layers/src/basic.rs:35-36.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, float scale,
                             float* __restrict__ out, int H, int V, int* __restrict__ bad) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < V;
  if (!ok && threadIdx.x == 0 && bad) atomicExch(bad, 1);
  const TW* row = table + (size_t)(ok ? tok : 0) * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? kf_load(row, i) * scale : 0.f;
}

KF_API int kf_embed(const int* tokens, const void* table, int table_dtype, float scale, float* out,
                    int T, int H, int V, int* bad_flag, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == KF_F32)
    kf_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, tokens, (const float*)table, scale, out, H, V, bad_flag);
  else if (table_dtype == KF_BF16)
    kf_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, scale, out, H, V, bad_flag);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// cos/sin of position * inv_freq[i], all in 32-bit (accurate sincosf: no fast-math in this library).
// The product of a position and a 32-bit frequency has up to 48 significant bits; rounded to 32-bit it is off by up to
// 2.4e-4 rad at position 4,000, which a 32-bit engine with scores of 40 shows in its logits.  So the product is kept as
// an unevaluated sum hi + lo (lo = fma(p, f, -hi) is its exact rounding error) and the tables are
// cos(hi) (1 - lo^2/2) - lo sin(hi) and sin(hi) (1 - lo^2/2) + lo cos(hi): exact to second order in lo, which is below
// 2^-11 up to position 8,192 and below 2^-8 up to 131,072 (error below 1e-7 there).
// Reference: crates/kf-backend-cuda/src/kernels/rope.cu:4-14 (angle as one 32-bit product).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int T, int half) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, i = idx - t * half;
  const float p = (float)positions[t], f = inv_freq[i];
  const float hi = __fmul_rn(p, f);
  const float lo = __fmaf_rn(p, f, -hi);
  float s, c;
  sincosf(hi, &s, &c);
  const float h = 1.f - 0.5f * lo * lo;
  cos_out[idx] = __fmaf_rn(-lo, s, c * h);
  sin_out[idx] = __fmaf_rn(lo, c, s * h);
}

KF_API int kf_rope_table(const int* positions, const float* inv_freq, float* cos_out, float* sin_out,
                         int T, int half, cudaStream_t stream) {
  if (T <= 0 || half <= 0) return KF_OK;
  const int n = T * half;
  kf_launch(rope_table_kernel, dim3(kf_ceil_div(n, 256)), dim3(256), 0, stream, positions, inv_freq, cos_out, sin_out, T, half);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// out[t, j] = act(gu[t, j]) * gu[t, I + j]: gate columns first, up columns second.
// Reference: crates/kf-backend-cuda/src/kernels/elementwise.cu:42-44.
template <typename TI, typename TO>
__global__ void gated_act_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int T, int I, int act) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const size_t n = (size_t)T * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I, j = idx - t * I;
    const float g = kf_load(gu, t * 2 * I + j), u = kf_load(gu, t * 2 * I + I + j);
    kf_store(out, idx, kf_act(g, act) * u);
  }
}

KF_API int kf_gated_act(const void* gu, int in_dtype, void* out, int out_dtype, int T, int I, int act, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  const size_t n = (size_t)T * I;
  const int blocks = (int)((n + 255) / 256 > kf_sm_count() * 16 ? kf_sm_count() * 16 : (n + 255) / 256);
  if (in_dtype == KF_F32 && out_dtype == KF_F32)
    kf_launch(gated_act_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, T, I, act);
  else if (in_dtype == KF_F32 && out_dtype == KF_BF16)
    kf_launch(gated_act_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (__nv_bfloat16*)out, T, I, act);
  else if (in_dtype == KF_BF16 && out_dtype == KF_BF16)
    kf_launch(gated_act_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I, act);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

__global__ void add_kernel(const float* __restrict__ a, float* __restrict__ x, size_t n) {
  kf_pdl_trigger();
  kf_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += a[i];
}

KF_API int kf_add(const float* a, float* x, long n, cudaStream_t stream) {
  if (n <= 0) return KF_OK;
  const long b = (n + 255) / 256;
  kf_launch(add_kernel, dim3((int)(b > kf_sm_count() * 16 ? kf_sm_count() * 16 : b)), dim3(256), 0, stream, a, x, (size_t)n);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// dst = (bf16 or f32) copy of src with conversion; used where a 32-bit weight meets bf16 activations.
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ src, TO* __restrict__ dst, size_t n) {
  kf_pdl_trigger();
  kf_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    kf_store(dst, i, kf_load(src, i));
}

KF_API int kf_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long n, cudaStream_t stream) {
  if (n <= 0) return KF_OK;
  const long b = (n + 255) / 256;
  const int blocks = (int)(b > kf_sm_count() * 16 ? kf_sm_count() * 16 : b);
  if (src_dtype == KF_BF16 && dst_dtype == KF_F32)
    kf_launch(convert_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)src, (float*)dst, (size_t)n);
  else if (src_dtype == KF_F32 && dst_dtype == KF_BF16)
    kf_launch(convert_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)src, (__nv_bfloat16*)dst, (size_t)n);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// ---- random weights: a counter-based generator that the host restates bit for bit ---------------------------------
// Element i of a tensor with 64-bit key k: three 64-bit words w_j = mix(k + (3 i + j) * 0x9E3779B97F4A7C15), j = 0..2
// (the splitmix64 finaliser), cut into twelve 16-bit numbers whose sum s has mean 393210 and standard deviation 65536
// (to 1e-10); value = float(s - 393210) * (std / 65536).  Integer arithmetic, one exact conversion and one 32-bit
// multiplication: the same bits on any machine (kungfu_b200/weights/store.py restates it with numpy).  The sum of
// twelve uniforms is bell-shaped within +-6 standard deviations, which is all random test weights need.
// The reference's tests draw their tensors from a small generator of their own the same way
// (crates/kf-backend-cuda/tests/common/mod.rs:71-97).
__host__ __device__ __forceinline__ unsigned long long kf_mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename TO>
__global__ void random_normal_kernel(TO* __restrict__ out, size_t n, unsigned long long key, float step) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    int s = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const unsigned long long w = kf_mix64(key + (3ull * i + j) * 0x9E3779B97F4A7C15ull);
      s += (int)(w & 0xFFFF) + (int)((w >> 16) & 0xFFFF) + (int)((w >> 32) & 0xFFFF) + (int)(w >> 48);
    }
    kf_store(out, i, __fmul_rn((float)(s - 393210), step));
  }
}

__global__ void random_table_kernel(int* __restrict__ out, size_t n, unsigned long long key) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = (int)(kf_mix64(key + (3ull * i) * 0x9E3779B97F4A7C15ull) & 0x7FFF);
}

// out[i] = the i-th value of stream `key` times std (32-bit or bfloat16, rounded to nearest even), or, for
// dtype -1, a 15-bit integer.
KF_API int kf_random_fill(void* out, int dtype, long n, unsigned long long key, float std, cudaStream_t stream) {
  if (n <= 0) return KF_OK;
  const long b = (n + 255) / 256;
  const int blocks = (int)(b > kf_sm_count() * 32 ? kf_sm_count() * 32 : b);
  const float step = std / 65536.0f;
  if (dtype == KF_F32) random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (size_t)n, key, step);
  else if (dtype == KF_BF16) random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (size_t)n, key, step);
  else if (dtype == -1) random_table_kernel<<<blocks, 256, 0, stream>>>((int*)out, (size_t)n, key);
  else return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}
