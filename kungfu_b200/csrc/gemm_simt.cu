// Generic matrix product  out[T, N] = x[T, K] . w[N, K]^T  with 32-bit FMA accumulation.
//
// This is the true 32-bit product of the engine (no tensor-core or reduced-precision mode) and the
// fallback for shapes the tensor-core kernel refuses.  Any T, N, K.  Every output element is summed
// over k in ascending order by one thread, so a row's result does not depend on T or on which other
// rows share the launch.  Reference counterpart: the 32x64x64 shared-tile product in
// crates/kf-backend-cuda/src/kernels/quant.cuh:110-171.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                 int T, int N, int K, float softcap) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;          // this thread loads row lr, k = lk..lk+3 of each tile
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int r = row0 + lr;
      const TX* p = x + (size_t)r * K + k0 + lk;
#pragma unroll
      for (int u = 0; u < 4; ++u) xs[lk + u][lr] = (r < T && k0 + lk + u < K) ? kf_load(p, u) : 0.f;
      const int c = col0 + lr;
      const TW* q = w + (size_t)c * K + k0 + lk;
#pragma unroll
      for (int u = 0; u < 4; ++u) ws[lk + u][lr] = (c < N && k0 + lk + u < K) ? kf_load(q, u) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c < N) kf_store(out, (size_t)r * N + c, kf_softcap(acc[i][j], softcap));
    }
  }
}

template <typename TX, typename TW>
static int launch(const TX* x, const TW* w, void* out, int out_dtype, int T, int N, int K, float softcap, cudaStream_t s) {
  dim3 grid(kf_ceil_div(N, BN), kf_ceil_div(T, BM));
  if (out_dtype == KF_F32)
    kf_launch(gemm_simt_kernel<TX, TW, float>, dim3(grid), dim3(256), 0, s, x, w, (float*)out, T, N, K, softcap);
  else if (out_dtype == KF_BF16)
    kf_launch(gemm_simt_kernel<TX, TW, __nv_bfloat16>, dim3(grid), dim3(256), 0, s, x, w, (__nv_bfloat16*)out, T, N, K, softcap);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// softcap > 0 applies cap * tanh(v / cap) to every output element.
KF_API int kf_linear_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                          int T, int N, int K, float softcap, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return KF_OK;
  if (K <= 0) return KF_ERR_SIZE;
  if (x_dtype == KF_F32 && w_dtype == KF_F32) return launch((const float*)x, (const float*)w, out, out_dtype, T, N, K, softcap, stream);
  if (x_dtype == KF_BF16 && w_dtype == KF_BF16) return launch((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, out_dtype, T, N, K, softcap, stream);
  if (x_dtype == KF_F32 && w_dtype == KF_BF16) return launch((const float*)x, (const __nv_bfloat16*)w, out, out_dtype, T, N, K, softcap, stream);
  if (x_dtype == KF_BF16 && w_dtype == KF_F32) return launch((const __nv_bfloat16*)x, (const float*)w, out, out_dtype, T, N, K, softcap, stream);
  return KF_ERR_DTYPE;
}
