// Rotate queries and keys by the step's cos/sin table and write keys and values into the request's pages.
//
// Input is the 32-bit result of the stacked q|k|v product, one row per token:
//   [ n_heads*d | n_kv_heads*d | n_kv_heads*d ].
// Pairs are (i, i + rot/2) for i < rot/2; elements at or beyond `rot` pass through unrotated
// (reference: crates/kf-backend-cuda/src/kernels/rope.cu:16-37, fused append fused.cu:143-188).
// Page layout: pages[page][0 = key | 1 = value][kv head][slot in page][d].
// A row whose request index is negative is padding: its query is zeroed and nothing is written to pages.
#include "common.cuh"

template <typename TQ, typename TKV>
__global__ void rope_kv_append_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int rot, int nh, int nkv, int d,
                                      const int* __restrict__ positions, const int* __restrict__ row_req,
                                      const int* __restrict__ block_table, int table_stride, int page_size,
                                      TKV* __restrict__ pages, TQ* __restrict__ q_out, int write_kv) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int t = blockIdx.x;
  const int req = row_req[t];
  const int half = rot >> 1;
  const int row_w = (nh + 2 * nkv) * d;
  const float* in = qkv + (size_t)t * row_w;
  const float* c = cos_t ? cos_t + (size_t)t * half : nullptr;
  const float* s = sin_t ? sin_t + (size_t)t * half : nullptr;
  TQ* qo = q_out + (size_t)t * nh * d;

  // queries: every (head, element)
  for (int e = threadIdx.x; e < nh * d; e += blockDim.x) {
    const int i = e % d;
    float v = in[e];
    if (req < 0) v = 0.f;
    else if (i < half) v = v * c[i] - in[e + half] * s[i];
    else if (i < rot) v = in[e - half] * s[i - half] + v * c[i - half];
    kf_store(qo, e, v);
  }
  if (!write_kv || req < 0) return;
  const int pos = positions[t];
  const int page = block_table[(size_t)req * table_stride + pos / page_size];
  if (page < 0) return;                                     // never for a reserved position; guards the store
  const int slot = pos % page_size;
  const size_t head_stride = (size_t)page_size * d;
  TKV* kbase = pages + ((size_t)page * 2 + 0) * nkv * head_stride + (size_t)slot * d;
  TKV* vbase = pages + ((size_t)page * 2 + 1) * nkv * head_stride + (size_t)slot * d;
  const float* kin = in + nh * d;
  const float* vin = kin + nkv * d;
  for (int e = threadIdx.x; e < nkv * d; e += blockDim.x) {
    const int h = e / d, i = e - h * d;
    float v = kin[e];
    if (i < half) v = v * c[i] - kin[e + half] * s[i];
    else if (i < rot) v = kin[e - half] * s[i - half] + v * c[i - half];
    kf_store(kbase, (size_t)h * head_stride + i, v);
    kf_store(vbase, (size_t)h * head_stride + i, vin[e]);
  }
}

// The same four elements at a time (head size and rot/2 multiples of 4): 16-byte loads of the row and of the tables.
__device__ __forceinline__ void kf_store_vec4(float* o, size_t i, float4 v) { *reinterpret_cast<float4*>(o + i) = v; }
__device__ __forceinline__ void kf_store_vec4(__nv_bfloat16* o, size_t i, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(o + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// One group of four elements of a head (i = first element within the head), rotated.
__device__ __forceinline__ float4 kf_rotated4(const float* __restrict__ head, int i, int half, int rot,
                                              const float* __restrict__ c, const float* __restrict__ s) {
  const float4 v = *reinterpret_cast<const float4*>(head + i);
  if (i < half) {
    const float4 p = *reinterpret_cast<const float4*>(head + i + half);
    const float4 cc = *reinterpret_cast<const float4*>(c + i), ss = *reinterpret_cast<const float4*>(s + i);
    return make_float4(v.x * cc.x - p.x * ss.x, v.y * cc.y - p.y * ss.y, v.z * cc.z - p.z * ss.z, v.w * cc.w - p.w * ss.w);
  }
  if (i < rot) {
    const float4 p = *reinterpret_cast<const float4*>(head + i - half);
    const float4 cc = *reinterpret_cast<const float4*>(c + i - half), ss = *reinterpret_cast<const float4*>(s + i - half);
    return make_float4(p.x * ss.x + v.x * cc.x, p.y * ss.y + v.y * cc.y, p.z * ss.z + v.z * cc.z, p.w * ss.w + v.w * cc.w);
  }
  return v;
}

template <typename TQ, typename TKV>
__global__ void rope_kv_append_vec_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int rot, int nh, int nkv, int d,
                                          const int* __restrict__ positions, const int* __restrict__ row_req,
                                          const int* __restrict__ block_table, int table_stride, int page_size,
                                          TKV* __restrict__ pages, TQ* __restrict__ q_out, int write_kv) {
  kf_pdl_trigger();
  const int t = blockIdx.x;
  const int req = row_req[t];                                  // the step's integers do not depend on earlier kernels
  const int pos = positions[t];
  const int page = (write_kv && req >= 0) ? block_table[(size_t)req * table_stride + pos / page_size] : -1;
  kf_pdl_wait();
  qkv = kf_produced(qkv), cos_t = kf_produced(cos_t), sin_t = kf_produced(sin_t);
  const int half = rot >> 1;
  const int row_w = (nh + 2 * nkv) * d;
  const float* in = qkv + (size_t)t * row_w;
  const float* c = cos_t ? cos_t + (size_t)t * half : nullptr;
  const float* s = sin_t ? sin_t + (size_t)t * half : nullptr;
  TQ* qo = q_out + (size_t)t * nh * d;
  const int d4 = d >> 2;
  const size_t head_stride = (size_t)page_size * d;
  const int slot = pos % page_size;
  TKV* kbase = page >= 0 ? pages + ((size_t)page * 2 + 0) * nkv * head_stride + (size_t)slot * d : nullptr;
  TKV* vbase = page >= 0 ? pages + ((size_t)page * 2 + 1) * nkv * head_stride + (size_t)slot * d : nullptr;
  const int n4 = (nh + 2 * nkv) * d4;                          // groups of four in the row: q heads, k heads, v heads
  for (int e = threadIdx.x; e < n4; e += blockDim.x) {
    const int hd = e / d4, i = (e - hd * d4) * 4;
    if (hd < nh) {
      const float4 v = req < 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : kf_rotated4(in + (size_t)hd * d, i, half, rot, c, s);
      kf_store_vec4(qo, (size_t)hd * d + i, v);
    } else if (page >= 0) {
      if (hd < nh + nkv) kf_store_vec4(kbase, (size_t)(hd - nh) * head_stride + i, kf_rotated4(in + (size_t)hd * d, i, half, rot, c, s));
      else kf_store_vec4(vbase, (size_t)(hd - nh - nkv) * head_stride + i, *reinterpret_cast<const float4*>(in + (size_t)hd * d + i));
    }
  }
}

KF_API int kf_rope_kv_append(const float* qkv, const float* cos_t, const float* sin_t, int rot, int nh, int nkv, int d,
                             const int* positions, const int* row_req, const int* block_table, int table_stride,
                             int page_size, void* pages, int kv_dtype, void* q_out, int q_dtype, int write_kv,
                             int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (rot < 0 || rot > d || (rot & 1)) return KF_ERR_SIZE;
  if (rot > 0 && (!cos_t || !sin_t)) return KF_ERR_SIZE;
  const int threads = 256;
  const bool vec = d % 4 == 0 && rot % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)pages |
                                                   (uintptr_t)q_out) & 15) == 0;
#define KF_GO(TQ, TKV)                                                                                              \
  if (vec)                                                                                                          \
    kf_launch(rope_kv_append_vec_kernel<TQ, TKV>, dim3(T), dim3(threads), 0, stream, qkv, cos_t, sin_t, rot, nh, nkv, d, positions, \
              row_req, block_table, table_stride, page_size, (TKV*)pages, (TQ*)q_out, write_kv);                    \
  else                                                                                                              \
    kf_launch(rope_kv_append_kernel<TQ, TKV>, dim3(T), dim3(threads), 0, stream, qkv, cos_t, sin_t, rot, nh, nkv, d, positions, row_req, \
                                                            block_table, table_stride, page_size, (TKV*)pages,      \
                                                            (TQ*)q_out, write_kv)
  if (q_dtype == KF_F32 && kv_dtype == KF_F32) { KF_GO(float, float); }
  else if (q_dtype == KF_BF16 && kv_dtype == KF_BF16) { KF_GO(__nv_bfloat16, __nv_bfloat16); }
  else if (q_dtype == KF_F32 && kv_dtype == KF_BF16) { KF_GO(float, __nv_bfloat16); }
  else if (q_dtype == KF_BF16 && kv_dtype == KF_F32) { KF_GO(__nv_bfloat16, float); }
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
