// Paged attention for any head size up to 256, any number of heads and groups, any page size:
// one warp per (token row, query head), exact 32-bit arithmetic (expf, tanhf, no fast-math).
//
// For the row at position p of request r the warp walks keys lo..p in ascending chunks of 32,
// lo = max(0, p - window + 1) on a windowed layer, else 0 (reference: window rule
// crates/kf-backend-cuda/src/kernels/attention.cu:156, scores/softcap :80-81, lane-per-key online softmax :68-103):
//   s_j = (q . k_j) * scale;  s_j = cap * tanh(s_j / cap) if cap > 0
//   o   = sum_j softmax(s)_j v_j,  zeros if no key is visible.
// The order of every sum is fixed by (row, head) alone, so a row's result does not depend on how the
// step was cut or what else is in the batch.  This is the engine's 32-bit attention and the fallback of
// the bfloat16 path for head sizes the tensor-core kernels do not take.
#include "common.cuh"

constexpr int MAX_D = 256;
constexpr int WARPS = 4;

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const TQ* __restrict__ q, TQ* __restrict__ out, const TKV* __restrict__ pages,
                         const int* __restrict__ items, const int* __restrict__ positions,
                         const int* __restrict__ row_req, const int* __restrict__ block_table, int table_stride,
                         int page_size, int nh, int nkv, int d, float scale, float softcap, int window, int T) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * WARPS + warp;
  if (item >= (long)T * nh) return;                       // whole warp leaves together; no block barrier below
  const int it = (int)(item / nh), h = (int)(item - (long)it * nh);
  const int t = items ? items[it] : it;                    // `items` names the rows this launch handles
  const int req = row_req[t];
  TQ* o = out + ((size_t)t * nh + h) * d;
  if (req < 0) {                                            // padding row
    for (int i = lane; i < d; i += 32) kf_store(o, i, 0.f);
    return;
  }
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const TQ* qr = q + ((size_t)t * nh + h) * d;
  for (int i = lane; i < d; i += 32) qs[warp][i] = kf_load(qr, i);
  __syncwarp();

  const int* table = block_table + (size_t)req * table_stride;
  const size_t head_stride = (size_t)page_size * d;
  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int r = 0; r < MAX_D / 32; ++r) acc[r] = 0.f;

  for (int c0 = lo; c0 <= pos; c0 += 32) {
    const int j = c0 + lane;
    const bool valid = j <= pos;
    long kofs = -1;                                         // element offset of key j's row; the value row is +nkv*head_stride
    float s = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      kofs = (((long)page * 2) * nkv + kvh) * (long)head_stride + (long)(j % page_size) * d;
      const TKV* kr = pages + kofs;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(qs[warp][i], kf_load(kr, i), dot);
      s = kf_softcap(dot * scale, softcap);
    }
    const float m_new = fmaxf(m, kf_warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + kf_warp_sum(p);
#pragma unroll
    for (int r = 0; r < MAX_D / 32; ++r) acc[r] *= corr;
    const int n = min(32, pos - c0 + 1);
    for (int u = 0; u < n; ++u) {
      const float pu = __shfl_sync(0xffffffffu, p, u);
      const long vofs = __shfl_sync(0xffffffffu, kofs, u) + (long)nkv * (long)head_stride;
      const TKV* vr = pages + vofs;
#pragma unroll
      for (int r = 0; r < MAX_D / 32; ++r) {
        const int i = lane + 32 * r;
        if (i < d) acc[r] = fmaf(pu, kf_load(vr, i), acc[r]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int r = 0; r < MAX_D / 32; ++r) {
    const int i = lane + 32 * r;
    if (i < d) kf_store(o, i, acc[r] * inv);
  }
}

// items: rows of the step to process (null = rows 0..T-1); T is then the number of items.
KF_API int kf_attention_generic(const void* q, void* out, int q_dtype, const void* pages, int kv_dtype,
                                const int* items, const int* positions, const int* row_req, const int* block_table, int table_stride,
                                int page_size, int nh, int nkv, int d, float scale, float softcap, int window,
                                int T, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (d < 1 || d > MAX_D || nkv < 1 || nh % nkv != 0 || page_size < 1) return KF_ERR_SIZE;
  const long n_work = (long)T * nh;
  const int blocks = (int)((n_work + WARPS - 1) / WARPS);
#define KF_GO(TQ, TKV)                                                                                     \
  kf_launch(attention_generic_kernel<TQ, TKV>, dim3(blocks), dim3(WARPS * 32), 0, stream,                                     \
      (const TQ*)q, (TQ*)out, (const TKV*)pages, items, positions, row_req, block_table, table_stride, page_size, \
      nh, nkv, d, scale, softcap, window, T)
  if (q_dtype == KF_F32 && kv_dtype == KF_F32) KF_GO(float, float);
  else if (q_dtype == KF_BF16 && kv_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
