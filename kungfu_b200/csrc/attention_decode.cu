// Split-KV decode attention over paged bfloat16 keys and values: one query row per item, softcap and window.
//
// Work: a block is (item, kv head, split of the visible keys, group of up to HT query heads that share the kv
// head).  Inside a block every "lane group" of D/8 lanes owns one key at a time: each lane loads 16 bytes of the
// key row, the partial dot products of the HT heads are summed across the lane group by shuffles, the score is
// capped, and the lane accumulates its 8 value elements with an online softmax of its own.  Lane groups, warps
// and splits are merged at the end, always in index order; the block that arrives last for an (item, kv head,
// head group) merges the splits (no block waits for another).  Scores, softmax and sums are 32-bit.
// Head sizes 16, 32, 64, 128, 256 (D/8 lanes per key must divide a warp); other sizes use the generic kernel.
// Reference counterpart: crates/kf-backend-cuda/src/kernels/attention_decode.cuh:93-458 (split-KV, last block merges).
#include "common.cuh"

namespace {

constexpr int DEC_WARPS = 8;
constexpr int UNROLL = 4;

template <int HT>
struct State {
  float m[HT], l[HT], acc[HT][8];
};

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(p[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// 16-byte load that does not linger in L1: every key and value is read once per step
__device__ __forceinline__ uint4 ld_stream(const __nv_bfloat16* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
// 32-bit exponential and softcap through the hardware's base-2 exponential and reciprocal (relative error ~1e-6,
// far below the rounding of the bfloat16 operands); the 32-bit path of the engine uses expf/tanhf instead.
__device__ __forceinline__ float exp_fast(float x) { return exp2f(x * 1.4426950408889634f); }
__device__ __forceinline__ float softcap_fast(float x, float cap) {
  if (cap <= 0.f) return x;
  const float e = exp2f(x * (2.f * 1.4426950408889634f / cap));       // exp(2x/cap)
  return cap * (1.f - __fdividef(2.f, e + 1.f));                       // cap * tanh(x/cap)
}

// merge (m2, l2, a2) into (m, l, a)
__device__ __forceinline__ void merge1(float& m, float& l, float* a, float m2, float l2, const float* a2) {
  const float mn = fmaxf(m, m2);
  const float c1 = (m == -INFINITY) ? 0.f : expf(m - mn);
  const float c2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
  l = l * c1 + l2 * c2;
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = a[i] * c1 + a2[i] * c2;
  m = mn;
}

template <int D, int HT>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages,
                   const int* __restrict__ items, int n_items, const int* __restrict__ positions,
                   const int* __restrict__ row_req, const int* __restrict__ table, int table_stride, int page_size,
                   int nh, int nkv, float scale, float softcap, int window, int n_splits,
                   float* __restrict__ partial, int* __restrict__ counters, __nv_bfloat16* __restrict__ out) {
  kf_pdl_trigger();
  kf_pdl_wait();
  constexpr int LPK = D / 8;                 // lanes per key
  constexpr int KPW = 32 / LPK;              // keys per warp and iteration
  constexpr int PSTRIDE = D + 2;             // partial record: acc[D], m, l
  __shared__ float sm_acc[DEC_WARPS][HT][D];
  __shared__ float sm_ml[DEC_WARPS][HT][2];
  __shared__ int s_last;

  const int item = blockIdx.x / nkv, kvh = blockIdx.x - item * nkv;
  const int split = blockIdx.y, hz = blockIdx.z;
  const int G = nh / nkv;
  const int h_first = kvh * G + hz * HT;                      // first query head of this block
  const int h_count = min(HT, G - hz * HT);
  const int t = items ? items[item] : item;
  const int req = row_req[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPK, chunk = lane - grp * LPK;      // which key of the iteration, which 8 elements
  __nv_bfloat16* orow = out + (size_t)t * nh * D;

  if (req < 0) {                                              // padding row: zeros, no partials, no counter
    if (split == 0)
      for (int e = threadIdx.x; e < h_count * D; e += blockDim.x) orow[(size_t)h_first * D + e] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos + 1 - lo;
  int per = (n_keys + n_splits - 1) / n_splits;
  per = (per + 63) & ~63;                                     // whole 64-key runs per split
  const int k_begin = lo + split * per;
  const int k_end = min(pos + 1, k_begin + per);

  float qf[HT][8];
#pragma unroll
  for (int h = 0; h < HT; ++h) {
    if (h < h_count) {
      const uint4 r = *reinterpret_cast<const uint4*>(q + ((size_t)t * nh + h_first + h) * D + chunk * 8);
      unpack8(r, qf[h]);
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[h][i] *= scale;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) qf[h][i] = 0.f;
    }
  }
  State<HT> st;
#pragma unroll
  for (int h = 0; h < HT; ++h) {
    st.m[h] = -INFINITY;
    st.l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) st.acc[h][i] = 0.f;
  }
  const int* tab = table + (size_t)req * table_stride;
  const size_t head_stride = (size_t)page_size * D;
  const size_t v_off = (size_t)nkv * head_stride;             // from a key row to the value row of the same slot

  for (int k0 = k_begin + warp * KPW * UNROLL; k0 < k_end; k0 += DEC_WARPS * KPW * UNROLL) {
    uint4 kr[UNROLL], vr[UNROLL];
    bool valid[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int j = k0 + u * KPW + grp;
      valid[u] = j < k_end;
      if (valid[u]) {
        const int page = tab[j / page_size];
        const __nv_bfloat16* kp = pages + ((size_t)page * 2 * nkv + kvh) * head_stride + (size_t)(j % page_size) * D + chunk * 8;
        kr[u] = ld_stream(kp);
        vr[u] = ld_stream(kp + v_off);
      } else {
        kr[u] = make_uint4(0, 0, 0, 0);
        vr[u] = make_uint4(0, 0, 0, 0);
      }
    }
    // scores of the UNROLL keys of this lane group, all heads (independent chains)
    float s[UNROLL][HT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float kf[8];
      unpack8(kr[u], kf);
#pragma unroll
      for (int h = 0; h < HT; ++h) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(qf[h][i], kf[i], d);
        s[u][h] = d;
      }
    }
#pragma unroll
    for (int o = LPK / 2; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int h = 0; h < HT; ++h) s[u][h] += __shfl_xor_sync(0xffffffffu, s[u][h], o);
    // one online-softmax update per head for the whole batch of keys
#pragma unroll
    for (int h = 0; h < HT; ++h) {
      float mn = st.m[h];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        s[u][h] = valid[u] ? softcap_fast(s[u][h], softcap) : -INFINITY;
        mn = fmaxf(mn, s[u][h]);
      }
      if (mn == -INFINITY) continue;                          // nothing valid yet for this lane group
      const float c = exp_fast(st.m[h] - mn);                 // exp(-inf) = 0 on the first batch
      float lsum = 0.f;
      float p[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) { p[u] = exp_fast(s[u][h] - mn); lsum += p[u]; }
      st.l[h] = st.l[h] * c + lsum;
      st.m[h] = mn;
#pragma unroll
      for (int i = 0; i < 8; ++i) st.acc[h][i] *= c;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        float vf[8];
        unpack8(vr[u], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) st.acc[h][i] = fmaf(p[u], vf[i], st.acc[h][i]);
      }
    }
  }
  // ---- merge the lane groups of a warp (same chunk, different key streams), in a fixed order -------------------
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int h = 0; h < HT; ++h) {
      const float m2 = __shfl_xor_sync(0xffffffffu, st.m[h], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, st.l[h], o);
      float a2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a2[i] = __shfl_xor_sync(0xffffffffu, st.acc[h][i], o);
      merge1(st.m[h], st.l[h], st.acc[h], m2, l2, a2);
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int h = 0; h < HT; ++h) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_acc[warp][h][chunk * 8 + i] = st.acc[h][i];
      if (chunk == 0) { sm_ml[warp][h][0] = st.m[h]; sm_ml[warp][h][1] = st.l[h]; }
    }
  }
  __syncthreads();
  // ---- merge the warps; thread e owns (head, element) ----------------------------------------------------------
  const size_t rec_base = (((size_t)t * nh + h_first) * n_splits + split) * PSTRIDE;   // + h * n_splits * PSTRIDE
  for (int e = threadIdx.x; e < h_count * D; e += blockDim.x) {
    const int h = e / D, i = e - h * D;
    float m = -INFINITY;
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, sm_ml[w][h][0]);
    float l = 0.f, a = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = sm_ml[w][h][0];
      const float c = (mw == -INFINITY) ? 0.f : expf(mw - m);
      l += sm_ml[w][h][1] * c;
      a += sm_acc[w][h][i] * c;
    }
    if (n_splits == 1) {
      orow[(size_t)(h_first + h) * D + i] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
    } else {
      float* rec = partial + rec_base + (size_t)h * n_splits * PSTRIDE;
      rec[i] = a;
      if (i == 0) { rec[D] = m; rec[D + 1] = l; }
    }
  }
  if (n_splits == 1) return;
  // ---- the block that arrives last merges the splits, in split order ---------------------------------------------
  __threadfence();
  __syncthreads();
  const int cidx = (item * nkv + kvh) * gridDim.z + hz;
  if (threadIdx.x == 0) s_last = (atomicAdd(&counters[cidx], 1) == n_splits - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < h_count * D; e += blockDim.x) {
    const int h = e / D, i = e - h * D;
    const float* rec0 = partial + (((size_t)t * nh + h_first + h) * n_splits) * PSTRIDE;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, __ldcg(rec0 + (size_t)s * PSTRIDE + D));
    float l = 0.f, a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = __ldcg(rec0 + (size_t)s * PSTRIDE + D);
      const float c = (ms == -INFINITY) ? 0.f : expf(ms - m);
      l += __ldcg(rec0 + (size_t)s * PSTRIDE + D + 1) * c;
      a += __ldcg(rec0 + (size_t)s * PSTRIDE + i) * c;
    }
    orow[(size_t)(h_first + h) * D + i] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
  }
  if (threadIdx.x == 0) counters[cidx] = 0;
}

template <int D, int HT>
int launch_decode(const void* q, const void* pages, const int* items, int n_items, const int* positions, const int* row_req,
                  const int* table, int table_stride, int page_size, int nh, int nkv, float scale, float softcap, int window,
                  int n_splits, float* partial, int* counters, void* out, cudaStream_t stream) {
  const int G = nh / nkv;
  dim3 grid(n_items * nkv, n_splits, kf_ceil_div(G, HT));
  kf_launch(attn_decode_kernel<D, HT>, dim3(grid), dim3(DEC_WARPS * 32), 0, stream, 
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, items, n_items, positions, row_req, table, table_stride,
      page_size, nh, nkv, scale, softcap, window, n_splits, partial, counters, (__nv_bfloat16*)out);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <int D>
int launch_decode_d(int ht, const void* q, const void* pages, const int* items, int n_items, const int* positions,
                    const int* row_req, const int* table, int table_stride, int page_size, int nh, int nkv, float scale,
                    float softcap, int window, int n_splits, float* partial, int* counters, void* out, cudaStream_t s) {
#define KF_ARGS q, pages, items, n_items, positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, n_splits, partial, counters, out, s
  if (ht == 1) return launch_decode<D, 1>(KF_ARGS);
  if (ht == 2) return launch_decode<D, 2>(KF_ARGS);
  return launch_decode<D, 4>(KF_ARGS);
#undef KF_ARGS
}

}  // namespace

KF_API int kf_attention_decode_supported(int d) { return d == 16 || d == 32 || d == 64 || d == 128 || d == 256; }

// Heads per block and the number of counters / partial floats a launch needs.
KF_API int kf_attention_decode_plan(int n_items, int nh, int nkv, int d, int max_keys, int* ht_out, int* splits_out) {
  const int G = nh / nkv;
  const int ht = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
  const long blocks = (long)n_items * nkv * kf_ceil_div(G, ht);
  // two blocks of this kernel are resident per SM: fill one wave of 2 x 148 blocks, never a second partial wave
  int splits = (int)((2 * 148) / blocks);
  const int by_len = (max_keys + 255) / 256;                  // at least 256 keys per split
  if (splits > by_len) splits = by_len;
  if (splits > 32) splits = 32;
  if (splits < 1) splits = 1;
  *ht_out = ht;
  *splits_out = splits;
  return KF_OK;
}

// q, out: [T, nh*d] bfloat16.  items: rows of the step this launch handles (null = rows 0..n_items-1).
// partial: n_rows_total * nh * splits * (d + 2) floats; counters: n_items * nkv * ceil(G/ht) zeroed ints (left zero).
KF_API int kf_attention_decode(const void* q, void* out, const void* pages, const int* items, int n_items,
                               const int* positions, const int* row_req, const int* table, int table_stride,
                               int page_size, int nh, int nkv, int d, float scale, float softcap, int window, int ht,
                               int n_splits, float* partial, int* counters, cudaStream_t stream) {
  if (n_items <= 0) return KF_OK;
  if (nkv < 1 || nh % nkv != 0 || page_size < 1 || n_splits < 1) return KF_ERR_SIZE;
  if (n_splits > 1 && (!partial || !counters)) return KF_ERR_SIZE;
#define KF_ARGS ht, q, pages, items, n_items, positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, n_splits, partial, counters, out, stream
  switch (d) {
    case 16: return launch_decode_d<16>(KF_ARGS);
    case 32: return launch_decode_d<32>(KF_ARGS);
    case 64: return launch_decode_d<64>(KF_ARGS);
    case 128: return launch_decode_d<128>(KF_ARGS);
    case 256: return launch_decode_d<256>(KF_ARGS);
  }
#undef KF_ARGS
  return KF_ERR_SIZE;
}

// ---- decode attention for callers that cannot allocate ---------------------------------------------------------
// See attention_decode_static.h.  The split partials and the arrival counters live in the two file-scope device
// arrays below instead of caller-provided buffers.
#include "attention_decode_static.h"
#include <mutex>

static __device__ __align__(256) float g_static_partial[KF_DECODE_STATIC_MAX_PARTIAL_FLOATS];
static __device__ __align__(256) int g_static_counters[KF_DECODE_STATIC_MAX_COUNTERS];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
float* g_static_partial_ptr[MAX_DEVICES] = {};
int* g_static_counters_ptr[MAX_DEVICES] = {};
}  // namespace

KF_API int kf_attention_decode_static(const void* q, void* out, const void* pages, int n_rows, const int* positions,
                                      const int* row_req, const int* table, int table_stride, int page_size, int nh,
                                      int nkv, int d, float scale, float softcap, int window, int max_keys,
                                      cudaStream_t stream) {
  if (n_rows <= 0) return KF_OK;
  if (nkv < 1 || nh % nkv != 0 || page_size < 1 || !kf_attention_decode_supported(d)) return KF_ERR_SIZE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return KF_ERR_SETUP;
  float* partial = nullptr;
  int* counters = nullptr;
  {
    // One-time set-up per device, with that device current: in host code the arrays' names are host-side
    // stand-ins, not device addresses, so the addresses the kernel gets are asked for here.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_partial_ptr[dev]) {
      float* p = nullptr;
      int* c = nullptr;
      cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_partial);
      if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&c, g_static_counters);
      if (e != cudaSuccess || !p || !c) {
        kf_record_cuda_error(e);
        return KF_ERR_SETUP;
      }
      g_static_partial_ptr[dev] = p;
      g_static_counters_ptr[dev] = c;
    }
    partial = g_static_partial_ptr[dev];
    counters = g_static_counters_ptr[dev];
  }
  int ht = 1, splits = 1;
  kf_attention_decode_plan(n_rows, nh, nkv, d, max_keys, &ht, &splits);
  const long n_counters = (long)n_rows * nkv * kf_ceil_div(nh / nkv, ht);
  const long n_partial = (long)n_rows * nh * splits * (d + 2);
  if (n_counters > KF_DECODE_STATIC_MAX_COUNTERS || n_partial > KF_DECODE_STATIC_MAX_PARTIAL_FLOATS) {
    kf_record_message("kf_attention_decode_static: rows * heads * splits * (head_dim + 2) exceeds the built-in scratch");
    return KF_ERR_SIZE;
  }
  // The arrays keep what the last call left; the counters must start at zero.
  if (cudaMemsetAsync(counters, 0, (size_t)n_counters * sizeof(int), stream) != cudaSuccess) {
    kf_record_cuda_error(cudaGetLastError());
    return KF_ERR_LAUNCH;
  }
  return kf_attention_decode(q, out, pages, nullptr, n_rows, positions, row_req, table, table_stride, page_size, nh, nkv,
                             d, scale, softcap, window, ht, splits, partial, counters, stream);
}
