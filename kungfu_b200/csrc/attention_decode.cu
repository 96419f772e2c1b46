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
#include "mma_tiles.cuh"

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


// Partial record of one (row, head, split): acc[D], m, l and two floats of padding, so that records start on 16 bytes.
#define KF_PSTRIDE(D) ((D) + 4)
constexpr int MERGE_MAX_HEADS = 16;
constexpr int MERGE_MAX_SPLITS = 64;

// The block that arrived last merges the splits of its heads.  Loads from L2 are the whole cost here, so they are
// made independent of one another.  Up to eight splits: a thread asks for the maxima, the sums and its four elements of
// every split at once (one round trip) and weighs them itself.  More: first every (head, split) pair's maximum is
// and sum are fetched by a thread of its own, a warp per head turns them into weights exp(m_s - m) / l in shared memory,
// and then every thread sums four elements over the splits with sixteen 16-byte loads in flight.  Splits are summed in index order.
template <int D, bool BASE2>
__device__ __forceinline__ void merge_splits(const float* __restrict__ partial, size_t first_record, int n_heads,
                                             int n_splits, __nv_bfloat16* __restrict__ o_first) {
  constexpr int PS = KF_PSTRIDE(D);
  __shared__ float s_w[MERGE_MAX_HEADS][MERGE_MAX_SPLITS];
  const float* rec0 = partial + first_record * PS;              // record (h, s) at rec0 + (h * n_splits + s) * PS
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, n_warps = blockDim.x >> 5;
  if (n_splits <= 8) {
    for (int e = tid; e < n_heads * (D / 4); e += blockDim.x) {
      const int h = e / (D / 4), i4 = e - h * (D / 4);
      const float* src = rec0 + (size_t)h * n_splits * PS;
      float ms[8], ls[8];
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool in = u < n_splits;
        const float* rec = src + (size_t)(in ? u : 0) * PS;
        ms[u] = in ? __ldcg(rec + D) : -INFINITY;
        ls[u] = in ? __ldcg(rec + D + 1) : 0.f;
        v[u] = in ? __ldcg(reinterpret_cast<const float4*>(rec + i4 * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float m = -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) m = fmaxf(m, ms[u]);
      float l = 0.f;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float c = (ms[u] == -INFINITY) ? 0.f : (BASE2 ? exp2f(ms[u] - m) : expf(ms[u] - m));
        l += ls[u] * c;
        a.x += v[u].x * c; a.y += v[u].y * c; a.z += v[u].z * c; a.w += v[u].w * c;
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * inv, a.y * inv), hi = __floats2bfloat162_rn(a.z * inv, a.w * inv);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(o_first + (size_t)h * D + i4 * 4) = packed;
    }
    return;
  }
  __shared__ float s_l[MERGE_MAX_HEADS][MERGE_MAX_SPLITS];
  for (int idx = tid; idx < n_heads * n_splits; idx += blockDim.x) {
    const int h = idx / n_splits, sp = idx - h * n_splits;
    s_w[h][sp] = __ldcg(rec0 + (size_t)idx * PS + D);
    s_l[h][sp] = __ldcg(rec0 + (size_t)idx * PS + D + 1);
  }
  __syncthreads();
  for (int h = warp; h < n_heads; h += n_warps) {
    float m = -INFINITY;
    for (int sp = lane; sp < n_splits; sp += 32) m = fmaxf(m, s_w[h][sp]);
    m = kf_warp_max(m);
    float l = 0.f;
    for (int sp = lane; sp < n_splits; sp += 32) {
      const float ms = s_w[h][sp];
      const float c = (ms == -INFINITY) ? 0.f : (BASE2 ? exp2f(ms - m) : expf(ms - m));
      l += s_l[h][sp] * c;
      s_w[h][sp] = c;
    }
    // the sum over splits in a fixed order: lanes hold interleaved splits, the butterfly adds them the same way each time
    l = kf_warp_sum(l);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __syncwarp();
    for (int sp = lane; sp < n_splits; sp += 32) s_w[h][sp] *= inv;
  }
  __syncthreads();
  for (int e = tid; e < n_heads * (D / 4); e += blockDim.x) {
    const int h = e / (D / 4), i4 = e - h * (D / 4);
    const float* src = rec0 + (size_t)h * n_splits * PS + i4 * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < n_splits; sp += 16) {              // sixteen 16-byte loads in flight
      float4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = sp + u < n_splits ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + u) * PS)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const float c = sp + u < n_splits ? s_w[h][sp + u] : 0.f;
        a.x += v[u].x * c; a.y += v[u].y * c; a.z += v[u].z * c; a.w += v[u].w * c;
      }
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o_first + (size_t)h * D + i4 * 4) = packed;
  }
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
  constexpr int PSTRIDE = KF_PSTRIDE(D);
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
  merge_splits<D, false>(partial, ((size_t)t * nh + h_first) * n_splits, h_count, n_splits, orow + (size_t)h_first * D);
  if (threadIdx.x == 0) counters[cidx] = 0;
}

// ---- the tensor-core variant -----------------------------------------------------------------------------------
// Same work split (item, kv head, key split), but the query heads that share the kv head (up to 16) are the rows
// of one m16n8k16 tile, so a key costs a handful of instructions instead of a warp's worth of shuffles.  Each of the
// 4 warps walks its own 16-key tiles of the split: the tile's key and value rows are gathered from the pages into
// warp-private shared memory by cp.async (double-buffered, so the next tile is in flight while this one is used),
// S = Q K^T (16 heads x 16 keys) and O += P V run on mma.sync with 32-bit accumulators, the online softmax is the
// one of the prompt kernel.  Warps are merged through shared memory in warp order, splits by the last block.
constexpr int DM_WARPS = 8;                       // two per scheduler: a warp's tile is one chain of dependent instructions
constexpr int DM_BUFS = 3;                        // buffers of one key tile or one value tile per warp: one in use, two in flight
constexpr int DM_KEYS = 16;                       // keys per warp tile

// With `qkv` given (the 32-bit q|k|v rows of the step, a row = [nh*D | nkv*D | nkv*D]) the kernel also does what the
// rotate-and-append kernel would: it rotates its query heads itself, and the block whose key range holds the row's own
// position rotates the new key, writes key and value into the page (if `write_kv`) and then reads them like any other.
// What does not depend on earlier kernels of the step (the step's integers, keys of earlier steps) is requested
// before the grid dependency is waited for.
template <int D>
__global__ void __launch_bounds__(DM_WARPS * 32)
attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ qkv, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int rot, int write_kv, __nv_bfloat16* pages,
                       const int* __restrict__ items, int n_items, const int* __restrict__ positions,
                       const int* __restrict__ row_req, const int* __restrict__ table, int table_stride, int page_size,
                       int nh, int nkv, float scale, float softcap, int window, int n_splits,
                       float* __restrict__ partial, int* __restrict__ counters, __nv_bfloat16* __restrict__ out) {
  using namespace kf_mma;
  kf_pdl_trigger();
  constexpr int CH = D / 8;
  constexpr int NT_O = D / 8;
  constexpr int KS_QK = D / 16;
  constexpr int PSTRIDE = KF_PSTRIDE(D);
  constexpr int TILE = DM_KEYS * D;                               // elements of one key (or value) tile
  extern __shared__ __align__(128) uint8_t dm_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dm_smem);  // [16][D]
  __nv_bfloat16* sKV = sQ + 16 * D;                               // [warp][buffer][16][D]
  __shared__ float sm_ml[DM_WARPS][16][2];
  __shared__ int s_last;

  // ---- the step's integers: written before the step's first kernel, so readable at once -------------------------------
  const int item = blockIdx.x / nkv, kvh = blockIdx.x - item * nkv;
  const int split = blockIdx.y;
  const int G = nh / nkv;
  const int h_first = kvh * G;
  const int t = items ? items[item] : item;
  const int req = row_req[t];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  __nv_bfloat16* orow = out + (size_t)t * nh * D;
  if (req < 0) {
    kf_pdl_wait();
    if (split == 0)
      for (int e = tid; e < G * D; e += blockDim.x) orow[(size_t)h_first * D + e] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n_keys = pos + 1 - lo;
  int per = (n_keys + n_splits - 1) / n_splits;
  per = (per + 63) & ~63;
  const int k_begin = lo + split * per;
  const int k_end = min(pos + 1, k_begin + per);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + DM_KEYS - 1) / DM_KEYS : 0;
  // the tile that holds the row's own key: an earlier kernel of this step writes that key (or this block does)
  const int own_tile = (pos >= k_begin && pos < k_end) ? (pos - k_begin) / DM_KEYS : -1;

  const int* tab = table + (size_t)req * table_stride;
  const size_t head_stride = (size_t)page_size * D;
  const size_t v_off = (size_t)nkv * head_stride;
  __nv_bfloat16* my = sKV + (size_t)warp * DM_BUFS * TILE;        // [buffer]

  // A warp walks its tiles (warp, warp + DM_WARPS, ...) as the sequence K0 V0 K1 V1 ...: item n is the keys (n even) or
  // the values (n odd) of its tile n / 2 and lands in buffer n % DM_BUFS.
  const int n_mine = n_tiles > warp ? (n_tiles - warp + DM_WARPS - 1) / DM_WARPS : 0;
  const int n_loads = 2 * n_mine;
  long row_base = -1;                                             // lanes 0..15: where key j0 + lane of the item's tile lies
  auto load_item = [&](int n, int buf) {
    const int tile = warp + (n >> 1) * DM_WARPS;
    const int j0 = k_begin + tile * DM_KEYS;
    // lanes 0..15 look up the row of key j0 + lane; everyone fetches a row's base by shuffle
    row_base = -1;
    if (lane < DM_KEYS) {
      const int j = j0 + lane;
      if (j < k_end) {
        const int page = tab[j / page_size];
        if (page >= 0) row_base = ((long)page * 2 * nkv + kvh) * (long)head_stride + (long)(j % page_size) * D;
      }
    }
    __nv_bfloat16* dst = my + (size_t)buf * TILE;
    const size_t off = (n & 1) ? v_off : 0;
#pragma unroll
    for (int i = 0; i < (DM_KEYS * CH + 31) / 32; ++i) {
      const int idx = lane + 32 * i;
      const int r = idx / CH, c = idx - r * CH;
      const long b = __shfl_sync(0xffffffffu, row_base, r & 15);
      if (idx < DM_KEYS * CH) {
        const bool ok = b >= 0;
        cp_async16(tile_ptr<D>(dst, r, c), pages + (ok ? b : 0) + off + c * 8, ok);
      }
    }
  };

  // the first items of this warp, except those of the tile with the row's own key: keys of earlier steps
#pragma unroll
  for (int n = 0; n < DM_BUFS; ++n)
    if (n < n_loads && warp + (n >> 1) * DM_WARPS != own_tile) load_item(n, n);
  kf_pdl_wait();
  q = kf_produced(q), qkv = kf_produced(qkv), cos_t = kf_produced(cos_t), sin_t = kf_produced(sin_t);

  if (qkv != nullptr) {
    // ---- Q: rotated here; rows 0..G-1 are the heads of this kv head, the rest of the 16 rows are zero ---------------------
    const float* in = qkv + (size_t)t * (nh + 2 * nkv) * D;
    const int half = rot >> 1;
    const float* cs = cos_t + (size_t)t * half;
    const float* sn = sin_t + (size_t)t * half;
    auto rotated8 = [&](const float* head, int c8) -> uint4 {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int i = c8 * 8 + e;
        float x = head[i];
        if (i < half) x = x * cs[i] - head[i + half] * sn[i];
        else if (i < rot) x = head[i - half] * sn[i - half] + x * cs[i - half];
        v[e] = x;
      }
      return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    };
    for (int idx = tid; idx < 16 * CH; idx += blockDim.x) {
      const int r = idx / CH, c = idx - r * CH;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < G) v = rotated8(in + (size_t)(h_first + r) * D, c);
      *reinterpret_cast<uint4*>(tile_ptr<D>(sQ, r, c)) = v;
    }
    // ---- the row's own key and value: rotated, written to the page by the block that will read them ---------------------
    if (write_kv && own_tile >= 0) {
      const int page = tab[pos / page_size];
      if (page >= 0) {
        __nv_bfloat16* kdst = pages + ((long)page * 2 * nkv + kvh) * (long)head_stride + (long)(pos % page_size) * D;
        const float* kin = in + (size_t)(nh + kvh) * D;
        const float* vin = in + (size_t)(nh + nkv + kvh) * D;
        for (int c = tid; c < CH; c += blockDim.x) {
          *reinterpret_cast<uint4*>(kdst + c * 8) = rotated8(kin, c);
          const float* vv = vin + c * 8;
          *reinterpret_cast<uint4*>(kdst + v_off + c * 8) =
              make_uint4(pack_bf16(vv[0], vv[1]), pack_bf16(vv[2], vv[3]), pack_bf16(vv[4], vv[5]), pack_bf16(vv[6], vv[7]));
        }
      }
    }
  } else {
    // ---- Q as the rotate-and-append kernel left it ---------------------------------------------------------------------
    for (int idx = tid; idx < 16 * CH; idx += blockDim.x) {
      const int r = idx / CH, c = idx - r * CH;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < G) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * nh + h_first + r) * D + c * 8);
      *reinterpret_cast<uint4*>(tile_ptr<D>(sQ, r, c)) = v;
    }
  }
  __syncthreads();                                                // Q in place; the new key and value are in the page
  {
    // the own-key tile, if it is one of this warp's first tiles; then all first items are one group, and empty groups
    // keep the count of one group per item that the loop below relies on
#pragma unroll
    for (int n = 0; n < DM_BUFS; ++n)
      if (n < n_loads && warp + (n >> 1) * DM_WARPS == own_tile) load_item(n, n);
#pragma unroll
    for (int n = 0; n < DM_BUFS; ++n) cp_async_commit();
  }

  float o_acc[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) { o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float cap2 = softcap > 0.f ? 2.f * LOG2E / softcap : 0.f;

  int buf = 0;                                                     // buffer of the item in use: item n is in n % DM_BUFS
  for (int it = 0; it < n_mine; ++it) {
    const int tile = warp + it * DM_WARPS;
    // ---- the keys of the tile: item 2 it, its group and at most two younger ones are outstanding -----------------------
    cp_async_wait<DM_BUFS - 1>();
    __syncwarp();
    const __nv_bfloat16* k_s = my + (size_t)buf * TILE;
    const int j0 = k_begin + tile * DM_KEYS;

    // two accumulators per 8 keys (even and odd steps along the head), so that the chain of dependent MMAs is half as long
    float s_acc[2][4], s_odd[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f;
      s_odd[n][0] = s_odd[n][1] = s_odd[n][2] = s_odd[n][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < KS_QK; ++ks) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, tile_ptr<D>(sQ, lane & 15, ks * 2 + (lane >> 4)));
      ldmatrix_x4(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(k_s), (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
      if (ks & 1) {
        mma_bf16(s_odd[0], a, b[0], b[1]);
        mma_bf16(s_odd[1], a, b[2], b[3]);
      } else {
        mma_bf16(s_acc[0], a, b[0], b[1]);
        mma_bf16(s_acc[1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s_acc[n][e] += s_odd[n][e];
    }
    __syncwarp();                                                  // every lane has read the keys: their buffer takes item 2 it + 3
    if (2 * it + DM_BUFS < n_loads) load_item(2 * it + DM_BUFS, buf);
    cp_async_commit();
    buf = buf + 1 == DM_BUFS ? 0 : buf + 1;
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int j = j0 + n * 8 + tq * 2 + (e & 1);
        float s = s_acc[n][e] * scale;
        if (softcap > 0.f) {
          const float ex = exp2f(s * cap2);
          s = softcap * (1.f - __fdividef(2.f, ex + 1.f));
        }
        s = (j < k_end) ? s * LOG2E : -INFINITY;
        s_acc[n][e] = s;
        m_new[r] = fmaxf(m_new[r], s);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
      m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
      corr[r] = (m_new[r] == -INFINITY) ? 1.f : exp2f(m_run[r] - m_new[r]);
      m_run[r] = m_new[r];
    }
    float l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = (m_new[r] == -INFINITY) ? 0.f : exp2f(s_acc[n][e] - m_new[r]);
        s_acc[n][e] = p;
        l_add[r] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + l_add[r];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      o_acc[n][0] *= corr[0]; o_acc[n][1] *= corr[0];
      o_acc[n][2] *= corr[1]; o_acc[n][3] *= corr[1];
    }
    uint32_t a[4];
    a[0] = pack_bf16(s_acc[0][0], s_acc[0][1]);
    a[1] = pack_bf16(s_acc[0][2], s_acc[0][3]);
    a[2] = pack_bf16(s_acc[1][0], s_acc[1][1]);
    a[3] = pack_bf16(s_acc[1][2], s_acc[1][3]);
    // ---- the values of the tile: item 2 it + 1 ----------------------------------------------------------------------
    cp_async_wait<DM_BUFS - 1>();
    __syncwarp();
    const __nv_bfloat16* v_s = my + (size_t)buf * TILE;
#pragma unroll
    for (int np = 0; np < NT_O / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(v_s), (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
      mma_bf16(o_acc[2 * np], a, b[0], b[1]);
      mma_bf16(o_acc[2 * np + 1], a, b[2], b[3]);
    }
    __syncwarp();                                                  // the values' buffer takes item 2 it + 4
    if (2 * it + 1 + DM_BUFS < n_loads) load_item(2 * it + 1 + DM_BUFS, buf);
    cp_async_commit();
    buf = buf + 1 == DM_BUFS ? 0 : buf + 1;
  }
  cp_async_wait<0>();
  // ---- merge the warps through shared memory (the tile buffers are free now) ---------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  __syncthreads();
  float* sm_o = reinterpret_cast<float*>(sKV);                     // [warp][G][D]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + r * 8;
    if (row < G) {
#pragma unroll
      for (int n = 0; n < NT_O; ++n) {
        float* dst = sm_o + ((size_t)warp * G + row) * D + n * 8 + tq * 2;
        dst[0] = o_acc[n][2 * r];
        dst[1] = o_acc[n][2 * r + 1];
      }
      if (tq == 0) { sm_ml[warp][row][0] = m_run[r]; sm_ml[warp][row][1] = l_run[r]; }
    }
  }
  __syncthreads();
  const size_t rec_base = (((size_t)t * nh + h_first) * n_splits + split) * PSTRIDE;
  for (int e = tid; e < G * D; e += blockDim.x) {
    const int h = e / D, i = e - h * D;
    float m = -INFINITY;
    for (int w = 0; w < DM_WARPS; ++w) m = fmaxf(m, sm_ml[w][h][0]);
    float l = 0.f, a = 0.f;
    for (int w = 0; w < DM_WARPS; ++w) {
      const float mw = sm_ml[w][h][0];
      const float c = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      l += sm_ml[w][h][1] * c;
      a += sm_o[((size_t)w * G + h) * D + i] * c;
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
  __threadfence();
  __syncthreads();
  const int cidx = item * nkv + kvh;
  if (tid == 0) s_last = (atomicAdd(&counters[cidx], 1) == n_splits - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();                                               // maxima here are base-2 scaled
  merge_splits<D, true>(partial, ((size_t)t * nh + h_first) * n_splits, G, n_splits, orow + (size_t)h_first * D);
  if (tid == 0) counters[cidx] = 0;
}

// Blocks of the tensor-core decode kernel that one SM holds at a time (shared memory or registers, whichever binds), as
// the runtime reports it; also sets the kernel's shared-memory limit.  0 if that fails.
template <int D>
int decode_mma_blocks_per_sm() {
  static int cached = -1;
  if (cached >= 0) return cached;
  const size_t smem = (size_t)(16 * D + DM_WARPS * DM_BUFS * DM_KEYS * D) * 2;
  int n = 0;
  if (cudaFuncSetAttribute(attn_decode_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_mma_kernel<D>, DM_WARPS * 32, smem) != cudaSuccess) {
    kf_record_cuda_error(cudaGetLastError());
    return 0;
  }
  cached = n;
  return n;
}

template <int D>
int launch_decode_mma(const float* qkv, const float* cos_t, const float* sin_t, int rot, int write_kv,
                      const void* q, const void* pages, const int* items, int n_items, const int* positions,
                      const int* row_req, const int* table, int table_stride, int page_size, int nh, int nkv, float scale,
                      float softcap, int window, int n_splits, float* partial, int* counters, void* out, cudaStream_t stream) {
  const size_t smem = (size_t)(16 * D + DM_WARPS * DM_BUFS * DM_KEYS * D) * 2;
  if (decode_mma_blocks_per_sm<D>() < 1) return KF_ERR_SETUP;
  kf_launch(attn_decode_mma_kernel<D>, dim3(n_items * nkv, n_splits), dim3(DM_WARPS * 32), smem, stream,
            (const __nv_bfloat16*)q, qkv, cos_t, sin_t, rot, write_kv, (__nv_bfloat16*)const_cast<void*>(pages), items, n_items,
            positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, n_splits, partial, counters,
            (__nv_bfloat16*)out);
  KF_CHECK_LAUNCH();
  return KF_OK;
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

// The tensor-core variant: ht = 0 selects it in kf_attention_decode.  It takes groups of up to 16 query heads.
static int g_forced_splits = 0;
#ifdef KF_TUNING
// Measurement hook of a tuning build: a fixed number of splits for the tensor-core decode kernel (0: the planner's choice).
KF_API void kf_set_attention_decode_splits(int splits) { g_forced_splits = splits; }
#endif

KF_API int kf_attention_decode_mma_plan(int n_items, int nh, int nkv, int d, int max_keys, int* splits_out) {
  if (g_forced_splits > 0) { *splits_out = g_forced_splits; return KF_OK; }
  const long blocks = (long)n_items * nkv;
  // fill one wave: as many splits as resident blocks allow
  long per_sm = d == 256 ? decode_mma_blocks_per_sm<256>() : d == 128 ? decode_mma_blocks_per_sm<128>()
              : d == 64 ? decode_mma_blocks_per_sm<64>() : d == 32 ? decode_mma_blocks_per_sm<32>()
              : d == 16 ? decode_mma_blocks_per_sm<16>() : 0;
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  int splits = (int)((kf_sm_count() * per_sm) / blocks);
  const int by_len = (max_keys + 255) / 256;
  if (splits > by_len) splits = by_len;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  *splits_out = splits;
  return KF_OK;
}

KF_API int kf_attention_decode_supported(int d) { return d == 16 || d == 32 || d == 64 || d == 128 || d == 256; }

// Heads per block and the number of counters / partial floats a launch needs.
KF_API int kf_attention_decode_plan(int n_items, int nh, int nkv, int d, int max_keys, int* ht_out, int* splits_out) {
  const int G = nh / nkv;
  const int ht = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
  const long blocks = (long)n_items * nkv * kf_ceil_div(G, ht);
  // two blocks of this kernel are resident per SM: fill one wave of two blocks per SM, never a second partial wave
  int splits = (int)((2 * kf_sm_count()) / blocks);
  const int by_len = (max_keys + 255) / 256;                  // at least 256 keys per split
  if (splits > by_len) splits = by_len;
  if (splits > 32) splits = 32;
  if (splits < 1) splits = 1;
  *ht_out = ht;
  *splits_out = splits;
  return KF_OK;
}

// q, out: [T, nh*d] bfloat16.  items: rows of the step this launch handles (null = rows 0..n_items-1).
// partial: n_rows_total * nh * splits * (d + 4) floats; counters: n_items * nkv * ceil(G/ht) zeroed ints (left zero).
KF_API int kf_attention_decode(const void* q, void* out, const void* pages, const int* items, int n_items,
                               const int* positions, const int* row_req, const int* table, int table_stride,
                               int page_size, int nh, int nkv, int d, float scale, float softcap, int window, int ht,
                               int n_splits, float* partial, int* counters, cudaStream_t stream) {
  if (n_items <= 0) return KF_OK;
  if (nkv < 1 || nh % nkv != 0 || page_size < 1 || n_splits < 1) return KF_ERR_SIZE;
  if (n_splits > 1 && (!partial || !counters)) return KF_ERR_SIZE;
  if (n_splits > MERGE_MAX_SPLITS || ht > MERGE_MAX_HEADS) return KF_ERR_SIZE;
  if (ht == 0) {                                     // tensor-core variant
    if (nh / nkv > 16) return KF_ERR_SIZE;
#define KF_MMA_ARGS nullptr, nullptr, nullptr, 0, 0, q, pages, items, n_items, positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, n_splits, partial, counters, out, stream
    switch (d) {
      case 16: return launch_decode_mma<16>(KF_MMA_ARGS);
      case 32: return launch_decode_mma<32>(KF_MMA_ARGS);
      case 64: return launch_decode_mma<64>(KF_MMA_ARGS);
      case 128: return launch_decode_mma<128>(KF_MMA_ARGS);
      case 256: return launch_decode_mma<256>(KF_MMA_ARGS);
    }
#undef KF_MMA_ARGS
    return KF_ERR_SIZE;
  }
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

// The tensor-core decode kernel with the rotation of q and k and the append of k and v done inside it: `qkv` is the
// 32-bit [T, (nh + 2 nkv) d] result of the stacked product, cos_t / sin_t the step's [T, rot/2] tables (null when rot is
// 0).  Every row handled must be the only row of its request at the request's last position (a decode row).
KF_API int kf_attention_decode_fused(const float* qkv, const float* cos_t, const float* sin_t, int rot, int write_kv, void* out,
                                     void* pages, const int* items, int n_items, const int* positions, const int* row_req,
                                     const int* table, int table_stride, int page_size, int nh, int nkv, int d, float scale,
                                     float softcap, int window, int n_splits, float* partial, int* counters,
                                     cudaStream_t stream) {
  if (n_items <= 0) return KF_OK;
  if (!qkv || nkv < 1 || nh % nkv != 0 || nh / nkv > 16 || page_size < 1 || n_splits < 1) return KF_ERR_SIZE;
  if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && (!cos_t || !sin_t))) return KF_ERR_SIZE;
  if (n_splits > 1 && (!partial || !counters)) return KF_ERR_SIZE;
  if (n_splits > MERGE_MAX_SPLITS) return KF_ERR_SIZE;
#define KF_MMA_ARGS qkv, cos_t, sin_t, rot, write_kv, nullptr, pages, items, n_items, positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, n_splits, partial, counters, out, stream
  switch (d) {
    case 16: return launch_decode_mma<16>(KF_MMA_ARGS);
    case 32: return launch_decode_mma<32>(KF_MMA_ARGS);
    case 64: return launch_decode_mma<64>(KF_MMA_ARGS);
    case 128: return launch_decode_mma<128>(KF_MMA_ARGS);
    case 256: return launch_decode_mma<256>(KF_MMA_ARGS);
  }
#undef KF_MMA_ARGS
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

// The size rule of kf_attention_decode_static for a launch of `splits` key splits with `ht` heads per block: KF_OK if the
// built-in arrays hold its partial results and counters (one split needs neither), else KF_ERR_SIZE with a message.
KF_API int kf_attention_decode_static_fits(int n_rows, int nh, int nkv, int d, int ht, int splits) {
  if (n_rows < 0 || nkv < 1 || nh % nkv != 0 || ht < 1 || splits < 1 || !kf_attention_decode_supported(d)) return KF_ERR_SIZE;
  if (splits == 1) return KF_OK;
  const long n_counters = (long)n_rows * nkv * kf_ceil_div(nh / nkv, ht);
  const long n_partial = (long)n_rows * nh * splits * (d + 4);
  if (n_counters > KF_DECODE_STATIC_MAX_COUNTERS || n_partial > KF_DECODE_STATIC_MAX_PARTIAL_FLOATS) {
    kf_record_message("kf_attention_decode_static: rows * heads * splits * (head_dim + 4) exceeds the built-in scratch");
    return KF_ERR_SIZE;
  }
  return KF_OK;
}

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
  if (kf_attention_decode_static_fits(n_rows, nh, nkv, d, ht, splits) != KF_OK) return KF_ERR_SIZE;
  if (splits > 1) {                     // with one split the kernel writes its result directly and touches neither array
    // The arrays keep what the last call left; the counters must start at zero.
    const long n_counters = (long)n_rows * nkv * kf_ceil_div(nh / nkv, ht);
    if (cudaMemsetAsync(counters, 0, (size_t)n_counters * sizeof(int), stream) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_LAUNCH;
    }
  }
  return kf_attention_decode(q, out, pages, nullptr, n_rows, positions, row_req, table, table_stride, page_size, nh, nkv,
                             d, scale, softcap, window, ht, splits, partial, counters, stream);
}
