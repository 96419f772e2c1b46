// Sampling support on the device: greedy argmax, and the top-k candidates with the row's log-sum-exp.
//
// argmax: the first maximum wins (reference: crates/kf-engine/src/sampler.rs:219-227).
// top-k: ids by falling value, the lower id first among equals, plus lse = m + ln sum exp(x - m)
// (reference: crates/kf-backend-cpu/src/ops.rs:168-195; the device version there is a radix select,
// crates/kf-backend-cuda/src/kernels/sample.cu:194-320).  Here one block per row selects the k-th largest
// key by four 8-bit radix passes over an order-preserving 32-bit image of the value, then gathers and
// ranks the survivors in shared memory.
#include "common.cuh"

__device__ __forceinline__ unsigned kf_orderable(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);      // larger float <=> larger unsigned
}

// Block-wide (value, index) maximum with the lower index winning ties; result valid in thread 0.
__device__ __forceinline__ void block_argmax(float& best, int& bi, float* sv, int* si) {
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nwarp ? sv[lane] : -INFINITY;
    bi = lane < nwarp ? si[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
  }
}

// Stage 1: block (chunk, row) scans its slice of the row.  With one chunk it writes the answer itself.
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, int chunks,
                              float* __restrict__ part_val, int* __restrict__ part_idx) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.y, chunk = blockIdx.x;
  const float* r = logits + (size_t)row * V;
  const int per = (V + chunks - 1) / chunks;
  const int begin = chunk * per, end = min(V, begin + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = r[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  block_argmax(best, bi, sv, si);
  if (threadIdx.x == 0) {
    if (chunks == 1) out[row] = bi == 0x7fffffff ? 0 : bi;
    else { part_val[row * chunks + chunk] = best; part_idx[row * chunks + chunk] = bi; }
  }
}

// Stage 2: one warp per row merges the chunks in index order.
__global__ void argmax_merge_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    int* __restrict__ out, int chunks) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += 32) {
    const float v = part_val[row * chunks + c];
    const int i = part_idx[row * chunks + c];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

// scratch: rows * 64 floats followed by rows * 64 ints (may be null when V < 16384: one chunk is used).
KF_API int kf_argmax(const float* logits, int* out, int rows, int V, float* scratch, cudaStream_t stream) {
  if (rows <= 0) return KF_OK;
  if (V <= 0) return KF_ERR_SIZE;
  int chunks = (scratch && V >= 16384) ? 64 : 1;
  float* pv = scratch;
  int* pi = scratch ? (int*)(scratch + (size_t)rows * 64) : nullptr;
  kf_launch(argmax_kernel, dim3(chunks, rows), dim3(chunks == 1 ? 1024 : 256), 0, stream, logits, out, V, chunks, pv, pi);
  KF_CHECK_LAUNCH();
  if (chunks > 1) {
    kf_launch(argmax_merge_kernel, dim3(rows), dim3(32), 0, stream, pv, pi, out, chunks);
    KF_CHECK_LAUNCH();
  }
  return KF_OK;
}

constexpr int TOPK_MAX = 128;
constexpr int TOPK_THREADS = 1024;

// out_ids[row, k], out_vals[row, k], out_lse[row]
__global__ void __launch_bounds__(TOPK_THREADS)
topk_lse_kernel(const float* __restrict__ logits, int* __restrict__ out_ids, float* __restrict__ out_vals,
                float* __restrict__ out_lse, int V, int k) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ unsigned hist[256];
  __shared__ float red[33];
  __shared__ unsigned s_prefix, s_mask;
  __shared__ int s_need, s_count, s_ties_taken;
  __shared__ float cv[TOPK_MAX];
  __shared__ int ci[TOPK_MAX];
  const float* row = logits + (size_t)blockIdx.x * V;
  const int tid = threadIdx.x;

  // ---- log-sum-exp -------------------------------------------------------------------------------
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = kf_warp_max(mx);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid < 32) {
    float t = tid < (blockDim.x >> 5) ? red[tid] : -INFINITY;
    t = kf_warp_max(t);
    if (tid == 0) red[32] = t;
  }
  __syncthreads();
  mx = red[32];
  float sum = 0.f;
  for (int i = tid; i < V; i += blockDim.x) sum += expf(row[i] - mx);
  sum = kf_block_sum(sum, red);
  if (tid == 0) out_lse[blockIdx.x] = mx + logf(sum);

  // ---- radix select of the k-th largest key ------------------------------------------------------------
  if (tid == 0) { s_prefix = 0u; s_mask = 0u; s_need = k; }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix, mask = s_mask;
    for (int i = tid; i < V; i += blockDim.x) {
      const unsigned key = kf_orderable(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need;
      int b = 255;
      for (; b > 0; --b) {
        if ((int)hist[b] >= need) break;
        need -= (int)hist[b];
      }
      s_need = need;                                       // how many keys with this digit are still wanted
      s_prefix = prefix | ((unsigned)b << shift);
      s_mask = mask | (255u << shift);
    }
    __syncthreads();
  }
  const unsigned kth = s_prefix;                           // key of the k-th largest element
  const int ties_wanted = s_need;                          // elements equal to it that belong to the top k
  if (tid == 0) { s_count = 0; s_ties_taken = 0; }
  __syncthreads();
  // strictly greater keys: all of them (there are k - ties_wanted)
  for (int i = tid; i < V; i += blockDim.x) {
    const float v = row[i];
    if (kf_orderable(v) > kth) {
      const int slot = atomicAdd(&s_count, 1);
      if (slot < TOPK_MAX) { cv[slot] = v; ci[slot] = i; }
    }
  }
  __syncthreads();
  // equal keys: the lowest ids win.  Walk the row in blocks of blockDim.x in ascending order.
  const int base_count = s_count;
  for (int i0 = 0; i0 < V && s_ties_taken < ties_wanted; i0 += blockDim.x) {
    const int i = i0 + tid;
    const bool eq = i < V && kf_orderable(row[i]) == kth;
    // rank of this thread among the equal ones of this block of ids
    const unsigned ballot = __ballot_sync(0xffffffffu, eq);
    __shared__ int warp_cnt[32];
    if ((tid & 31) == 0) warp_cnt[tid >> 5] = __popc(ballot);
    __syncthreads();
    int before = s_ties_taken;
    for (int wdx = 0; wdx < (tid >> 5); ++wdx) before += warp_cnt[wdx];
    before += __popc(ballot & ((1u << (tid & 31)) - 1u));
    if (eq && before < ties_wanted) { cv[base_count + before] = row[i]; ci[base_count + before] = i; }
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int wdx = 0; wdx < (int)(blockDim.x >> 5); ++wdx) tot += warp_cnt[wdx];
      s_ties_taken = min(ties_wanted, s_ties_taken + tot);
    }
    __syncthreads();
  }
  // ---- rank the k survivors: falling value, lower id first among equals -----------------------------------
  if (tid < k) {
    const float v = cv[tid];
    const int id = ci[tid];
    int rank = 0;
    for (int j = 0; j < k; ++j) {
      const float vj = cv[j];
      const int ij = ci[j];
      if (vj > v || (vj == v && ij < id)) ++rank;
    }
    out_ids[(size_t)blockIdx.x * k + rank] = id;
    out_vals[(size_t)blockIdx.x * k + rank] = v;
  }
}

// k <= 128 and k <= V.  Values must not be NaN.
KF_API int kf_topk_lse(const float* logits, int* out_ids, float* out_vals, float* out_lse, int rows, int V, int k,
                       cudaStream_t stream) {
  if (rows <= 0) return KF_OK;
  if (k < 1 || k > TOPK_MAX || k > V) return KF_ERR_SIZE;
  kf_launch(topk_lse_kernel, dim3(rows), dim3(TOPK_THREADS), 0, stream, logits, out_ids, out_vals, out_lse, V, k);
  KF_CHECK_LAUNCH();
  return KF_OK;
}
