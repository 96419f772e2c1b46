// Sampling on the device: the greedy argmax, the top candidates of a row with its log-sum-exp, and the whole draw
// (repeat penalty, temperature, top-k, min-p, top-p, the generator) from per-request state that lives on the device.
//
// Rules and their order are the reference's (crates/kf-engine/src/sampler.rs:37-100): the penalty divides positive and
// multiplies negative logits of the last `repeat_window` tokens; temperature <= 0 takes the first maximum (:219-227);
// else tokens are ranked by falling logit, the lower id first among equals; the first top_k stay (0: all);
// w = exp((l - max) / T); min-p keeps w >= min_p w_max; top-p keeps the shortest prefix whose mass reaches top_p of
// the top-k mass; r = next_f32() times the kept mass, and the walk down the ranking stops at the first token whose
// running mass exceeds r.  The generator is xorshift64 (:20-34).  Masses are summed in 64-bit here (the reference
// sums 32-bit numbers one after the other on the host), so that the result does not depend on how a row is cut.
//
// Shape.  A row is read ONCE: blocks (slice, row) of 4,096 columns apply the penalty, take the slice's maximum and
// sum of exponentials (for the log-sum-exp) and select its 64 largest keys in shared memory; one block per row then
// selects the 64 largest of those, ranks them, and draws.  The reference cuts a row into slices for the same reason
// (crates/kf-backend-cuda/src/kernels/sample.cu:194-320: at most 16 slices of about 8,192 columns, then a merge).
// A key is 64 bits, (order-preserving image of the value) << 32 | ~id: no two keys are equal, a larger key ranks first,
// and selection is an 8-bit radix walk from the top byte with no special case for equal values.
// Rows whose rules reach below the 64th candidate (top_k of 0 or more than 64, at a temperature above 0) are finished
// by a third kernel that answers "where in the ranking does the running mass (or count) reach x" by the same radix
// walk over the whole row, its histogram bins holding 64-bit masses.
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


// ---- keys ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long kf_key(float v, unsigned id) {
  if (v == 0.f) v = 0.f;                                 // -0 and +0 are one value: the lower id ranks first among them
  return ((unsigned long long)kf_orderable(v) << 32) | (unsigned long long)(0xFFFFFFFFu - id);
}
__device__ __forceinline__ float kf_key_value(unsigned long long key) {
  const unsigned o = (unsigned)(key >> 32);
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o);
}
__device__ __forceinline__ int kf_key_id(unsigned long long key) { return (int)(0xFFFFFFFFu - (unsigned)(key & 0xFFFFFFFFull)); }

__device__ __forceinline__ float kf_penalized(float v, float penalty) { return v > 0.f ? v / penalty : v * penalty; }

// Per-request sampler state, 32-bit words (kungfu_b200/sampling/sampler.py packs it):
//  [0,1] generator state  [2] temperature  [3] top_p  [4] min_p  [5] repeat_penalty  [6] top_k  [7] repeat_window
//  [8] tokens recorded so far  [16..272) the last 256 of them, token i at 16 + i % 256
constexpr int ST_WORDS = 272, ST_RNG = 0, ST_TEMP = 2, ST_TOP_P = 3, ST_MIN_P = 4, ST_PENALTY = 5, ST_TOP_K = 6,
              ST_WINDOW = 7, ST_COUNT = 8, ST_RING = 16, RING = 256;
constexpr int CAND = 64;               // candidates kept per slice and per row (reference: TOP = 64, session.rs:80)
constexpr int SLICE = 4096;            // columns per block of the first kernel
constexpr int SL_THREADS = 256;
constexpr int SL_CAND_MAX = 1024;      // keys of a slice that can still be among its 64 largest, after the bound (a list in shared memory)
constexpr int MG_THREADS = 1024;        // the second kernel: one block per row, its loads from L2 are the cost

__device__ __forceinline__ float st_f(const int* st, int w) { return __int_as_float(st[w]); }

// Among `n` 64-bit keys in shared memory (all different, or zero for "absent"), a threshold that exactly `want` keys
// reach: an 8-bit radix walk from the top byte, which ends as soon as a bin is wanted whole (the threshold is then that
// bin's lowest possible key, not a key of the set).  Called by all threads of a block (a multiple of 32, at least 256); hist: 256 ints,
// sh: 1 u64 + 1 int.  Returns 0 when fewer than `want` keys are present.  Logits of one row share their top bytes, so
// a warp first finds which of its lanes hold the same bin and adds to the histogram once per bin.
__device__ __forceinline__ unsigned long long select_key(const unsigned long long* keys, int n, int want, int* hist,
                                                         unsigned long long* sh_prefix, int* sh_need) {
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid == 0) { *sh_prefix = 0ull; *sh_need = want; }
  __syncthreads();
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (int b = tid; b < 256; b += blockDim.x) hist[b] = 0;
    __syncthreads();
    const unsigned long long prefix = *sh_prefix;
    const unsigned long long mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
    for (int i0 = 0; i0 < n; i0 += blockDim.x) {
      const int i = i0 + tid;
      const unsigned long long k = i < n ? keys[i] : 0ull;
      const bool in = k != 0ull && (k & mask) == prefix;
      const unsigned act = __ballot_sync(0xffffffffu, in);
      if (in) {
        const int bin = (int)((k >> shift) & 255ull);
        const unsigned same = __match_any_sync(act, bin);
        if (lane == __ffs(same) - 1) atomicAdd(&hist[bin], __popc(same));
      }
    }
    __syncthreads();
    if (tid < 32) {                                       // warp 0: bins 255 down to 0, eight per lane
      const int need = *sh_need;
      int mine[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[j] = hist[255 - (tid * 8 + j)]; sum += mine[j]; }
      int incl = sum;                                     // inclusive scan over lanes (lane 0 holds the highest bins)
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += t;
      }
      int above = incl - sum;                             // keys in higher bins than this lane's
      int found = -1, found_need = 0;
      bool whole = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (found < 0 && above + mine[j] >= need && above < need) {
          found = 255 - (tid * 8 + j);
          found_need = need - above;
          whole = found_need == mine[j];
        }
        above += mine[j];
      }
      const unsigned who = __ballot_sync(0xffffffffu, found >= 0);
      if (who == 0u) { if (tid == 0) *sh_need = -1; }     // fewer keys than wanted
      else if (tid == __ffs(who) - 1) {
        *sh_prefix = prefix | ((unsigned long long)found << shift);
        *sh_need = whole ? 0 : found_need;                // 0: every key of that bin is wanted, the walk is over
      }
    }
    __syncthreads();
    if (*sh_need < 0) return 0ull;
    if (*sh_need == 0) break;
  }
  return *sh_prefix;
}

// ---- kernel 1: one slice of one row -----------------------------------------------------------------------------------
// out_keys [rows, n_slices, 64] (zero = absent), out_stats [rows, n_slices, 2] = (maximum, sum of exp(v - maximum)) of the
// slice BEFORE the penalty (only when `need_stats`).  states may be null (no penalty); slot_rows etc. as in kf_sample.
// A row whose request takes the best token (temperature <= 0) needs one key per slice, unless `rank_all` (the caller
// wants the ranked candidates themselves).
__device__ __forceinline__ const int* row_state(int row, const int* logit_rows, const int* row_req, const int* req_slot,
                                                const int* states) {
  if (states == nullptr) return nullptr;
  const int lr = logit_rows ? logit_rows[row] : row;
  const int rq = row_req ? row_req[lr] : 0;
  if (rq < 0) return nullptr;
  return states + (size_t)(req_slot ? req_slot[rq] : rq) * ST_WORDS;
}

__global__ void __launch_bounds__(SL_THREADS)
sample_slices_kernel(const float* __restrict__ logits, int V, int n_slices, const int* __restrict__ logit_rows,
                     const int* __restrict__ row_req, const int* __restrict__ req_slot, const int* __restrict__ states,
                     unsigned long long* __restrict__ out_keys, float* __restrict__ out_stats, int need_stats, int rank_all) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ unsigned long long keys[SLICE];
  __shared__ float red[33];
  __shared__ int hist[256];
  __shared__ unsigned long long sh_prefix;
  __shared__ int sh_need, sh_count;
  const int row = blockIdx.y, slice = blockIdx.x, tid = threadIdx.x;
  const int c0 = slice * SLICE, n = min(SLICE, V - c0);
  const float* src = logits + (size_t)row * V + c0;
  float* vals = reinterpret_cast<float*>(keys);           // the values sit in the lower half until the keys are made
  const int* st = row_state(row, logit_rows, row_req, req_slot, states);
  const bool best_only = !rank_all && st != nullptr && st_f(st, ST_TEMP) <= 0.f;
  float mx = -INFINITY;
  {
    float r[SLICE / SL_THREADS];                          // every load of the thread in flight at once
#pragma unroll
    for (int j = 0; j < SLICE / SL_THREADS; ++j) { const int i = tid + j * SL_THREADS; r[j] = i < n ? src[i] : -INFINITY; }
#pragma unroll
    for (int j = 0; j < SLICE / SL_THREADS; ++j) {
      const int i = tid + j * SL_THREADS;
      if (i < n) { vals[i] = r[j]; mx = fmaxf(mx, r[j]); }
    }
  }
  if (need_stats) {
    mx = kf_warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
      float t = tid < SL_THREADS / 32 ? red[tid] : -INFINITY;
      t = kf_warp_max(t);
      if (tid == 0) red[32] = t;
    }
    __syncthreads();
    mx = red[32];
    float sum = 0.f;
    for (int i = tid; i < n; i += SL_THREADS) sum += expf(vals[i] - mx);
    sum = kf_block_sum(sum, red);
    if (tid == 0) {
      out_stats[((size_t)row * n_slices + slice) * 2] = mx;
      out_stats[((size_t)row * n_slices + slice) * 2 + 1] = sum;
    }
  }
  __syncthreads();
  // the repeat penalty on this slice's columns (one thread: at most 256 tokens, applied as often as they occur)
  if (st != nullptr && tid == 0) {
    const float pen = st_f(st, ST_PENALTY);
    if (pen != 1.f) {
      const int count = st[ST_COUNT], window = min(min(st[ST_WINDOW], RING), count);
      for (int j = count - window; j < count; ++j) {
        const int t = st[ST_RING + (j & (RING - 1))] - c0;
        if (t >= 0 && t < n) vals[t] = kf_penalized(vals[t], pen);
      }
    }
  }
  __syncthreads();
  unsigned long long* dst = out_keys + ((size_t)row * n_slices + slice) * CAND;
  if (best_only) {                                        // the slice's best key and 63 absent ones
    unsigned long long best = 0ull;
    for (int i = tid; i < n; i += SL_THREADS) {
      const unsigned long long k = kf_key(vals[i], (unsigned)(c0 + i));
      best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    __syncthreads();                                      // everyone has read its values: the keys' array is free
    if ((tid & 31) == 0) keys[SLICE - 1 - (tid >> 5)] = best;
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < SL_THREADS / 32; ++w) { const unsigned long long other = keys[SLICE - 1 - w]; best = other > best ? other : best; }
      dst[0] = best;
    } else if (tid < CAND) {
      dst[tid] = 0ull;
    }
    return;
  }
  // values -> keys: the keys overwrite the values, so every thread first takes its values into registers
  {
    float mine[SLICE / SL_THREADS];
#pragma unroll
    for (int j = 0; j < SLICE / SL_THREADS; ++j) { const int i = tid + j * SL_THREADS; mine[j] = i < n ? vals[i] : 0.f; }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < SLICE / SL_THREADS; ++j) {
      const int i = tid + j * SL_THREADS;
      keys[i] = i < n ? kf_key(mine[j], (unsigned)(c0 + i)) : 0ull;
    }
    __syncthreads();
  }
  // The slice's 64 largest keys.  A walk over all 4,096 keys is most of this kernel's time, so first a bound: every thread
  // takes the largest of its sixteen keys; the 64th largest of those 256 is reached by at least 64 keys of the slice, so
  // only keys that reach it can be among the 64 largest.  Usually that leaves a hundred or two, and the exact walk runs
  // over them; if it leaves more than the list holds (keys in falling order thread by thread), over everything.
  __shared__ unsigned long long cand[SL_CAND_MAX];
  unsigned long long mine[SLICE / SL_THREADS], lmax = 0ull;
#pragma unroll
  for (int j = 0; j < SLICE / SL_THREADS; ++j) { mine[j] = keys[tid + j * SL_THREADS]; lmax = mine[j] > lmax ? mine[j] : lmax; }
  cand[tid] = lmax;                                       // SL_CAND_MAX >= SL_THREADS
  if (tid == 0) sh_count = 0;
  __syncthreads();
  const unsigned long long bound = select_key(cand, SL_THREADS, CAND, hist, &sh_prefix, &sh_need);   // 0: fewer than 64 non-empty threads
  __syncthreads();
  int n_mine = 0;
#pragma unroll
  for (int j = 0; j < SLICE / SL_THREADS; ++j) n_mine += (mine[j] != 0ull && mine[j] >= bound) ? 1 : 0;
  int at = n_mine ? atomicAdd(&sh_count, n_mine) : 0;
  __syncthreads();
  const int n_cand = sh_count;
  const bool listed = n_cand <= SL_CAND_MAX;
  if (listed) {
#pragma unroll
    for (int j = 0; j < SLICE / SL_THREADS; ++j)
      if (mine[j] != 0ull && mine[j] >= bound) cand[at++] = mine[j];
  }
  __syncthreads();
  const unsigned long long* pool = listed ? cand : keys;
  const int n_pool = listed ? n_cand : SLICE;
  const unsigned long long kth = select_key(pool, n_pool, CAND, hist, &sh_prefix, &sh_need);
  if (tid == 0) sh_count = 0;
  __syncthreads();
  for (int i = tid; i < n_pool; i += SL_THREADS) {
    const unsigned long long k = pool[i];
    if (k != 0ull && k >= kth) {                          // kth = 0: fewer than 64 columns, all of them
      const int where = atomicAdd(&sh_count, 1);
      if (where < CAND) dst[where] = k;
    }
  }
  __syncthreads();
  for (int i = sh_count + tid; i < CAND; i += SL_THREADS) dst[i] = 0ull;
}

// xorshift64 and its 24-bit fraction (sampler.rs:20-34)
__device__ __forceinline__ float next_f32(unsigned long long& x) {
  x ^= x << 13;
  x ^= x >> 7;
  x ^= x << 17;
  return (float)(unsigned)(x >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ void record_token(int* st, int token) {
  const int count = st[ST_COUNT];
  st[ST_RING + (count & (RING - 1))] = token;
  st[ST_COUNT] = count + 1;
}

// ---- kernel 2: one row: merge, rank, draw -----------------------------------------------------------------------------
// Dynamic shared memory: n_slices * 64 keys.  flags[row] = 1 when the row must be finished by the third kernel.
__global__ void __launch_bounds__(MG_THREADS)
sample_merge_kernel(const unsigned long long* __restrict__ slice_keys, const float* __restrict__ slice_stats, int n_slices,
                    int V, const int* __restrict__ logit_rows, const int* __restrict__ row_req,
                    const int* __restrict__ req_slot, int* __restrict__ states, int draw, int* __restrict__ out_ids,
                    int* __restrict__ cand_ids, float* __restrict__ cand_vals, float* __restrict__ cand_lse, int k_out,
                    int* __restrict__ flags) {
  kf_pdl_trigger();
  kf_pdl_wait();
  extern __shared__ unsigned long long all_keys[];
  __shared__ unsigned long long top[CAND];
  __shared__ unsigned long long ranked[CAND];
  __shared__ int hist[256];
  __shared__ unsigned long long sh_prefix;
  __shared__ int sh_need, sh_count;
  const int row = blockIdx.x, tid = threadIdx.x;
  const int n = n_slices * CAND;
  if (draw && cand_ids == nullptr && cand_lse == nullptr) {
    // a row that takes the best token: the first kernel left one key per slice
    int* st0 = const_cast<int*>(row_state(row, logit_rows, row_req, req_slot, states));
    if (st0 != nullptr && st_f(st0, ST_TEMP) <= 0.f) {
      if (tid >= 32) return;
      unsigned long long best = 0ull;
      for (int sl = tid; sl < n_slices; sl += 32) {
        const unsigned long long k = slice_keys[((size_t)row * n_slices + sl) * CAND];
        best = k > best ? k : best;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
      }
      if (tid == 0) {
        if (flags) flags[row] = 0;
        const int token = kf_key_id(best);
        out_ids[row] = token;
        record_token(st0, token);
      }
      return;
    }
  }
#pragma unroll 4
  for (int i = tid; i < n; i += MG_THREADS) all_keys[i] = slice_keys[(size_t)row * n + i];
  if (tid < CAND) { top[tid] = 0ull; ranked[tid] = 0ull; }
  __syncthreads();
  const int k = min(CAND, V);
  const unsigned long long kth = select_key(all_keys, n, k, hist, &sh_prefix, &sh_need);
  if (tid == 0) sh_count = 0;
  __syncthreads();
  for (int i = tid; i < n; i += MG_THREADS) {
    const unsigned long long key = all_keys[i];
    if (key != 0ull && key >= kth) {
      const int at = atomicAdd(&sh_count, 1);
      if (at < CAND) top[at] = key;
    }
  }
  __syncthreads();
  if (tid < CAND && top[tid] != 0ull) {                    // rank = number of larger keys
    int rank = 0;
    const unsigned long long mine = top[tid];
    for (int j = 0; j < CAND; ++j) rank += top[j] > mine ? 1 : 0;
    ranked[rank] = mine;
  }
  __syncthreads();
  if (cand_ids != nullptr && tid < k_out) {
    cand_ids[(size_t)row * k_out + tid] = kf_key_id(ranked[tid]);
    cand_vals[(size_t)row * k_out + tid] = kf_key_value(ranked[tid]);
  }
  if (cand_lse != nullptr && tid < 32) {
    float m = -INFINITY;
    for (int s = tid; s < n_slices; s += 32) m = fmaxf(m, slice_stats[((size_t)row * n_slices + s) * 2]);
    m = kf_warp_max(m);
    float sum = 0.f;
    for (int s = tid; s < n_slices; s += 32) {
      const float ms = slice_stats[((size_t)row * n_slices + s) * 2];
      sum += slice_stats[((size_t)row * n_slices + s) * 2 + 1] * expf(ms - m);
    }
    sum = kf_warp_sum(sum);
    if (tid == 0) cand_lse[row] = m + logf(sum);
  }
  if (!draw) return;
  __shared__ float w[CAND];                                // weights of the ranked candidates, one thread each
  {
    const int* st1 = row_state(row, logit_rows, row_req, req_slot, states);
    if (st1 != nullptr && tid < CAND) {
      const float t1 = st_f(st1, ST_TEMP);
      w[tid] = (t1 > 0.f && ranked[tid] != 0ull) ? expf((kf_key_value(ranked[tid]) - kf_key_value(ranked[0])) / t1) : 0.f;
    }
  }
  __syncthreads();
  if (tid != 0) return;
  if (flags) flags[row] = 0;
  const int lr = logit_rows ? logit_rows[row] : row;
  const int rq = row_req ? row_req[lr] : 0;
  if (rq < 0) { out_ids[row] = 0; return; }                // a padding row of a replayed graph
  int* st = states + (size_t)(req_slot ? req_slot[rq] : rq) * ST_WORDS;
  const float temp = st_f(st, ST_TEMP);
  const int top_k = st[ST_TOP_K];
  int token;
  if (temp <= 0.f) {
    token = kf_key_id(ranked[0]);
  } else if (top_k >= 1 && (top_k <= CAND || V <= CAND)) {
    const int n1 = min(min(top_k, k), V);
    const float min_p = st_f(st, ST_MIN_P), top_p = st_f(st, ST_TOP_P);
    double mass1 = 0.0;
    for (int i = 0; i < n1; ++i) mass1 += (double)w[i];
    int keep = n1;
    if (min_p > 0.f) {
      keep = 0;
      while (keep < n1 && w[keep] >= min_p) ++keep;         // w of the first is 1
      if (keep < 1) keep = 1;
    }
    if (top_p < 1.f) {
      double acc = 0.0;
      int m = 0;
      const double target = (double)top_p * mass1;
      while (m < keep) { acc += (double)w[m]; ++m; if (acc >= target) break; }
      keep = m;
    }
    double mass3 = 0.0;
    for (int i = 0; i < keep; ++i) mass3 += (double)w[i];
    unsigned long long x = ((unsigned long long)(unsigned)st[ST_RNG + 1] << 32) | (unsigned)st[ST_RNG];
    const double r = (double)next_f32(x) * mass3;
    st[ST_RNG] = (int)(unsigned)(x & 0xFFFFFFFFull);
    st[ST_RNG + 1] = (int)(unsigned)(x >> 32);
    double run = 0.0;
    int pick = keep - 1;
    for (int i = 0; i < keep; ++i) { run += (double)w[i]; if (r < run) { pick = i; break; } }
    token = kf_key_id(ranked[pick]);
  } else {
    if (flags) flags[row] = 1;                             // the third kernel draws (and records the token)
    return;
  }
  out_ids[row] = token;
  record_token(st, token);
}

// ---- kernel 3: rows whose rules reach below the 64th candidate ------------------------------------------------------------
// One block per flagged row.  `pen` [rows, V]: scratch for the row after the penalty.
constexpr int FULL_THREADS = 1024;

struct Located { unsigned long long key; double before; };   // the key at which the target is reached, mass (count) ranked before it

// Walk the ranking (falling key) of the kept set {key >= lo_key, w >= min_w} until the running mass (by_mass) or count
// reaches `target` (strictly exceeds it when `strict`); returns that key and what ranks before it.  If the whole set
// does not reach the target, the set's last key.  All threads call it; hist: 256 doubles.
__device__ Located locate(const float* __restrict__ pen, int V, float vmax, float temp, unsigned long long lo_key, float min_w,
                          double target, bool by_mass, bool strict, double* hist, unsigned long long* sh_prefix,
                          double* sh_before, int* sh_done) {
  const int tid = threadIdx.x;
  if (tid == 0) { *sh_prefix = 0ull; *sh_before = 0.0; *sh_done = 0; }
  __syncthreads();
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (int b = tid; b < 256; b += FULL_THREADS) hist[b] = 0.0;
    __syncthreads();
    const unsigned long long prefix = *sh_prefix;
    const unsigned long long mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
    for (int i = tid; i < V; i += FULL_THREADS) {
      const float v = pen[i];
      const unsigned long long key = kf_key(v, (unsigned)i);
      if (key < lo_key || (key & mask) != prefix) continue;
      const float w = expf((v - vmax) / temp);
      if (w < min_w) continue;
      atomicAdd(&hist[(int)((key >> shift) & 255ull)], by_mass ? (double)w : 1.0);
    }
    __syncthreads();
    if (tid == 0) {
      double before = *sh_before;
      int b = 255, last_nonempty = -1;
      bool hit = false;
      for (; b >= 0; --b) {
        if (hist[b] == 0.0) continue;
        last_nonempty = b;
        const double upto = before + hist[b];
        if (strict ? (upto > target) : (upto >= target)) { hit = true; break; }
        before = upto;
      }
      if (!hit) {                                         // the set ends before the target: its last key
        b = last_nonempty;
        if (b >= 0) before -= hist[b];
        *sh_done = 1;                                     // from here on: walk to the smallest key of the set
        target = 1e300;
      }
      if (b < 0) b = 0;
      *sh_prefix = prefix | ((unsigned long long)b << shift);
      *sh_before = before;
    }
    __syncthreads();
    if (*sh_done) {                                       // keep choosing the lowest non-empty bin
      strict = false;
      target = 1e300;
    }
  }
  Located out;
  out.key = *sh_prefix;
  out.before = *sh_before;
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(FULL_THREADS)
sample_full_kernel(const float* __restrict__ logits, int V, const int* __restrict__ logit_rows, const int* __restrict__ row_req,
                   const int* __restrict__ req_slot, int* __restrict__ states, const int* __restrict__ flags,
                   float* __restrict__ pen_all, int* __restrict__ out_ids) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ double hist[256];
  __shared__ double red[33];
  __shared__ unsigned long long sh_prefix;
  __shared__ double sh_before;
  __shared__ int sh_done;
  __shared__ float sh_vmax;
  const int row = blockIdx.x, tid = threadIdx.x;
  if (!flags[row]) return;
  const int lr = logit_rows ? logit_rows[row] : row;
  const int rq = row_req ? row_req[lr] : 0;
  if (rq < 0) return;
  int* st = states + (size_t)(req_slot ? req_slot[rq] : rq) * ST_WORDS;
  const float temp = st_f(st, ST_TEMP), top_p = st_f(st, ST_TOP_P), min_p = st_f(st, ST_MIN_P), penalty = st_f(st, ST_PENALTY);
  const int top_k = st[ST_TOP_K];
  const float* src = logits + (size_t)row * V;
  float* pen = pen_all + (size_t)row * V;
  for (int i = tid; i < V; i += FULL_THREADS) pen[i] = src[i];
  __syncthreads();
  if (tid == 0 && penalty != 1.f) {
    const int count = st[ST_COUNT], window = min(min(st[ST_WINDOW], RING), count);
    for (int j = count - window; j < count; ++j) {
      const int t = st[ST_RING + (j & (RING - 1))];
      if (t >= 0 && t < V) pen[t] = kf_penalized(pen[t], penalty);
    }
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int i = tid; i < V; i += FULL_THREADS) mx = fmaxf(mx, pen[i]);
  mx = kf_warp_max(mx);
  if ((tid & 31) == 0) red[tid >> 5] = (double)mx;
  __syncthreads();
  if (tid == 0) {
    float t = -INFINITY;
    for (int wdx = 0; wdx < FULL_THREADS / 32; ++wdx) t = fmaxf(t, (float)red[wdx]);
    sh_vmax = t;
  }
  __syncthreads();
  const float vmax = sh_vmax;
  // the first top_k of the ranking (all when top_k is 0): lo1 = the key of the last of them
  unsigned long long lo = 0ull;
  if (top_k > 0 && top_k < V)
    lo = locate(pen, V, vmax, temp, 0ull, 0.f, (double)top_k, false, false, hist, &sh_prefix, &sh_before, &sh_done).key;
  // their mass
  double part = 0.0;
  for (int i = tid; i < V; i += FULL_THREADS) {
    const float v = pen[i];
    if (kf_key(v, (unsigned)i) >= lo) part += (double)expf((v - vmax) / temp);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = part;
  __syncthreads();
  if (tid == 0) { double t = 0.0; for (int wdx = 0; wdx < FULL_THREADS / 32; ++wdx) t += red[wdx]; red[32] = t; }
  __syncthreads();
  const double mass1 = red[32];
  const float min_w = min_p > 0.f ? min_p : 0.f;           // w of the first is 1: w >= min_p w_max
  // top-p: the shortest prefix of the kept set whose mass reaches top_p of mass1
  if (top_p < 1.f) {
    const Located c = locate(pen, V, vmax, temp, lo, min_w, (double)top_p * mass1, true, false, hist, &sh_prefix, &sh_before, &sh_done);
    if (c.key > lo) lo = c.key;
  }
  // mass of what is kept
  part = 0.0;
  for (int i = tid; i < V; i += FULL_THREADS) {
    const float v = pen[i];
    if (kf_key(v, (unsigned)i) >= lo) { const float w = expf((v - vmax) / temp); if (w >= min_w) part += (double)w; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = part;
  __syncthreads();
  if (tid == 0) { double t = 0.0; for (int wdx = 0; wdx < FULL_THREADS / 32; ++wdx) t += red[wdx]; red[32] = t; }
  __syncthreads();
  const double mass3 = red[32];
  unsigned long long x = ((unsigned long long)(unsigned)st[ST_RNG + 1] << 32) | (unsigned)st[ST_RNG];
  const double r = (double)next_f32(x) * mass3;            // every thread computes the same number
  const Located pick = locate(pen, V, vmax, temp, lo, min_w, r, true, true, hist, &sh_prefix, &sh_before, &sh_done);
  if (tid == 0) {
    st[ST_RNG] = (int)(unsigned)(x & 0xFFFFFFFFull);
    st[ST_RNG + 1] = (int)(unsigned)(x >> 32);
    const int token = kf_key_id(pick.key);
    out_ids[row] = token;
    record_token(st, token);
  }
}

KF_API int kf_sample_state_words() { return ST_WORDS; }
KF_API int kf_sample_slices(int V) { return kf_ceil_div(V, SLICE); }
KF_API int kf_sample_candidates() { return CAND; }

// The whole end of a step for `rows` rows of 32-bit logits [rows, V]:
//   slice_keys: rows * slices * 64 u64, slice_stats: rows * slices * 2 floats (scratch, slices = kf_sample_slices(V));
//   cand_ids / cand_vals [rows, k_out] and cand_lse [rows]: the ranked candidates after the penalty and the
//   log-sum-exp of the row before it (each may be null; k_out <= 64);
//   states: per-request sampler states (null: no penalty, no draw); the request of row i is
//   req_slot[row_req[logit_rows[i]]] (each map may be null for the identity; a negative request skips the row);
//   out_ids [rows]: the drawn tokens (when states is given);
//   flags [rows] and pen [rows, V]: scratch for rows that need the whole ranking; with pen null such rows are an error
//   the caller must have excluded (status KF_ERR_SIZE is NOT raised on the device: the host decides, see `full`).
KF_API int kf_sample(const float* logits, int rows, int V, unsigned long long* slice_keys, float* slice_stats,
                     int* cand_ids, float* cand_vals, float* cand_lse, int k_out, const int* logit_rows, const int* row_req,
                     const int* req_slot, int* states, int* out_ids, int* flags, float* pen, int full, cudaStream_t stream) {
  if (rows <= 0) return KF_OK;
  if (V <= 0 || k_out < 0 || k_out > CAND || (cand_ids && k_out > V)) return KF_ERR_SIZE;
  if (states && (!out_ids || !flags)) return KF_ERR_SIZE;
  if (full && (!pen || !states)) return KF_ERR_SIZE;
  const int n_slices = kf_ceil_div(V, SLICE);
  const size_t merge_smem = (size_t)n_slices * CAND * sizeof(unsigned long long);
  if (merge_smem > 200 * 1024) return KF_ERR_SIZE;        // a vocabulary beyond 1.6 million columns
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  kf_launch(sample_slices_kernel, dim3(n_slices, rows), dim3(SL_THREADS), 0, stream, logits, V, n_slices, logit_rows, row_req,
            req_slot, (const int*)states, slice_keys, slice_stats, cand_lse != nullptr ? 1 : 0,
            (cand_ids != nullptr || cand_lse != nullptr) ? 1 : 0);
  KF_CHECK_LAUNCH();
  kf_launch(sample_merge_kernel, dim3(rows), dim3(MG_THREADS), merge_smem, stream, (const unsigned long long*)slice_keys,
            (const float*)slice_stats, n_slices, V, logit_rows, row_req, req_slot, states, states ? 1 : 0, out_ids, cand_ids,
            cand_vals, cand_lse, k_out, flags);
  KF_CHECK_LAUNCH();
  if (full) {
    kf_launch(sample_full_kernel, dim3(rows), dim3(FULL_THREADS), 0, stream, logits, V, logit_rows, row_req, req_slot, states,
              (const int*)flags, pen, out_ids);
    KF_CHECK_LAUNCH();
  }
  return KF_OK;
}
