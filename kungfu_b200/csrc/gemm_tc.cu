// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) with TMA-fed shared memory and the
// accumulator in tensor memory:   out[T, N] = x[T, K] . w[N, K]^T,  32-bit accumulation.
//
// Shape of the kernel.  The weight tile is the MMA's "A" operand (128 rows of w = 128 output features = the 128
// lanes of tensor memory) and the activation tile its "B" operand (BN token rows, BN in {16..256}), both K-major
// in shared memory with the 128-byte swizzle, 64 k-elements per stage.  So the accumulator holds D[feature, token],
// the same kernel serves decode (BN = 16, many stages of pure weight streaming) and prefill (BN = 256), and an
// epilogue thread owns one output feature: for a given token the 32 lanes of a warp store 32 consecutive features.
//   warp 0   : one lane issues the TMA loads (cp.async.bulk.tensor.2d) stage by stage
//   warp 1   : allocates tensor memory; one lane issues tcgen05.mma (4 per stage, K = 16 each) and the commits
//   warps 2-5: epilogue, each reads its quarter of the 128 lanes with tcgen05.ld and stores
// Epilogues: plain 32-bit store with optional softcap (logits), bfloat16 store, and the gated feed-forward
// (two accumulators, gate rows and up rows of the stacked matrix against the same activation tile, out =
// act(gate) * up).  Split-K (grid z) writes 32-bit partials; the CTA that arrives last for a tile sums them in
// split order and runs the epilogue, so the result does not depend on arrival order.
// Ragged edges (N, T, K not multiples of the tile) are zero-filled by TMA and masked at the store.
// Every wait on an mbarrier is bounded: after the limit the kernel records an error code and leaves through the
// common exit that frees tensor memory.
// Further down, for more rows: a persistent kernel with two accumulator sets (128-token tiles), CTA pairs
// (cta_group::2) on 256 x 256 tiles, the same pairs with K cut inside a cluster of 4 or 8 CTAs for a few hundred rows,
// and the pairs' q,k,v product that rotates q and k and files k and v in its epilogue; `plan_linear` says which runs.
// The reference runs these products as 32-bit SIMT tiles (crates/kf-backend-cuda/src/kernels/quant.cuh:110-171).
#include "common.cuh"
#include "tc_common.cuh"
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

namespace {

using namespace kf_tc;

// A test can make the weight-streaming kernel's producer leave out the loads of every stage from this one on (-1: never),
// so that a wait on operands that never arrive runs into its limit; see kf_test_gemm_give_up.
static __device__ int g_test_drop_from_stage = -1;

template <int BN>
struct Tile {
  static constexpr int COLS = BN < 32 ? 32 : BN;                 // tensor-memory columns per accumulator
  static constexpr int A_BYTES = BM * BK * 2;                    // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;
};

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               void* __restrict__ out, int T, int N, int K, int ld_out, float softcap, int act, int up_offset,
               int stages, int cluster_reduce, float* __restrict__ partial, int* __restrict__ counters,
               int* __restrict__ error_flag) {
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr int NACC = GATED ? 2 : 1;
  constexpr int COLS = Tile<BN>::COLS;
  constexpr int TMEM_COLS = COLS * NACC;
  constexpr int STAGE_BYTES = Tile<BN>::A_BYTES * NACC + Tile<BN>::B_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
  const int splits = gridDim.z;
  const int nkb_total = (K + BK - 1) / BK;
  const int kb_per = (nkb_total + splits - 1) / splits;
  const int kb_begin = blockIdx.z * kb_per;
  const int kb_end = min(nkb_total, kb_begin + kb_per);
  const int nkb = kb_end - kb_begin;                              // >= 1 by the host's choice of splits

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);    // the stage ring
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  int* s_flags = (int*)(tmem_slot + 1);                           // [0] abort, [1] arrival order of this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    s_flags[0] = 0;
    s_flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  kf_pdl_trigger();                                               // the next kernel may start its own prologue

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------------------------
    // The weight tiles of the first stages do not depend on the previous kernel of the stream: they are requested
    // before the grid dependency is waited for, so weight streaming overlaps the predecessor's tail.
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
      const int drop = g_test_drop_from_stage;
      const int pre_all = nkb < stages ? nkb : stages;
      const int pre = (drop >= 0 && drop < pre_all) ? drop : pre_all;      // a test leaves later loads out
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + (size_t)i * STAGE_BYTES;
        mbar_expect_tx(&full[i], STAGE_BYTES);
        const int k = (kb_begin + i) * BK;
        tma_load_2d(st, &tm_w, &full[i], k, f0);
        if (GATED) tma_load_2d(st + Tile<BN>::A_BYTES, &tm_w, &full[i], k, up_offset + f0);
      }
      kf_pdl_wait();                                               // activations come from the previous kernel
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + (size_t)i * STAGE_BYTES + Tile<BN>::A_BYTES * NACC, &tm_x, &full[i], (kb_begin + i) * BK, t0);
      for (int i = pre_all; i < nkb && drop < 0; ++i) {
        const int s = i % stages;
        if (!mbar_wait(&empty[s], ((i / stages) - 1) & 1)) {
          atomicExch(error_flag, ERR_WAIT_EMPTY);
          s_flags[0] = 1;
          break;
        }
        uint8_t* st = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        const int k = (kb_begin + i) * BK;
        tma_load_2d(st, &tm_w, &full[s], k, f0);
        if (GATED) tma_load_2d(st + Tile<BN>::A_BYTES, &tm_w, &full[s], k, up_offset + f0);
        tma_load_2d(st + Tile<BN>::A_BYTES * NACC, &tm_x, &full[s], k, t0);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BN);
      bool ok = true;
      const uint64_t da0 = umma_desc(smem), db0 = umma_desc(smem + Tile<BN>::A_BYTES * NACC);
      const uint64_t du0 = umma_desc(smem + Tile<BN>::A_BYTES);
      int s = 0;
      uint32_t ph = 0;
      for (int i = 0; i < nkb && ok; ++i) {
        if (!mbar_wait(&full[s], ph)) {
          atomicExch(error_flag, ERR_WAIT_FULL);
          s_flags[0] = 1;
          ok = false;
          break;
        }
        const uint64_t so = (uint64_t)((uint32_t)s * (uint32_t)(STAGE_BYTES >> 4));   // descriptors hold address >> 4
        const uint64_t da = da0 + so, du = du0 + so, db = db0 + so;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {                                // 32 bytes per K = 16 step
          const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
          umma(tmem_base, da + 2 * k, db + 2 * k, idesc, accumulate);
          if (GATED) umma(tmem_base + COLS, du + 2 * k, db + 2 * k, idesc, accumulate);
        }
        umma_commit(&empty[s]);                                               // frees the stage when the MMAs have read it
        if (++s == stages) { s = 0; ph ^= 1; }
      }
      umma_commit(acc_full);                                                   // accumulator complete (or abandoned)
    }
  } else {
    // ---- epilogue: warps 2..5, each owns the lane quarter (warp % 4) ---------------------------------------------
    kf_pdl_wait();                                                             // before any global write
    const int quarter = warp & 3;
    const int f = f0 + quarter * 32 + lane;                                    // this thread's output feature
    const bool acc_ok = mbar_wait(acc_full, 0);
    if (!acc_ok && lane == 0) atomicExch(error_flag, ERR_WAIT_ACC);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool good = acc_ok && s_flags[0] == 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int n_out = GATED ? up_offset : N;                                   // features this launch produces
    const int pw = GATED ? 2 * up_offset : N;                                  // width of a partial row

    auto finish = [&](float v, float u) -> float {
      if (EPI == EPI_GATED) return act_fast(v, act) * u;
      if (EPI == EPI_F32) return kf_softcap(v, softcap);
      return v;
    };
    auto store = [&](int t, float r) {
      if (EPI == EPI_F32) ((float*)out)[(size_t)t * ld_out + f] = r;
      else ((__nv_bfloat16*)out)[(size_t)t * ld_out + f] = __float2bfloat16_rn(r);
    };

    if (good && splits == 1) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16], u[16];
        tmem_ld16(lane_addr + c0, v);
        if (GATED) tmem_ld16(lane_addr + COLS + c0, u);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = t0 + c0 + j;
          if (t < T && f < n_out) store(t, finish(v[j], GATED ? u[j] : 0.f));
        }
      }
    } else if (splits > 1 && cluster_reduce) {
      // ---- split-K inside a thread-block cluster: partial tiles stay in shared memory ------------------------------
      // Each CTA of the cluster (one per K split) parks its accumulator in its own shared memory (the pipeline
      // stages are free by now); after a cluster barrier CTA r sums, in split order, the tokens t with t % splits == r
      // straight out of its peers' shared memory and stores them.
      float* red = reinterpret_cast<float*>(smem);                           // [NACC][BN][128]
      const int fl = quarter * 32 + lane;
      if (good) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16], u[16];
          tmem_ld16(lane_addr + c0, v);
          if (GATED) tmem_ld16(lane_addr + COLS + c0, u);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            red[(size_t)(c0 + j) * BM + fl] = v[j];
            if (GATED) red[(size_t)(BN + c0 + j) * BM + fl] = u[j];
          }
        }
      }
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      const int rank = blockIdx.z;
      const uint32_t red_addr = smem_u32(red);
      const int t_hi = min(BN, T - t0);
      uint32_t remote[8];
#pragma unroll
      for (int z = 0; z < 8; ++z)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[z]) : "r"(red_addr), "r"(z < splits ? z : 0));
      // All peers' values of several tokens are requested before any is added, so the remote latencies overlap (a token
      // tile of 256 would otherwise pay one round trip per token); the sum itself runs in split order.
      constexpr int TB = BN >= 64 ? 4 : 1;                                      // tokens per batch of remote loads
      for (int tl0 = rank; tl0 < t_hi; tl0 += splits * TB) {
        float pv[TB][8], pu[TB][8];
#pragma unroll
        for (int b = 0; b < TB; ++b) {
          const int tl = tl0 + b * splits;
          const uint32_t off = (uint32_t)(((size_t)tl * BM + fl) * 4);
          const uint32_t off_u = (uint32_t)(((size_t)(BN + tl) * BM + fl) * 4);
#pragma unroll
          for (int z = 0; z < 8; ++z) {
            pv[b][z] = 0.f;
            pu[b][z] = 0.f;
            if (z < splits && tl < t_hi) {
              asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv[b][z]) : "r"(remote[z] + off) : "memory");
              if (GATED) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pu[b][z]) : "r"(remote[z] + off_u) : "memory");
            }
          }
        }
#pragma unroll
        for (int b = 0; b < TB; ++b) {
          const int tl = tl0 + b * splits;
          float v = 0.f, u = 0.f;
#pragma unroll
          for (int z = 0; z < 8; ++z) { v += pv[b][z]; u += pu[b][z]; }
          if (tl < t_hi && f < n_out) store(t0 + tl, finish(v, u));
        }
      }
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");      // nobody leaves while peers still read
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else if (splits > 1) {
      if (good) {
        float* mine = partial + (size_t)blockIdx.z * T * pw;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16], u[16];
          tmem_ld16(lane_addr + c0, v);
          if (GATED) tmem_ld16(lane_addr + COLS + c0, u);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t < T && f < n_out) {
              mine[(size_t)t * pw + f] = v[j];
              if (GATED) mine[(size_t)t * pw + up_offset + f] = u[j];
            }
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        s_flags[1] = atomicAdd(&counters[tile], 1);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (s_flags[1] == splits - 1) {                                          // last to arrive: reduce in split order
        __threadfence();
        const int t_end = min(T, t0 + BN);
        if (f < n_out) {
          for (int t = t0; t < t_end; ++t) {
            float v = 0.f, u = 0.f;
            for (int z = 0; z < splits; ++z) {
              const float* p = partial + ((size_t)z * T + t) * pw;
              v += __ldcg(p + f);
              if (GATED) u += __ldcg(p + up_offset + f);
            }
            store(t, finish(v, u));
          }
        }
        if (warp == 2 && lane == 0) counters[blockIdx.y * gridDim.x + blockIdx.x] = 0;
      }
    }
  }
  if (warp < 2 && splits > 1 && cluster_reduce) {                  // the two non-epilogue warps join both cluster barriers
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  // ---- common exit: everyone meets, then tensor memory is freed by the warp that allocated it ------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


// ---- persistent variant for many tokens ------------------------------------------------------------------------------
// One CTA per SM walks tiles (feature tile fastest, so that CTAs running side by side share the token tile in L2) and
// keeps TWO accumulators in tensor memory: while the epilogue warps drain one (tcgen05.ld, activation, store), the MMA
// warp already fills the other, and the TMA warp runs ahead through the stage ring across tile boundaries.
template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                          void* __restrict__ out, int T, int N, int K, int ld_out, float softcap, int act, int up_offset,
                          int stages, int* __restrict__ error_flag) {
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr int NACC = GATED ? 2 : 1;
  constexpr int COLS = Tile<BN>::COLS;
  constexpr int ACC_COLS = COLS * NACC;                           // columns of one accumulator set
  constexpr int TMEM_COLS = 2 * ACC_COLS <= 256 ? 256 : 512;
  static_assert(2 * ACC_COLS <= 512, "two accumulator sets must fit tensor memory");
  constexpr int STAGE_BYTES = Tile<BN>::A_BYTES * NACC + Tile<BN>::B_BYTES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;                            // [2]
  uint64_t* acc_empty = acc_full + 2;                             // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* s_abort = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_feat = GATED ? up_offset : N;
  const int n_ft = (n_feat + BM - 1) / BM, n_tt = (T + BN - 1) / BN;
  const int n_tiles = n_ft * n_tt;
  const int nkb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  kf_pdl_trigger();

  if (warp == 0) {
    // ---- TMA producer: one stream of k blocks across all of this CTA's tiles ------------------------------------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
      kf_pdl_wait();
      int s = 0;                                                   // running stage and the parity its `empty` shows
      uint32_t ph = 1;                                             // when free: 1 before the first pass (nothing to wait for)
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int f0 = (tile % n_ft) * BM, t0 = (tile / n_ft) * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[s], ph)) {
            atomicExch(error_flag, ERR_WAIT_EMPTY);
            *s_abort = 1;
            ok = false;
            break;
          }
          uint8_t* st = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          const int k = kb * BK;
          tma_load_2d(st, &tm_w, &full[s], k, f0);
          if (GATED) tma_load_2d(st + Tile<BN>::A_BYTES, &tm_w, &full[s], k, up_offset + f0);
          tma_load_2d(st + Tile<BN>::A_BYTES * NACC, &tm_x, &full[s], k, t0);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ------------------------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BN);
      const uint64_t da0 = umma_desc(smem), db0 = umma_desc(smem + Tile<BN>::A_BYTES * NACC);
      const uint64_t du0 = umma_desc(smem + Tile<BN>::A_BYTES);
      int s = 0;
      uint32_t ph = 0;
      int ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++ti) {
        const int buf = ti & 1;
        if (ti >= 2 && !mbar_wait(&acc_empty[buf], (uint32_t)((ti >> 1) - 1) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full[s], ph)) { ok = false; break; }
          const uint64_t so = (uint64_t)((uint32_t)s * (uint32_t)(STAGE_BYTES >> 4));   // descriptors advance by address >> 4
          const uint64_t da = da0 + so, db = db0 + so, du = du0 + so;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            umma(acc, da + 2 * k, db + 2 * k, idesc, accumulate);
            if (GATED) umma(acc + COLS, du + 2 * k, db + 2 * k, idesc, accumulate);
          }
          umma_commit(&empty[s]);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        umma_commit(&acc_full[buf]);
      }
      if (!ok) { atomicExch(error_flag, ERR_WAIT_FULL); *s_abort = 1; }
    }
  } else {
    // ---- epilogue: drains one accumulator set while the other is being filled -----------------------------------------
    kf_pdl_wait();
    const int quarter = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    int ti = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
      const int buf = ti & 1;
      const int f0 = (tile % n_ft) * BM, t0 = (tile / n_ft) * BN;
      const int f = f0 + quarter * 32 + lane;
      if (!mbar_wait(&acc_full[buf], (uint32_t)(ti >> 1) & 1) || *s_abort) {
        if (lane == 0) atomicExch(error_flag, ERR_WAIT_ACC);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = lane_addr + buf * ACC_COLS;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16], u[16];
        tmem_ld16(acc + c0, v);
        if (GATED) tmem_ld16(acc + COLS + c0, u);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = t0 + c0 + j;
          if (t < T && f < n_feat) {
            float r;
            if (EPI == EPI_GATED) r = act_fast(v[j], act) * u[j];
            else if (EPI == EPI_F32) r = kf_softcap(v[j], softcap);
            else r = v[j];
            if (EPI == EPI_F32) ((float*)out)[(size_t)t * ld_out + f] = r;
            else ((__nv_bfloat16*)out)[(size_t)t * ld_out + f] = __float2bfloat16_rn(r);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&acc_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


// ---- CTA-pair variant (cta_group::2) for many tokens -------------------------------------------------------------------
// Two CTAs of a cluster work on one 256-feature x 256-token tile: each holds its own 128 feature rows of the weights
// and HALF of the token tile (128 rows) in shared memory; one thread of the leader CTA issues tcgen05.mma.cta_group::2
// (M 256, N 256), which reads both CTAs' operands and fills 128 lanes x 256 columns of tensor memory in each CTA.
// Per MMA each SM fetches 4 KB + 4 KB of operands instead of 4 KB + 8 KB, and per k stage TMA fills 32 KB instead of
// 48 KB, which is what the single-CTA kernel runs out of (shared-memory bandwidth).
// Barriers: full[s] lives in the leader and counts the bytes of both CTAs' loads (the loads carry .cta_group::2 so
// that the peer's may signal the leader's barrier); empty[s] and acc_full[b] are signalled in both CTAs by a multicast
// tcgen05.commit; acc_empty[b] lives in the leader and is arrived at by the 256 epilogue threads of the pair.
// No TMA load uses multicast.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {     // arrives at `bar` in both CTAs of the pair
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Four warps per quarter of the lanes drain an accumulator (each takes a quarter of its columns): the epilogue of the
// gated product cannot overlap the next tile (its two accumulators fill tensor memory), and the last epilogue of every
// launch is exposed too.
constexpr int PAIR_THREADS = 576;
constexpr int PAIR_SPLIT_STAGES = 6;                            // the split variant parks 128 KB of partial sums in its ring

// What the q,k,v product needs to rotate and file its own result (EPI_ROPE): a CTA owns one head of 256 (or two of 128), its
// two accumulators are the head's features i and i + half (weight rows h * d + i and h * d + half + i; with two heads the
// second head's in lanes 64-127, fetched as boxes of 64 weight rows), so one thread holds both elements of a rotation pair.  q heads go to q_out rotated, k heads rotated and v heads as they are into the request's
// page at the token's position; rows of no request (padding) give zero q and write no keys.
struct RopeArgs {
  const float* cos_t;                                             // [T, half] by token row
  const float* sin_t;
  const int* positions;
  const int* row_req;
  const int* block_table;
  int table_stride, page_size, nh, nkv, write_kv;
  int half;                                                       // head size / 2: 128 (a CTA holds one head) or 64 (two heads)
  __nv_bfloat16* pages;                                           // [page][k, v][nkv][page_size][head size]
  __nv_bfloat16* q_out;                                           // [T, nh * head size]
};

template <int EPI, int PN>                                        // PN: tokens of the pair's tile = MMA N (256, or 128 for EPI_ROPE)
__device__ __forceinline__ void
gemm_tc_pair_body(const CUtensorMap& tm_w, const CUtensorMap& tm_x, void* __restrict__ out, int T, int N, int K, int ld_out,
                  float softcap, int act, int up_offset, int stages, int* __restrict__ error_flag, const RopeArgs& ra) {
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr bool ROPE = EPI == EPI_ROPE;
  constexpr int NACC = (GATED || ROPE) ? 2 : 1;
  constexpr int NBUF = NACC * PN * 2 <= 512 ? 2 : 1;              // accumulator sets in tensor memory (512 columns)
  constexpr int A_BYTES = BM * BK * 2, BH_BYTES = (PN / 2) * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES * NACC + BH_BYTES;
  constexpr int TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;                            // [2]
  uint64_t* acc_empty = acc_full + 2;                             // [2] (used in the leader)
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* s_abort = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int n_feat = GATED ? up_offset : N;
  // ROPE: a CTA's "feature tile" is one head (its 128 rotation pairs), a pair's tile two heads
  const int hpc = ROPE ? BM / ra.half : 1;                        // heads per CTA
  const int n_ft = ROPE ? (ra.nh + 2 * ra.nkv + 2 * hpc - 1) / (2 * hpc) : (n_feat + 2 * BM - 1) / (2 * BM), n_tt = (T + PN - 1) / PN;
  const int n_tiles = n_ft * n_tt;
  const int nkb = (K + BK - 1) / BK;
  const int second = ROPE ? BM : up_offset;                       // weight rows of the second accumulator, after the first's

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * (PAIR_THREADS - 64)); }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                             // the peer's barriers exist before anyone signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  kf_pdl_trigger();

  if (warp == 0) {
    // ---- TMA producer (both CTAs): own weight rows, own half of the token tile; bytes are counted in the leader --------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
      kf_pdl_wait();
      int s = 0;
      uint32_t ph = 1;                                             // parity of `empty` when the stage is free
      bool ok = true;
      const uint32_t full0 = map_to_rank(smem_u32(&full[0]), 0);   // the leader's full[0], as a cluster address
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        const int f0 = ((tile % n_ft) * 2 + (int)rank) * (ROPE ? 2 * BM : BM);
        const int t0 = (tile / n_ft) * PN + (int)rank * (PN / 2);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[s], ph)) {
            atomicExch(error_flag, ERR_WAIT_EMPTY);
            *s_abort = 1;
            ok = false;
            break;
          }
          uint8_t* st = smem + (size_t)s * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          const uint32_t bar = full0 + 8u * (uint32_t)s;
          const int k = kb * BK;
          if (ROPE && hpc == 2) {                                                    // two heads of 128: four boxes of 64 weight rows
            tma_load_2d_pair(st, &tm_w, bar, k, f0);
            tma_load_2d_pair(st + A_BYTES / 2, &tm_w, bar, k, f0 + BM);
            tma_load_2d_pair(st + A_BYTES, &tm_w, bar, k, f0 + BM / 2);
            tma_load_2d_pair(st + A_BYTES + A_BYTES / 2, &tm_w, bar, k, f0 + BM + BM / 2);
          } else {
            tma_load_2d_pair(st, &tm_w, bar, k, f0);
            if (NACC == 2) tma_load_2d_pair(st + A_BYTES, &tm_w, bar, k, second + f0);
          }
          tma_load_2d_pair(st + A_BYTES * NACC, &tm_x, bar, k, t0);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (leader only) ------------------------------------------------------------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      const uint64_t da0 = umma_desc(smem), db0 = umma_desc(smem + A_BYTES * NACC), du0 = umma_desc(smem + A_BYTES);
      int s = 0;
      uint32_t ph = 0;
      int ti = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++ti) {
        const int buf = ti % NBUF;
        if (ti >= NBUF && !mbar_wait(&acc_empty[buf], (uint32_t)((ti / NBUF) - 1) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * NACC * PN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full[s], ph)) { ok = false; break; }
          const uint64_t so = (uint64_t)((uint32_t)s * (uint32_t)(STAGE_BYTES >> 4));
          const uint64_t da = da0 + so, db = db0 + so, du = du0 + so;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            umma_pair(acc, da + 2 * k, db + 2 * k, idesc, accumulate);
            if (NACC == 2) umma_pair(acc + PN, du + 2 * k, db + 2 * k, idesc, accumulate);
          }
          umma_commit_pair(&empty[s]);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(&acc_full[buf]);
      }
      if (!ok) { atomicExch(error_flag, ERR_WAIT_FULL); *s_abort = 1; }
    }
  } else {
    // ---- epilogue (both CTAs): each drains its own 128 lanes ------------------------------------------------------------
    kf_pdl_wait();
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;                          // which quarter of the tile's tokens this warp drains
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    int ti = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++ti) {
      const int buf = ti % NBUF;
      const int f0 = ((tile % n_ft) * 2 + (int)rank) * (ROPE ? 2 * BM : BM), t0 = (tile / n_ft) * PN;
      const int f = f0 + quarter * 32 + lane;
      // ROPE: where this warp's PN / 4 rows go (one or two rows per lane), looked up while the accumulator is still being filled:
      // for k and v heads the row's slot in the pages (in rows of 256), for q heads 0; -1 for rows of no request
      const int head = ((tile % n_ft) * 2 + (int)rank) * hpc + (hpc == 2 ? quarter >> 1 : 0);
      const bool is_q = ROPE && head < ra.nh, is_k = ROPE && !is_q && head < ra.nh + ra.nkv;
      const bool is_v = ROPE && !is_q && !is_k && head < ra.nh + 2 * ra.nkv;
      const bool rope_work = is_q || ((is_k || is_v) && ra.write_kv);
      int meta_a = -1, meta_b = -1;
      if (ROPE && rope_work) {
        const int kvh = is_k ? head - ra.nh : head - ra.nh - ra.nkv;
#pragma unroll
        for (int cc = 0; cc < PN / 128; ++cc) {
          const int t = t0 + col_half * (PN / 4) + cc * 32 + lane;
          int m = -1;
          if (t < T) {
            const int req = __ldg(ra.row_req + t);
            if (req >= 0) {
              m = 0;
              if (!is_q) {
                const int pos = __ldg(ra.positions + t);
                const int page = __ldg(ra.block_table + (size_t)req * ra.table_stride + pos / ra.page_size);
                m = ((page * 2 + (is_v ? 1 : 0)) * ra.nkv + kvh) * ra.page_size + pos % ra.page_size;
              }
            }
          }
          if (cc) meta_b = m; else meta_a = m;
        }
      }
      if (!mbar_wait(&acc_full[buf], (uint32_t)(ti / NBUF) & 1) || *s_abort) {
        if (lane == 0) atomicExch(error_flag, ERR_WAIT_ACC);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = lane_addr + buf * NACC * PN;
      if constexpr (ROPE) {
        // this CTA's head: a q head (rotated to q_out), a k head (rotated into the page), a v head (into the page) or none
        const int i = (quarter * 32 + lane) & (ra.half - 1);                         // the rotation pair (i, i + half) of the head
        const int hd = 2 * ra.half;
        if (rope_work) {
#pragma unroll 1
          for (int cc = 0; cc < PN / 64; ++cc) {                                     // sixteen rows at a time
            const int c0 = col_half * (PN / 4) + cc * 16;
            // the rows' angles are all asked for before the accumulator is read and the first of them is used
            float cs[16], sn[16];
            if (!is_v) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int tc = min(t0 + c0 + j, T - 1);
                cs[j] = __ldg(ra.cos_t + (size_t)tc * ra.half + i);
                sn[j] = __ldg(ra.sin_t + (size_t)tc * ra.half + i);
              }
            }
            float v[16], u[16];
            tmem_ld16(acc + c0, v);
            tmem_ld16(acc + PN + c0, u);
            const int meta = (cc & 2) ? meta_b : meta_a;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c0 + j;
              const int m = __shfl_sync(0xffffffffu, meta, (cc & 1) * 16 + j);
              if (t >= T) continue;
              float a = v[j], b = u[j];
              if (!is_v) {
                const float x1 = a, x2 = b;
                a = x1 * cs[j] - x2 * sn[j];
                b = x2 * cs[j] + x1 * sn[j];
              }
              if (is_q) {
                if (m < 0) a = b = 0.f;
                __nv_bfloat16* q = ra.q_out + ((size_t)t * ra.nh + head) * hd + i;
                q[0] = __float2bfloat16_rn(a);
                q[ra.half] = __float2bfloat16_rn(b);
              } else if (m >= 0) {
                __nv_bfloat16* kv = ra.pages + (size_t)m * hd + i;
                kv[0] = __float2bfloat16_rn(a);
                kv[ra.half] = __float2bfloat16_rn(b);
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = col_half * (PN / 4); c0 < (col_half + 1) * (PN / 4); c0 += 32) {   // 32 tokens per wait on tensor memory
          float v[32], u[32];
          if (GATED) tmem_ld32x2(acc + c0, acc + PN + c0, v, u);
          else tmem_ld32(acc + c0, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t = t0 + c0 + j;
            if (t < T && f < n_feat) {
              float r;
              if (EPI == EPI_GATED) r = act_fast(v[j], act) * u[j];
              else if (EPI == EPI_F32) r = kf_softcap(v[j], softcap);
              else r = v[j];
              if (EPI == EPI_F32) ((float*)out)[(size_t)t * ld_out + f] = r;
              else ((__nv_bfloat16*)out)[(size_t)t * ld_out + f] = __float2bfloat16_rn(r);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[buf]), 0));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                             // no MMA of the pair is in flight, nobody signals a CTA that left
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int EPI>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    void* __restrict__ out, int T, int N, int K, int ld_out, float softcap, int act, int up_offset,
                    int stages, int* __restrict__ error_flag) {
  gemm_tc_pair_body<EPI, 256>(tm_w, tm_x, out, T, N, K, ld_out, softcap, act, up_offset, stages, error_flag, RopeArgs{});
}

// The q,k,v product of a prompt with head size 256 that rotates q and k and files k and v itself (no 32-bit q,k,v rows in
// memory, no kernel after it): see RopeArgs.
template <int PN>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_rope_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, int T, int N, int K,
                         int stages, int* __restrict__ error_flag, const __grid_constant__ RopeArgs ra) {
  gemm_tc_pair_body<EPI_ROPE, PN>(tm_w, tm_x, nullptr, T, N, K, 0, 0.f, 0, 0, stages, error_flag, ra);
}

// ---- CTA pairs with K cut inside a cluster, for a few hundred tokens ----------------------------------------------------
// With 256 x 256 tiles a portion of 256 to 1,024 tokens has fewer tiles than a quarter of the SMs.  Here a cluster of
// 2 x `splits` CTAs owns one tile: pair z (cluster ranks 2z, 2z + 1) multiplies the z-th part of K exactly as the pair
// kernel above does, every CTA parks its 128 features x 256 tokens of 32-bit partial sums in its own shared memory (the
// stage ring is free by then), and after a cluster barrier the CTA of pair z and half h sums, in split order, the tokens
// [z, z + 1) * 256 / splits of half h out of its peers' shared memory (16-byte loads) and stores them.  One tile per
// cluster; plain 32-bit or bfloat16 store.
__device__ __forceinline__ void umma_commit_pair_at(uint64_t* bar, uint32_t leader) {   // both CTAs of the pair led by `leader`
  const uint16_t mask = (uint16_t)(3u << leader);
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

template <int EPI>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_split_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                          void* __restrict__ out, int T, int N, int K, int ld_out, float softcap, int stages, int splits,
                          int* __restrict__ error_flag) {
  constexpr int PN = 256;
  constexpr int A_BYTES = BM * BK * 2, BH_BYTES = (PN / 2) * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + BH_BYTES;
  constexpr int TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  volatile int* s_abort = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const uint32_t half = rank & 1u, leader = rank & ~1u;
  const int z = (int)(rank >> 1);
  const int tile = blockIdx.x / (2 * splits);
  const int n_ft = (N + 2 * BM - 1) / (2 * BM);
  const int f0 = (tile % n_ft) * 2 * BM + (int)half * BM, t0 = (tile / n_ft) * PN;
  const int nkb_total = (K + BK - 1) / BK;
  const int kb_per = (nkb_total + splits - 1) / splits;
  const int kb0 = z * kb_per;
  const int nkb = min(nkb_total, kb0 + kb_per) - kb0;              // >= 1 by the host's choice of splits

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                             // the peers' barriers exist before anyone signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  kf_pdl_trigger();

  if (warp == 0) {
    // ---- TMA producer (every CTA): own weight rows, own half of the token tile; bytes are counted in the pair's leader ---
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
      const uint32_t full0 = map_to_rank(smem_u32(&full[0]), leader);
      const int tx0 = t0 + (int)half * (PN / 2);
      // the weights do not depend on the kernel before: the first stages' weight tiles are asked for at once
      const int pre = nkb < stages ? nkb : stages;
      for (int i = 0; i < pre; ++i) {
        if (half == 0) mbar_expect_tx(&full[i], 2 * STAGE_BYTES);
        tma_load_2d_pair(smem + (size_t)i * STAGE_BYTES, &tm_w, full0 + 8u * (uint32_t)i, (kb0 + i) * BK, f0);
      }
      kf_pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d_pair(smem + (size_t)i * STAGE_BYTES + A_BYTES, &tm_x, full0 + 8u * (uint32_t)i, (kb0 + i) * BK, tx0);
      int s = 0;
      uint32_t ph = 0;                                             // parity of `empty` when a stage has been used once
      for (int i = pre; i < nkb; ++i) {
        if (!mbar_wait(&empty[s], ph)) {
          atomicExch(error_flag, ERR_WAIT_EMPTY);
          *s_abort = 1;
          break;
        }
        uint8_t* st = smem + (size_t)s * STAGE_BYTES;
        if (half == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
        const uint32_t bar = full0 + 8u * (uint32_t)s;
        const int k = (kb0 + i) * BK;
        tma_load_2d_pair(st, &tm_w, bar, k, f0);
        tma_load_2d_pair(st + A_BYTES, &tm_x, bar, k, tx0);
        if (++s == stages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (the pair's leader only) --------------------------------------------------------------------------
    if (lane == 0 && half == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      const uint64_t da0 = umma_desc(smem), db0 = umma_desc(smem + A_BYTES);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(&full[s], ph)) { ok = false; break; }
        const uint64_t so = (uint64_t)((uint32_t)s * (uint32_t)(STAGE_BYTES >> 4));
        const uint64_t da = da0 + so, db = db0 + so;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_pair(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit_pair_at(&empty[s], leader);
        if (++s == stages) { s = 0; ph ^= 1; }
      }
      umma_commit_pair_at(acc_full, leader);
      if (!ok) { atomicExch(error_flag, ERR_WAIT_FULL); *s_abort = 1; }
    }
  } else {
    // ---- epilogue, first half: every CTA parks its own 128 lanes x 256 tokens in shared memory as [token][feature] -------
    const int quarter = warp & 3;
    const int col_q = (warp - 2) >> 2;                             // which quarter of the tile's tokens this warp drains
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float* red = reinterpret_cast<float*>(smem);
    const int fl = quarter * 32 + lane;
    if (!mbar_wait(acc_full, 0) || *s_abort) {
      if (lane == 0) atomicExch(error_flag, ERR_WAIT_ACC);
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = col_q * (PN / 4); c0 < (col_q + 1) * (PN / 4); c0 += 32) {
        float v[32];
        tmem_ld32(lane_addr + c0, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) red[(size_t)(c0 + j) * BM + fl] = v[j];
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                             // every partial tile of the cluster is parked
  if (warp >= 2) {
    // ---- epilogue, second half: sum this CTA's share of the tokens over the splits, in split order, and store ----------
    kf_pdl_wait();                                                 // before any global write
    const int te = threadIdx.x - 64;                               // 0..511
    const int fq = (te & 31) * 4, trow = te >> 5;                  // four features of one token per thread, 16 tokens a pass
    const int slice = PN / splits;
    const int f = f0 + fq;
    const uint32_t red_addr = smem_u32(smem) + (uint32_t)fq * 4u;
    uint32_t src[4];
#pragma unroll
    for (int zz = 0; zz < 4; ++zz) src[zz] = map_to_rank(red_addr, (uint32_t)((zz < splits ? zz : 0) * 2) + half);
    const bool vec = (f + 3 < N) && (ld_out % 4 == 0);
    for (int tl0 = z * slice + trow; tl0 < (z + 1) * slice; tl0 += 64) {
      float4 p[4][4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int tl = tl0 + b * 16;
#pragma unroll
        for (int zz = 0; zz < 4; ++zz) {
          p[b][zz] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (zz < splits && tl < (z + 1) * slice && t0 + tl < T) p[b][zz] = ld_cluster_f4(src[zz] + (uint32_t)tl * (BM * 4u));
        }
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int tl = tl0 + b * 16, t = t0 + tl;
        if (tl >= (z + 1) * slice || t >= T) continue;
        float r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int zz = 0; zz < 4; ++zz) { r[0] += p[b][zz].x; r[1] += p[b][zz].y; r[2] += p[b][zz].z; r[3] += p[b][zz].w; }
        if (EPI == EPI_F32) {
#pragma unroll
          for (int j = 0; j < 4; ++j) r[j] = kf_softcap(r[j], softcap);
          float* o = (float*)out + (size_t)t * ld_out + f;
          if (vec) *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
          else
            for (int j = 0; j < 4; ++j) if (f + j < N) o[j] = r[j];
        } else {
          __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)t * ld_out + f;
          if (vec) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
            uint2 w;
            w.x = *reinterpret_cast<uint32_t*>(&lo);
            w.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(o) = w;
          } else {
            for (int j = 0; j < 4; ++j) if (f + j < N) o[j] = __float2bfloat16_rn(r[j]);
          }
        }
      }
    }
  }
  cluster_sync_all();                                             // nobody leaves while a peer reads its shared memory
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

std::mutex g_map_mutex;
std::map<std::tuple<const void*, long, long, int>, CUtensorMap> g_maps;

// A 2-D map over a row-major [rows, cols] bfloat16 matrix with boxes of [box_rows, 64] and the 128-byte swizzle.
}  // namespace

bool kf_tc::tensor_maps_available() { return encode_fn() != nullptr; }

bool kf_tc::tensor_map(const void* base, long rows, long cols, int box_rows, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto key = std::make_tuple(base, rows, cols, box_rows);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUtensorMap m;
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  *out = m;
  return true;
}

namespace {

int g_cluster_reduce = 1;
int g_stage_cap_kb = 108;
// Choice of token tile and split-K for a launch.
int g_plan_bn = 0, g_plan_splits = 0;               // a tuning build can fix the plan of products over more than 64 rows

int g_pair = 1;             // many tokens: CTA pairs
int g_pair_split = 1;       // a few hundred tokens: CTA pairs with K cut inside the cluster
int g_pair_rope = 1;        // prompts, head size 256: the q,k,v product rotates and files its own result
int g_rope_pn = 0;          // tuning: token tile of that product (0: chosen by the tile count)
int pair_split_capacity(int splits);
int stream_cluster_capacity(int splits);

int plan_linear(int T, int N_features, int K, int gated, int* bn_out, int* splits_out) {
  const int n_sm = kf_sm_count();
  int bn = 16;
  while (bn < T && bn < 256) bn *= 2;
  if (gated && bn > 256) bn = 256;
  const int nkb = (K + BK - 1) / BK;
  if (T > 64 && g_plan_bn > 0) {
    *bn_out = g_plan_bn;
    *splits_out = g_plan_splits > nkb ? nkb : (g_plan_splits < 1 ? 1 : g_plan_splits);
    return KF_OK;
  }
  int splits = 1;
  if (!gated && T > 128 && g_pair) {
    // A few hundred tokens: with 256 x 256 tiles there are fewer tiles than CTA pairs.  While all clusters of a launch run
    // at once, K is cut four or two ways inside a cluster of pairs (`gemm_tc_pair_split_kernel`); with more tiles than
    // that, whole tiles on pairs.  Measured at the 2304-, 3584- and 4608-wide layers, 256 to 768 rows, against 64-token
    // tiles on the weight-streaming kernel: 9216 -> 2304 at 256 rows 33 -> 23 us, 14336 -> 3584 at 512 rows 77 -> 47 us,
    // 3584 -> 8192 at 512 rows 50 -> 28 us (whole tiles), nothing more than a tenth slower.
    const int tt = kf_ceil_div(T, 256);
    const int tiles = kf_ceil_div(N_features, 2 * BM) * tt;
    const bool filled = tt == 1 || (long)T * 5 >= (long)tt * 256 * 3;   // several token tiles: at least 0.6 full
    const int cap4 = g_pair_split ? pair_split_capacity(4) : 0, cap2 = g_pair_split ? pair_split_capacity(2) : 0;
    const int cut = (filled && tiles <= cap4 && nkb >= 32) ? 4 : (filled && tiles <= cap2 && nkb >= 16) ? 2 : 0;
    // Up to 192 rows the 64-token tiles are three and read the weights three times from L2: the clusters win where they
    // cover most of the GPU (14336 -> 3584 at 160 rows: 43 -> 30 us), and lose where they are few (9216 -> 2304: 19 -> 21 us).
    if (cut && (T > 192 || tiles * 2 * cut * 10 >= n_sm * 7)) { *bn_out = 256; *splits_out = cut; return KF_OK; }
    if (T >= 224 && tiles > n_sm / 4 - 4) { *bn_out = 256; *splits_out = 1; return KF_OK; }
  }
  if (T > 64 && gated) {
    // Prompt portions through the gated epilogue never split K (their partial tiles would have to go through global
    // memory); up to 256 rows a 128-token tile gives twice the tiles (measured at 256 rows, 9216 x 2304: 29 us against
    // 42 us with one 256-token tile and 220 us split in two).
    bn = T <= 256 ? 128 : 256;
  } else if (T > 64 && (T <= 512 || (T <= 1024 && K <= 4096 && (long)kf_ceil_div(N_features, BM) * kf_ceil_div(T, 64) <= 2 * n_sm))) {
    // Short portions: 64-token tiles on the weight-streaming kernel, two CTAs per SM, K cut so that about two CTAs per SM
    // run (measured at 2304-wide layers, 128 to 512 rows: 1.3x to 2x faster than one 256-token tile split four ways).
    // A cluster needs all its CTAs at once, so fewer CTAs fit than two per SM (clusters of eight: 32 x 8, not 296): K is
    // cut only as far as every cluster of the launch still runs at once (9216 -> 2304 at 128 rows, 36 tiles: in four 17.9 us,
    // in eight 22.7 us; 4096 -> 4608 at 128 rows, 72 tiles: in two 18.2 us, in four 22.7 us).
    bn = 64;
    const long tiles = (long)kf_ceil_div(N_features, BM) * kf_ceil_div(T, bn);
    while (splits < 8 && tiles * splits * 2 <= 2 * n_sm && nkb / (splits * 2) >= 8 && tiles <= stream_cluster_capacity(splits * 2))
      splits *= 2;
  } else {
    const long tiles = (long)kf_ceil_div(N_features, BM) * kf_ceil_div(T, bn);
    if (tiles <= n_sm / 2 && !(bn == 256 && g_pair)) {       // fewer tiles than half the SMs: cut K so that every SM streams
      splits = (int)(n_sm / tiles);                     // weights, in ONE wave (one CTA per SM fits)
      if (splits > 8) splits = 8;                      // a portable thread-block cluster holds 8 CTAs
      if (splits > nkb) splits = nkb;
    }
  }
  if (splits > 1) {
    const int kb_per = (nkb + splits - 1) / splits;
    splits = (nkb + kb_per - 1) / kb_per;              // no empty split
  }
  *bn_out = bn;
  *splits_out = splits;
  return KF_OK;
}

template <int BN, int EPI>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K, int ld_out, float softcap,
           int act, int up_offset, int splits, float* partial, int* counters, int* error_flag, cudaStream_t stream) {
  constexpr int NACC = EPI == EPI_GATED ? 2 : 1;
  constexpr int STAGE_BYTES = Tile<BN>::A_BYTES * NACC + Tile<BN>::B_BYTES;
  const int nkb = (K + BK - 1) / BK;
  const int kb_per = (nkb + splits - 1) / splits;
  int stages = (SMEM_LIMIT - 2048) / STAGE_BYTES;
  if (BN <= 64 && g_stage_cap_kb > 0) {                 // weight streaming: leave room for a second resident CTA so
    // that the next product can request its first tiles meanwhile.  The gated product gets 20 KB more (a third stage
    // at 64 tokens): its neighbours in a layer are plain products, and 128 + 96 KB still share an SM.
    const int cap = ((g_stage_cap_kb + (EPI == EPI_GATED ? 20 : 0)) * 1024) / STAGE_BYTES;
    if (stages > cap) stages = cap;
  }
  if (stages > kb_per) stages = kb_per;
  if (stages > 12) stages = 12;
  if (stages < 1) return KF_ERR_SIZE;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + 512;
  static bool configured = false;                      // per instantiation
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  const int n_feat = EPI == EPI_GATED ? up_offset : N;
  dim3 grid(kf_ceil_div(n_feat, BM), kf_ceil_div(T, BN), splits);
  // split-K inside a cluster needs the partial tile to fit the pipeline's shared memory and at most 8 CTAs
  const bool cluster = splits > 1 && splits <= 8 && g_cluster_reduce &&
                       (size_t)NACC * BN * BM * 4 <= (size_t)stages * STAGE_BYTES;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (kf_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = splits;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI>, tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, stages,
                     cluster ? 1 : 0, partial, counters, error_flag);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// How many clusters of `splits` CTAs of the weight-streaming kernel with 64-token tiles the GPU holds at once.
int stream_cluster_capacity(int splits) {
  static int cap[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (splits < 2 || splits > 8) return 1 << 30;
  if (cap[splits] < 0) {
    cap[splits] = 1 << 30;                                         // if it cannot be asked: no limit, as before
    constexpr int STAGE_BYTES = Tile<64>::A_BYTES + Tile<64>::B_BYTES;
    int stages = (SMEM_LIMIT - 2048) / STAGE_BYTES;
    if (g_stage_cap_kb > 0 && stages > g_stage_cap_kb * 1024 / STAGE_BYTES) stages = g_stage_cap_kb * 1024 / STAGE_BYTES;
    if (cudaFuncSetAttribute(gemm_tc_kernel<64, EPI_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1, 1, splits);
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = (size_t)stages * STAGE_BYTES + 1024 + 512;
      cudaLaunchAttribute cl;
      cl.id = cudaLaunchAttributeClusterDimension;
      cl.val.clusterDim.x = 1;
      cl.val.clusterDim.y = 1;
      cl.val.clusterDim.z = splits;
      cfg.attrs = &cl;
      cfg.numAttrs = 1;
      // The cluster query answers as if one CTA ran per SM (74 / 33 / 15 clusters of 2 / 4 / 8 here); two of these CTAs share
      // an SM's shared memory, and twice its answer is where the measured launches begin to take a second round.
      int n = 0;
      int dev = 0, sm_bytes = 0, block_reserved = 0;
      int per_sm = 1;
      if (cudaGetDevice(&dev) == cudaSuccess &&
          cudaDeviceGetAttribute(&sm_bytes, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess &&
          cudaDeviceGetAttribute(&block_reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) == cudaSuccess)
        per_sm = (int)((size_t)sm_bytes / (cfg.dynamicSmemBytes + (size_t)block_reserved));
      else
        cudaGetLastError();
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<64, EPI_F32>, &cfg) == cudaSuccess && n > 0) cap[splits] = n * (per_sm > 1 ? per_sm : 1);
      else cudaGetLastError();
    } else {
      cudaGetLastError();
    }
  }
  return cap[splits];
}

int g_persistent = 1;
int g_gated_wide = 1;      // gated products over >= 256 tokens: one 2 x (128 x 256) tile per CTA (less shared-memory fill per flop)

template <int BN, int EPI>
int launch_persistent(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K, int ld_out, float softcap,
                      int act, int up_offset, int* error_flag, cudaStream_t stream) {
  constexpr int NACC = EPI == EPI_GATED ? 2 : 1;
  constexpr int STAGE_BYTES = Tile<BN>::A_BYTES * NACC + Tile<BN>::B_BYTES;
  int stages = (SMEM_LIMIT - 2048) / STAGE_BYTES;
  if (stages > 8) stages = 8;
  if (stages < 2) return KF_ERR_SIZE;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + 512;
  static bool configured = false;
  const int n_sm = kf_sm_count();
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  const int n_feat = EPI == EPI_GATED ? up_offset : N;
  const int n_tiles = kf_ceil_div(n_feat, BM) * kf_ceil_div(T, BN);
  const int grid = n_tiles < n_sm ? n_tiles : n_sm;
  kf_launch(gemm_tc_persistent_kernel<BN, EPI>, dim3(grid), dim3(THREADS), smem, stream, tw, tx, out, T, N, K, ld_out,
            softcap, act, up_offset, stages, error_flag);
  KF_CHECK_LAUNCH();
  return KF_OK;
}


template <int EPI>
int launch_pair(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K, int ld_out, float softcap,
                int act, int up_offset, int* error_flag, cudaStream_t stream) {
  constexpr int NACC = EPI == EPI_GATED ? 2 : 1;
  constexpr int STAGE_BYTES = BM * BK * 2 * NACC + 128 * BK * 2;
  int stages = (SMEM_LIMIT - 2048) / STAGE_BYTES;
  if (stages > 8) stages = 8;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + 512;
  static bool configured = false;
  const int n_sm = kf_sm_count();
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  const int n_feat = EPI == EPI_GATED ? up_offset : N;
  const int n_tiles = kf_ceil_div(n_feat, 2 * BM) * kf_ceil_div(T, 256);
  int pairs = n_sm / 2;
  if (pairs > n_tiles) pairs = n_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(PAIR_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (kf_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<EPI>, tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, stages, error_flag);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <int PN>
int launch_pair_rope(const CUtensorMap& tw, const CUtensorMap& tx, int T, int N, int K, const RopeArgs& ra, int* error_flag,
                     cudaStream_t stream) {
  constexpr int STAGE_BYTES = BM * BK * 2 * 2 + (PN / 2) * BK * 2;
  int stages = (SMEM_LIMIT - 2048) / STAGE_BYTES;
  if (stages > 8) stages = 8;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024 + 512;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_pair_rope_kernel<PN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  const int n_tiles = kf_ceil_div(ra.nh + 2 * ra.nkv, 2 * (BM / ra.half)) * kf_ceil_div(T, PN);
  int pairs = kf_sm_count() / 2;
  if (pairs > n_tiles) pairs = n_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(PAIR_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (kf_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaLaunchKernelEx(&cfg, gemm_tc_pair_rope_kernel<PN>, tw, tx, T, N, K, stages, error_flag, ra);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <int EPI>
void pair_split_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int n_tiles, int splits, cudaStream_t stream) {
  constexpr int STAGE_BYTES = BM * BK * 2 + 128 * BK * 2;
  cfg->gridDim = dim3(2 * splits * n_tiles);
  cfg->blockDim = dim3(PAIR_THREADS);
  cfg->dynamicSmemBytes = (size_t)PAIR_SPLIT_STAGES * STAGE_BYTES + 1024 + 512;
  cfg->stream = stream;
  int na = 0;
  if (kf_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2 * splits;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  ++na;
  cfg->attrs = attr;
  cfg->numAttrs = na;
}

template <int EPI>
bool pair_split_configure() {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_pair_split_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return false;
    }
    configured = true;
  }
  return true;
}

// How many clusters of 2 x splits CTAs of the split pair kernel the GPU holds at once (0 if it cannot be asked).
int pair_split_capacity(int splits) {
  static int cap[5] = {-1, -1, -1, -1, -1};
  if (splits < 2 || splits > 4) return 0;
  if (cap[splits] < 0) {
    cap[splits] = 0;
    if (pair_split_configure<EPI_F32>()) {
      cudaLaunchConfig_t cfg = {};
      cudaLaunchAttribute attr[2];
      pair_split_config<EPI_F32>(&cfg, attr, 1, splits, nullptr);
      cfg.attrs = &attr[cfg.numAttrs - 1];                         // the query takes the cluster shape alone
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_split_kernel<EPI_F32>, &cfg) == cudaSuccess) cap[splits] = n;
      else cudaGetLastError();
    }
  }
  return cap[splits];
}

template <int EPI>
int launch_pair_split(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K, int ld_out, float softcap,
                      int splits, int* error_flag, cudaStream_t stream) {
  if (!pair_split_configure<EPI>()) return KF_ERR_SETUP;
  const int n_tiles = kf_ceil_div(N, 2 * BM) * kf_ceil_div(T, 256);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  pair_split_config<EPI>(&cfg, attr, n_tiles, splits, stream);
  cudaLaunchKernelEx(&cfg, gemm_tc_pair_split_kernel<EPI>, tw, tx, out, T, N, K, ld_out, softcap, PAIR_SPLIT_STAGES, splits, error_flag);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

template <int EPI>
int launch_bn(int bn, const CUtensorMap& tw, const CUtensorMap& tx, void* out, int T, int N, int K, int ld_out, float softcap,
              int act, int up_offset, int splits, float* partial, int* counters, int* error_flag, cudaStream_t s) {
  switch (bn) {
    case 16: return launch<16, EPI>(tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, splits, partial, counters, error_flag, s);
    case 32: return launch<32, EPI>(tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, splits, partial, counters, error_flag, s);
    case 64: return launch<64, EPI>(tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, splits, partial, counters, error_flag, s);
    case 128: return launch<128, EPI>(tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, splits, partial, counters, error_flag, s);
    case 256: return launch<256, EPI>(tw, tx, out, T, N, K, ld_out, softcap, act, up_offset, splits, partial, counters, error_flag, s);
  }
  return KF_ERR_SIZE;
}

}  // namespace

#ifdef KF_TUNING
// Measurement hooks, compiled only into a tuning build (-DKF_TUNING): they override the planner's choices.
KF_API void kf_set_gemm_cluster_reduce(int on) { g_cluster_reduce = on ? 1 : 0; }   // 0: split sums through global memory
KF_API void kf_set_gemm_stage_cap_kb(int kb) { g_stage_cap_kb = kb; }
KF_API void kf_set_gemm_persistent(int on) { g_persistent = on ? 1 : 0; }
KF_API void kf_set_gemm_pair(int on) { g_pair = on ? 1 : 0; }
KF_API void kf_set_gemm_pair_split(int on) { g_pair_split = on ? 1 : 0; }
KF_API void kf_set_gemm_pair_rope(int on) { g_pair_rope = on ? 1 : 0; }
KF_API void kf_set_gemm_rope_pn(int pn) { g_rope_pn = pn; }
KF_API int kf_gemm_pair_split_capacity(int splits) { return pair_split_capacity(splits); }
KF_API int kf_gemm_stream_cluster_capacity(int splits) { return stream_cluster_capacity(splits); }
KF_API void kf_set_gemm_plan(int bn, int splits) { g_plan_bn = bn; g_plan_splits = splits; }   // products over more than 64 rows
KF_API void kf_set_gemm_gated_wide(int on) { g_gated_wide = on ? 1 : 0; }
#endif

// For tests of the give-up path: every bounded wait of this file's kernels gives up after `limit_ns` nanoseconds (0: the
// built-in two seconds), and the weight-streaming kernel's producer issues no load for stages `drop_from_stage` and
// later (-1: all loads, the normal state).  A kernel whose wait runs out records a code in the error word it was
// given, skips its stores, still meets every barrier, frees its tensor memory and returns; the context stays usable.
KF_API int kf_test_gemm_give_up(unsigned long long limit_ns, int drop_from_stage) {
  const unsigned long long lim = limit_ns ? limit_ns : WAIT_LIMIT_NS;
  if (cudaMemcpyToSymbol(g_wait_limit_ns, &lim, sizeof(lim)) != cudaSuccess ||
      cudaMemcpyToSymbol(g_test_drop_from_stage, &drop_from_stage, sizeof(int)) != cudaSuccess) {
    kf_record_cuda_error(cudaGetLastError());
    return KF_ERR_SETUP;
  }
  return KF_OK;
}

// Whether the q,k,v product of this step can rotate and file its own result: head size 256 or 128 rotated in full, bfloat16
// everywhere, and so many rows that the product runs as whole tiles on CTA pairs.
KF_API int kf_linear_rope_append_supported(const void* x, const void* w, int T, int K, int n_heads, int n_kv_heads, int head_dim, int rot) {
  if (!g_pair || !g_pair_rope || (head_dim != 2 * BM && head_dim != BM) || rot != head_dim || T <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || encode_fn() == nullptr) return 0;
  int bn = 0, splits = 0;
  if (plan_linear(T, (n_heads + 2 * n_kv_heads) * head_dim, K, 0, &bn, &splits) != KF_OK) return 0;
  return bn == 256 && splits == 1;
}

// x[T, K] . w[(n_heads + 2 n_kv_heads) * d, K]^T with q and k rotated (pairs i, i + d / 2; cos, sin [T, d / 2] by row), q
// written to q_out[T, n_heads * d] and k, v into the pages of the rows' requests (if write_kv); all bfloat16, d 256 or 128.
KF_API int kf_linear_rope_append(const void* x, const void* w, int T, int K, int n_heads, int n_kv_heads, int head_dim, const float* cos_t,
                                 const float* sin_t, const int* positions, const int* row_req, const int* block_table,
                                 int table_stride, int page_size, void* pages, void* q_out, int write_kv, int* error_flag,
                                 cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (!kf_linear_rope_append_supported(x, w, T, K, n_heads, n_kv_heads, head_dim, head_dim) || !cos_t || !sin_t) return KF_ERR_SIZE;
  const int N = (n_heads + 2 * n_kv_heads) * head_dim;
  const int hpc = 2 * BM / head_dim;                              // heads per CTA: 1 or 2
  // Token tile: with 256 tokens a pair's tile is two heads x 256 tokens, twice a plain tile, and its two accumulators fill
  // tensor memory (no epilogue under the next tile's products); with 128 tokens two sets fit and tiles are as many as plain
  // ones.  Measured beside the two-kernel path (us per launch, 16 heads of 256 over 2304 / 32 heads over 3584): 768 rows
  // 25.2 -> 34.1 (256) / 23.7 (128) and 54.6 -> 47.0 / 58.3; 2,048 rows 43.6 -> 35.5 / 41.1 and 112.4 -> 94.5 / 111.2: the
  // large tile wherever its tiles occupy most pairs.
  const int tiles256 = kf_ceil_div(n_heads + 2 * n_kv_heads, 2 * hpc) * kf_ceil_div(T, 256);
  const int pn = g_rope_pn ? g_rope_pn : (tiles256 * 5 >= (kf_sm_count() / 2) * 3 ? 256 : 128);
  CUtensorMap tw, txp;
  if (!tensor_map(w, N, K, BM / hpc, &tw) || !tensor_map(x, T, K, pn / 2, &txp)) return KF_ERR_SETUP;
  RopeArgs ra;
  ra.half = head_dim / 2;
  ra.cos_t = cos_t;
  ra.sin_t = sin_t;
  ra.positions = positions;
  ra.row_req = row_req;
  ra.block_table = block_table;
  ra.table_stride = table_stride;
  ra.page_size = page_size;
  ra.nh = n_heads;
  ra.nkv = n_kv_heads;
  ra.write_kv = write_kv;
  ra.pages = (__nv_bfloat16*)pages;
  ra.q_out = (__nv_bfloat16*)q_out;
  return pn == 128 ? launch_pair_rope<128>(tw, txp, T, N, K, ra, error_flag, stream)
                   : launch_pair_rope<256>(tw, txp, T, N, K, ra, error_flag, stream);
}

// Whether the tensor-core kernel takes this product: bfloat16 operands, rows a multiple of 16 bytes, aligned bases.
KF_API int kf_linear_tc_supported(const void* x, const void* w, int K) {
  return (K % 8 == 0) && (((uintptr_t)x & 15) == 0) && (((uintptr_t)w & 15) == 0) && encode_fn() != nullptr;
}

// Choice of token tile and split-K for a launch; also used by the caller to size the partial buffer.
KF_API int kf_linear_tc_plan(int T, int N_features, int K, int gated, int* bn_out, int* splits_out) {
  return plan_linear(T, N_features, K, gated, bn_out, splits_out);
}

// mode: 0 = 32-bit out (softcap > 0 applies the cap), 1 = bfloat16 out, 2 = gated: w = [gate; up] stacked
// ([2*N, K]), out[T, N] = act(gate) * up in bfloat16.  `partial` must hold splits * T * (gated ? 2N : N) floats when
// the plan says splits > 1; `counters` one zero-initialised int per output tile (they are left zero).
KF_API int kf_linear_tc(const void* x, const void* w, void* out, int mode, int T, int N, int K, float softcap, int act,
                        int bn, int splits, float* partial, int* counters, int* error_flag, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return KF_OK;
  if (K <= 0 || K % 8 != 0) return KF_ERR_SIZE;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return KF_ERR_ALIGN;
  if (splits > 1 && (!partial || !counters)) return KF_ERR_SIZE;
  const int w_rows = mode == EPI_GATED ? 2 * N : N;
  CUtensorMap tw, tx;
  if (!tensor_map(w, w_rows, K, BM, &tw) || !tensor_map(x, T, K, bn, &tx)) return KF_ERR_SETUP;
  const int up_offset = mode == EPI_GATED ? N : 0;
  if (g_pair && g_pair_split && bn == 256 && (splits == 2 || splits == 4) && mode != EPI_GATED && ((uintptr_t)out & 15) == 0 &&
      (K + BK - 1) / BK >= splits) {
    // a few hundred tokens: one tile per cluster of 2 x splits CTAs, K cut between the pairs
    CUtensorMap txp;
    if (!tensor_map(x, T, K, 128, &txp)) return KF_ERR_SETUP;
    const int nkb = (K + BK - 1) / BK, kb_per = (nkb + splits - 1) / splits;
    const int sp = (nkb + kb_per - 1) / kb_per;                    // no empty split
    if (sp == splits) {
      if (mode == EPI_F32) return launch_pair_split<EPI_F32>(tw, txp, out, T, N, K, N, softcap, splits, error_flag, stream);
      return launch_pair_split<EPI_BF16>(tw, txp, out, T, N, K, N, softcap, splits, error_flag, stream);
    }
  }
  if (g_pair && splits == 1 && bn == 256) {
    // many tokens: CTA pairs; every CTA loads boxes of 128 rows (its weight rows, its half of the token tile)
    CUtensorMap txp;
    if (!tensor_map(x, T, K, 128, &txp)) return KF_ERR_SETUP;
    if (mode == EPI_F32) return launch_pair<EPI_F32>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream);
    if (mode == EPI_BF16) return launch_pair<EPI_BF16>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream);
    return launch_pair<EPI_GATED>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream);
  }
  if (g_persistent && splits == 1 && bn >= 128 && !(mode == EPI_GATED && bn == 256 && g_gated_wide)) {
    // many tokens: the persistent kernel with two accumulator sets.  The gated epilogue needs two accumulators per
    // set, so its token tile is 128; the token tensor map must match the tile.
    const int pbn = (mode == EPI_GATED) ? 128 : bn;
    CUtensorMap txp = tx;
    if (pbn != bn && !tensor_map(x, T, K, pbn, &txp)) return KF_ERR_SETUP;
    if (mode == EPI_F32) return pbn == 256 ? launch_persistent<256, EPI_F32>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream)
                                            : launch_persistent<128, EPI_F32>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream);
    if (mode == EPI_BF16) return pbn == 256 ? launch_persistent<256, EPI_BF16>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream)
                                             : launch_persistent<128, EPI_BF16>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream);
    return launch_persistent<128, EPI_GATED>(tw, txp, out, T, N, K, N, softcap, act, up_offset, error_flag, stream);
  }
  switch (mode) {
    case EPI_F32: return launch_bn<EPI_F32>(bn, tw, tx, out, T, N, K, N, softcap, act, up_offset, splits, partial, counters, error_flag, stream);
    case EPI_BF16: return launch_bn<EPI_BF16>(bn, tw, tx, out, T, N, K, N, softcap, act, up_offset, splits, partial, counters, error_flag, stream);
    case EPI_GATED: return launch_bn<EPI_GATED>(bn, tw, tx, out, T, N, K, N, softcap, act, up_offset, splits, partial, counters, error_flag, stream);
  }
  return KF_ERR_SIZE;
}
