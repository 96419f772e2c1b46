// A chain of bfloat16 products over few rows (decode) in ONE persistent kernel: the weight stream never stops.
//
// A decode step is a string of small products, each of which only streams its weight matrix through the tensor cores
// once.  Run as one kernel per product, every boundary costs the stream a few microseconds (the epilogue, the kernel
// boundary, the next kernel's first loads), in which an SM takes in nothing; at a few microseconds per product that is
// a third of the time.  Here up to CH_MAX_PHASES products that follow one another run as phases of one kernel:
//   warp 0   : one lane walks ALL phases' weight tiles in order and keeps the ring of 16 KB stages full by TMA; it
//              never waits for anything but a free stage, so weights of phase p+1 arrive while phase p still ends
//   warp 1   : one lane issues the tcgen05.mma's of the CTA's work item (128 features x 16 tokens x its K range)
//   warps 2-5: fill the item's activation rows into shared memory (plain bfloat16 rows, or rows a pending norm
//              defines, see NormIn), run the epilogue (split-K sums through the cluster's shared memory, activation,
//              store) and meet the other CTAs at a grid-wide barrier between phases
// Work item i of a phase = (feature tile i / splits, K split i % splits); CTA c takes items c, c + n_ctas, ...  The
// splits of a tile are consecutive CTAs of one cluster of 8, which sum their partial tiles in split order out of one
// another's shared memory (remote mbarriers say when a partial tile is parked and when it has been read).
// All CTAs must be resident at once (the host checks the occupancy of clusters before it uses this kernel).  Every wait
// is bounded; a wait that runs out records an error code, and every later wait of the CTA gives up at once.
// The reference has no counterpart: it launches one kernel per product (crates/kf-backend-cuda/src/exec.rs:1-60).
#include "common.cuh"
#include "tc_common.cuh"
#include <cuda.h>

using namespace kf_tc;

namespace {

constexpr int CH_BN = 16;                        // token rows of the tile
constexpr int CH_MAX_PHASES = 6;
constexpr int CH_CLUSTER = 8;
constexpr int CH_STAGE = BM * BK * 2;             // 16 KB: one weight tile
constexpr int CH_X_TILE = CH_BN * 128;            // 2 KB: the rows of one k block
constexpr int CH_MAX_X_TILES = 32;                // k blocks of one work item
constexpr int CH_COLS = 32;                       // tensor-memory columns per accumulator
enum { ERR_CH_EMPTY = 11, ERR_CH_FULL = 12, ERR_CH_ACC = 13, ERR_CH_X = 14, ERR_CH_GRID = 15, ERR_CH_RED = 16 };

struct ChainPhase {
  int n_out;                 // output features (gated: of act(gate) * up)
  int K;
  int mode;                  // EPI_F32, EPI_BF16, EPI_GATED
  int act;
  float softcap;
  int splits;                // 1, 2, 4 or 8
  int n_ft;                  // feature tiles
  int kb_per;                // k blocks per split
  int nkb_total;
  int ld_out;
  void* out;
  const __nv_bfloat16* x;    // [T, K] rows, or null: the rows come from `norm`
  NormIn norm;
};

struct ChainArgs {
  int n_phases, T, stages, n_ctas, x_bytes;
  int* gbar;                 // two ints, zero before the launch and left zero
  int* error_flag;
  ChainPhase ph[CH_MAX_PHASES];
};

struct ChainMaps {
  CUtensorMap w[CH_MAX_PHASES];
};

__global__ void __launch_bounds__(THREADS, 1)
gemm_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* xs = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // rows of the item; later its partial tile
  uint8_t* ring = xs + a.x_bytes;
  const int stages = a.stages;
  uint64_t* full = (uint64_t*)(ring + (size_t)stages * CH_STAGE);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint64_t* x_ready = acc_full + 1;
  uint64_t* red_ready = x_ready + 1;              // all splits of my tile have parked their partial tiles
  uint64_t* red_free = red_ready + 1;             // all splits of my tile have read mine
  uint32_t* tmem_slot = (uint32_t*)(red_free + 1);
  volatile int* s_abort = (volatile int*)(tmem_slot + 1);
  float* s_red = (float*)(tmem_slot + 4);          // 128 floats for the norm's row sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, n_ctas = a.n_ctas;
  const int T = a.T;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(x_ready, 128);
    mbar_init(red_ready, CH_CLUSTER);
    mbar_init(red_free, CH_CLUSTER);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * CH_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // peers' barriers exist before anyone arrives on them
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  kf_pdl_trigger();

  if (warp == 0) {
    // ---- weight stream: every tile of every phase, in the order the MMA warp uses them ------------------------------
    if (lane == 0) {
      for (int p = 0; p < a.n_phases; ++p) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.w[p]) : "memory");
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int p = 0; p < a.n_phases && ok; ++p) {
        const ChainPhase& P = a.ph[p];
        const int items = P.n_ft * P.splits;
        const int nacc = P.mode == EPI_GATED ? 2 : 1;
        for (int i = cta; i < items && ok; i += n_ctas) {
          const int tile = i / P.splits, z = i - tile * P.splits;
          const int kb0 = z * P.kb_per, kb1 = min(P.nkb_total, kb0 + P.kb_per);
          for (int kb = kb0; kb < kb1 && ok; ++kb) {
            for (int half = 0; half < nacc; ++half) {
              if (*s_abort || !mbar_wait(&empty[s], ph ^ 1)) {
                if (!*s_abort) atomicExch(a.error_flag, ERR_CH_EMPTY);
                *s_abort = 1;
                ok = false;
                break;
              }
              mbar_expect_tx(&full[s], CH_STAGE);
              tma_load_2d(ring + (size_t)s * CH_STAGE, &maps.w[p], &full[s], kb * BK, tile * BM + half * P.n_out);
              if (++s == stages) { s = 0; ph ^= 1; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ---------------------------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(CH_BN);
      const uint64_t d_ring = umma_desc(ring), d_x = umma_desc(xs);
      int s = 0;
      uint32_t ph = 0, item_parity = 0;
      bool ok = true;
      for (int p = 0; p < a.n_phases && ok; ++p) {
        const ChainPhase& P = a.ph[p];
        const int items = P.n_ft * P.splits;
        const bool gated = P.mode == EPI_GATED;
        for (int i = cta; i < items && ok; i += n_ctas) {
          const int tile = i / P.splits, z = i - tile * P.splits;
          const int kb0 = z * P.kb_per, kb1 = min(P.nkb_total, kb0 + P.kb_per);
          if (*s_abort || !mbar_wait(x_ready, item_parity)) {
            if (!*s_abort) atomicExch(a.error_flag, ERR_CH_X);
            *s_abort = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          for (int kb = kb0; kb < kb1 && ok; ++kb) {
            int sa = s, su = s;
            if (!mbar_wait(&full[s], ph)) ok = false;
            if (++s == stages) { s = 0; ph ^= 1; }
            if (gated && ok) {
              su = s;
              if (!mbar_wait(&full[s], ph)) ok = false;
              if (++s == stages) { s = 0; ph ^= 1; }
            }
            if (!ok) {
              atomicExch(a.error_flag, ERR_CH_FULL);
              *s_abort = 1;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = d_ring + (uint64_t)((uint32_t)sa * (uint32_t)(CH_STAGE >> 4));
            const uint64_t du = d_ring + (uint64_t)((uint32_t)su * (uint32_t)(CH_STAGE >> 4));
            const uint64_t db = d_x + (uint64_t)((uint32_t)(kb - kb0) * (uint32_t)(CH_X_TILE >> 4));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint32_t accumulate = (kb > kb0 || k > 0) ? 1u : 0u;
              umma(tmem_base, da + 2 * k, db + 2 * k, idesc, accumulate);
              if (gated) umma(tmem_base + CH_COLS, du + 2 * k, db + 2 * k, idesc, accumulate);
            }
            umma_commit(&empty[sa]);
            if (gated) umma_commit(&empty[su]);
          }
          umma_commit(acc_full);
          item_parity ^= 1;
        }
      }
    }
  } else {
    // ---- rows in, results out: warps 2..5 ---------------------------------------------------------------------------------
    kf_pdl_wait();                                                 // before any read of what earlier kernels wrote
    const int w4 = warp & 3, tid = w4 * 32 + lane;
    const uint32_t my_rank = cluster_ctarank();
    uint32_t item_parity = 0, red_parity = 0;
    bool red_pending = false;                                      // peers may still read my last partial tile
    bool ok = true;
    auto fail = [&](int code) {
      if (!*s_abort) atomicExch(a.error_flag, code);
      *s_abort = 1;
      ok = false;
    };
    for (int p = 0; p < a.n_phases; ++p) {
      const ChainPhase& P = a.ph[p];
      if (p > 0) {
        // ---- grid-wide barrier: what phase p-1 stored is visible to every CTA --------------------------------------------
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid == 0) {
          __threadfence();
          atomicAdd(a.gbar, 1);
          const int target = n_ctas * p;
          bool arrived = false;
          unsigned long long t0 = 0;
          for (int it = 0; it < WAIT_LIMIT && !*s_abort; ++it) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(a.gbar) : "memory");
            if (v >= target) { arrived = true; break; }
            if ((it & 255) == 255) {
              const unsigned long long now = global_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > WAIT_LIMIT_NS) break;
            }
          }
          if (!arrived) fail(ERR_CH_GRID);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      ok = ok && !*s_abort;
      const int items = P.n_ft * P.splits;
      const bool gated = P.mode == EPI_GATED;
      const int S = P.splits;
      for (int i = cta; i < items; i += n_ctas) {
        const int tile = i / S, z = i - tile * S;
        const int kb0 = z * P.kb_per, kb1 = min(P.nkb_total, kb0 + P.kb_per);
        const int nkb = kb1 - kb0;
        // ---- the item's rows ---------------------------------------------------------------------------------------
        if (red_pending) {                                         // xs is also my partial tile: peers must be done with it
          if (ok && !mbar_wait_cluster(red_free, red_parity ^ 1)) fail(ERR_CH_RED);
          red_pending = false;
        }
        if (ok) {
          if (P.x != nullptr) {
            copy_rows_to_smem<CH_BN>(P.x, T, P.K, kb0, nkb, xs, tid);
          } else if (T <= 8) {
            normed_rows_to_smem<CH_BN, 8>(P.norm, T, P.K, kb0, nkb, xs, tile == 0, w4, lane, s_red);
          } else {
            normed_rows_to_smem<CH_BN, 16>(P.norm, T, P.K, kb0, nkb, xs, tile == 0, w4, lane, s_red);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(x_ready);
        // ---- the accumulator --------------------------------------------------------------------------------------------
        if (ok && !mbar_wait(acc_full, item_parity)) fail(ERR_CH_ACC);
        item_parity ^= 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int f = tile * BM + tid;                             // this thread's output feature
        const uint32_t lane_addr = tmem_base + ((uint32_t)(w4 * 32) << 16);
        auto finish = [&](float v, float u) -> float {
          if (gated) return act_fast(v, P.act) * u;
          if (P.mode == EPI_F32) return kf_softcap(v, P.softcap);
          return v;
        };
        auto store = [&](int t, float r) {
          if (P.mode == EPI_F32) ((float*)P.out)[(size_t)t * P.ld_out + f] = r;
          else ((__nv_bfloat16*)P.out)[(size_t)t * P.ld_out + f] = __float2bfloat16_rn(r);
        };
        float v[16], u[16];
        if (ok) {
          tmem_ld16(lane_addr, v);
          if (gated) tmem_ld16(lane_addr + CH_COLS, u);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (S == 1) {
          if (ok && f < P.n_out) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (j < T) store(j, finish(v[j], gated ? u[j] : 0.f));
          }
        } else {
          // ---- split-K: park the partial tile, tell the peers, sum my share of the tokens in split order ---------------
          float* red = reinterpret_cast<float*>(xs);                // [gate|up][16 tokens][128 features]
          if (ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              red[j * BM + tid] = v[j];
              if (gated) red[(16 + j) * BM + tid] = u[j];
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const uint32_t base_rank = my_rank - (uint32_t)z;
          if (tid < S) mbar_arrive_remote(red_ready, base_rank + tid, CH_CLUSTER / S);
          if (ok && !mbar_wait_cluster(red_ready, red_parity)) fail(ERR_CH_RED);
          if (ok) {
            const uint32_t red_addr = smem_u32(red);
            uint32_t remote[CH_CLUSTER];
#pragma unroll
            for (int q = 0; q < CH_CLUSTER; ++q) remote[q] = map_to_cta(red_addr, base_rank + (q < S ? q : 0));
            const int t_hi = min(16, T);
            for (int tl = z; tl < t_hi; tl += S) {
              float pv[CH_CLUSTER], pu[CH_CLUSTER];
              const uint32_t off = (uint32_t)((tl * BM + tid) * 4), off_u = (uint32_t)(((16 + tl) * BM + tid) * 4);
#pragma unroll
              for (int q = 0; q < CH_CLUSTER; ++q) {
                pv[q] = 0.f;
                pu[q] = 0.f;
                if (q < S) {
                  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv[q]) : "r"(remote[q] + off) : "memory");
                  if (gated) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pu[q]) : "r"(remote[q] + off_u) : "memory");
                }
              }
              float sv = 0.f, su = 0.f;
#pragma unroll
              for (int q = 0; q < CH_CLUSTER; ++q) { sv += pv[q]; su += pu[q]; }
              if (f < P.n_out) store(tl, finish(sv, su));
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");                 // all of my reads of the peers are done
          if (tid < S) mbar_arrive_remote(red_free, base_rank + tid, CH_CLUSTER / S);
          red_parity ^= 1;
          red_pending = true;
        }
      }
    }
    if (red_pending && ok) {
      if (!mbar_wait_cluster(red_free, red_parity ^ 1)) fail(ERR_CH_RED);
    }
    // ---- leave the grid barrier's counters as they were found ---------------------------------------------------------
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(a.gbar + 1, 1) == n_ctas - 1) {
        a.gbar[0] = 0;
        a.gbar[1] = 0;
        __threadfence();
      }
    }
  }
  // ---- common exit ------------------------------------------------------------------------------------------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // nobody's shared memory goes away under a peer
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * CH_COLS) : "memory");
  }
}

// ---- host ----------------------------------------------------------------------------------------------------------------
int g_chain_clusters = -1;                        // clusters of 8 that are resident at once with the kernel's full footprint

int resident_clusters() {
  if (g_chain_clusters >= 0) return g_chain_clusters;
  g_chain_clusters = 0;
  if (cudaFuncSetAttribute(gemm_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) {
    kf_record_cuda_error(cudaGetLastError());
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CH_CLUSTER * 32);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_LIMIT;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CH_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_chain_kernel, &cfg) != cudaSuccess) {
    kf_record_cuda_error(cudaGetLastError());
    return 0;
  }
  g_chain_clusters = n;
  return n;
}

// Split count of one phase for a grid of n_ctas: the largest of 8, 4, 2, 1 whose items fit the grid in one round, raised
// as far as the rows of one item must fit their shared-memory region.  0 if nothing fits.
int chain_splits(int n_out, int K, int n_ctas) {
  const int n_ft = kf_ceil_div(n_out, BM), nkb = K / BK;
  int best = 0;
  for (int s = 1; s <= CH_CLUSTER; s *= 2) {
    if (s > nkb) break;
    const int kb_per = kf_ceil_div(nkb, s);
    if (kf_ceil_div(nkb, kb_per) != s) continue;                 // an empty split
    if (kb_per > CH_MAX_X_TILES) continue;
    if (best == 0 || n_ft * s <= n_ctas) best = s;
  }
  return best;
}

}  // namespace

// One product of a chain, as the caller describes it.
struct KfChainOp {
  const void* w;             // [rows, K] bfloat16; gated: gate rows then up rows, rows = 2 * n_out
  const void* x;             // [T, K] bfloat16 rows, or null: rows from the pending norm below
  void* out;                 // [T, n_out]: 32-bit (mode 0) or bfloat16 (modes 1, 2)
  int n_out, K, mode, act;
  float softcap;
  const float* branch;       // pending norm (see NormIn in tc_common.cuh); used when x is null
  const float* res_in;
  float* res_out;
  const void* w_post;
  const void* w_next;
  float eps_post, eps_next;
  int plus_post, plus_next;
};

// Whether a product of this shape can be a phase of a chain over T rows.
KF_API int kf_linear_chain_supported(int T, int n_out, int K) {
  if (T < 1 || T > CH_BN || n_out < 1 || K < BK || K % BK != 0 || !tensor_maps_available()) return 0;
  const int nc = resident_clusters();
  if (nc < 1) return 0;
  const int n_ctas = (nc < 148 / CH_CLUSTER ? nc : 148 / CH_CLUSTER) * CH_CLUSTER;
  return chain_splits(n_out, K, n_ctas) > 0 ? 1 : 0;
}

KF_API int kf_linear_chain_max_phases() { return CH_MAX_PHASES; }

// Runs ops[0..n) one after the other over the same T rows as one kernel.  gbar: two zero ints (left zero).
KF_API int kf_linear_chain(const KfChainOp* ops, int n, int T, int* gbar, int* error_flag, cudaStream_t stream) {
  if (n < 1 || n > CH_MAX_PHASES || T < 1 || T > CH_BN || !gbar || !error_flag) return KF_ERR_SIZE;
  const int nc = resident_clusters();
  if (nc < 1) return KF_ERR_SETUP;
  const int n_ctas = (nc < 148 / CH_CLUSTER ? nc : 148 / CH_CLUSTER) * CH_CLUSTER;
  ChainMaps maps;
  ChainArgs a = {};
  a.n_phases = n;
  a.T = T;
  a.n_ctas = n_ctas;
  a.gbar = gbar;
  a.error_flag = error_flag;
  int x_tiles = 8;                                                // the region also holds a partial tile (16 KB)
  for (int p = 0; p < n; ++p) {
    const KfChainOp& o = ops[p];
    if (o.n_out < 1 || o.K < BK || o.K % BK != 0 || o.mode < EPI_F32 || o.mode > EPI_GATED || !o.w || !o.out) return KF_ERR_SIZE;
    if (((uintptr_t)o.w & 15) || ((uintptr_t)o.x & 15) || ((uintptr_t)o.out & 15)) return KF_ERR_ALIGN;
    ChainPhase& P = a.ph[p];
    P.n_out = o.n_out;
    P.K = o.K;
    P.mode = o.mode;
    P.act = o.act;
    P.softcap = o.softcap;
    P.splits = chain_splits(o.n_out, o.K, n_ctas);
    if (P.splits < 1) return KF_ERR_SIZE;
    P.n_ft = kf_ceil_div(o.n_out, BM);
    P.nkb_total = o.K / BK;
    P.kb_per = kf_ceil_div(P.nkb_total, P.splits);
    P.ld_out = o.n_out;
    P.out = o.out;
    P.x = (const __nv_bfloat16*)o.x;
    if (!o.x) {
      if (!o.branch || !o.res_in || !o.res_out || o.res_in == o.res_out || !o.w_post || !o.w_next) return KF_ERR_SIZE;
      if (((uintptr_t)o.branch & 15) || ((uintptr_t)o.res_in & 15) || ((uintptr_t)o.res_out & 15) ||
          ((uintptr_t)o.w_post & 15) || ((uintptr_t)o.w_next & 15)) return KF_ERR_ALIGN;
      P.norm.branch = o.branch; P.norm.res_in = o.res_in; P.norm.res_out = o.res_out;
      P.norm.w_post = (const __nv_bfloat16*)o.w_post; P.norm.w_next = (const __nv_bfloat16*)o.w_next;
      P.norm.eps_post = o.eps_post; P.norm.eps_next = o.eps_next;
      P.norm.plus_post = o.plus_post; P.norm.plus_next = o.plus_next;
    }
    if (P.kb_per > x_tiles) x_tiles = P.kb_per;
    const int w_rows = o.mode == EPI_GATED ? 2 * o.n_out : o.n_out;
    if (!tensor_map(o.w, w_rows, o.K, BM, &maps.w[p])) return KF_ERR_SETUP;
  }
  for (int p = n; p < CH_MAX_PHASES; ++p) maps.w[p] = maps.w[0];
  a.x_bytes = x_tiles * CH_X_TILE;
  int stages = (SMEM_LIMIT - 2048 - a.x_bytes) / CH_STAGE;
  if (stages > 12) stages = 12;
  if (stages < 2) return KF_ERR_SIZE;
  a.stages = stages;
  const size_t smem = (size_t)a.x_bytes + (size_t)stages * CH_STAGE + 1024 + 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ctas);
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
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = CH_CLUSTER;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaLaunchKernelEx(&cfg, gemm_chain_kernel, maps, a);
  KF_CHECK_LAUNCH();
  return KF_OK;
}
