// Prompt-portion attention on the 5th-generation tensor cores: S = Q K^T and O += P V as tcgen05.mma with both
// accumulators in tensor memory, keys and values fetched page by page with TMA.
//
// A block is (tile of up to 128 consecutive rows of one request, query head).  Keys are walked in tiles of 64, which
// is one cache page (or a 64-aligned part of one), so a tile is a handful of TMA boxes [64 keys x 64 elements].
//   warp 8   : one lane issues the TMA loads of the Q tile (once) and of the K tiles into a two-stage ring
//   warp 11  : one lane issues the TMA loads of the V tiles into a ring of their own
//   warp 10  : one lane issues S_i = Q K_i^T (M 128, N 64, K = head size) into S buffer i % 2 as soon as the keys are
//              there and the softmax group has taken S_(i-2) out of that buffer: long before P_(i-2) is complete, so
//              the group finds its next scores waiting
//   warp 9   : allocates tensor memory; one lane issues O += P_i V_i (M 128, N = head size, K 64) with V as an
//              MN-major operand, as soon as P_i and the values are there
//   warps 0-7: two groups of four warps, one thread per query row (= tensor-memory lane) in each.  Group g takes the
//              key tiles i with i % 2 == g (which land in S buffer g): read the row of S, scale, cap, mask, take the
//              maximum, exponentiate, add to the group's sum, round P to bfloat16 into swizzled shared memory for the
//              second MMA.  The groups are out of step by half a tile, so while one waits (for S, for tensor memory,
//              for P V) the other has arithmetic to issue.  The row's running maximum, to which O is scaled, is one
//              word in shared memory that the groups hand to each other tile by tile.  At the end each thread reads
//              half of O's columns of its row, divides by the sum and stores.
// The running maximum used for the exponentials is only raised when a tile's maximum exceeds it by more than 8
// (a factor 256, harmless in bfloat16/32-bit accumulators); only then is O in tensor memory rescaled.  All of S, the
// softmax and the sums are 32-bit.  Every wait is bounded; on a timeout an error code is recorded and the block
// leaves through the common exit that frees tensor memory.
// Head sizes 64, 128, 256; page sizes that are multiples of 64.  Everything else runs the mma.sync kernel.
// Reference counterpart: crates/kf-backend-cuda/src/kernels/flash.cu (Ampere mma.sync on f16).
#include "common.cuh"
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

namespace {

constexpr int BMQ = 128;           // query rows per block
constexpr int BKV = 64;            // keys per tile
constexpr int THREADS = 384;
constexpr int SOFTMAX_THREADS = 256;
constexpr long WAIT_LIMIT = 20L * 1000 * 1000;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;
enum { ERR_ATTN_WAIT = 16 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (long i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(const void* smem) {
  uint64_t d = (uint64_t)((smem_u32(smem) & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand, 128-byte swizzle: a row of 128 bytes holds 64 consecutive N elements of one K index (one key);
// 8 keys form a 1024-byte group (stride byte offset), the next 64 N elements start `mn_block_bytes` further
// (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(const void* smem, uint32_t mn_block_bytes) {
  uint64_t d = (uint64_t)((smem_u32(smem) & 0x3FFFF) >> 4);
  d |= (uint64_t)(mn_block_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: D = f32, A = B = bf16, M = 128, N = n; b_mn = 1 makes B MN-major.
__device__ __forceinline__ uint32_t idesc(int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t id, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// max(a, b, c) in one instruction (three-input maximum of sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// cap * tanh(s / cap) in base-2 units for two scores with |s * ct| <= 1 (ct = scale / cap, c4 = cap * log2(e) * ct):
// tanh(t) = t * P(t^2), P of degree 6 fitted on Chebyshev nodes of [0, 1] (relative error 1.8e-7 in 32-bit Horner form,
// below that of the exp2 / reciprocal form), evaluated on the packed 32-bit pipe: no special-function unit.
__device__ __forceinline__ float2 capped2(float2 s, float ct, float c4) {
  const float2 t = __fmul2_rn(s, make_float2(ct, ct));
  const float2 u = __fmul2_rn(t, t);
  float2 p = __ffma2_rn(u, make_float2(1.045553596e-03f, 1.045553596e-03f), make_float2(-6.217069924e-03f, -6.217069924e-03f));
  p = __ffma2_rn(p, u, make_float2(2.030551992e-02f, 2.030551992e-02f));
  p = __ffma2_rn(p, u, make_float2(-5.346517637e-02f, -5.346517637e-02f));
  p = __ffma2_rn(p, u, make_float2(1.332539767e-01f, 1.332539767e-01f));
  p = __ffma2_rn(p, u, make_float2(-3.333285749e-01f, -3.333285749e-01f));
  p = __ffma2_rn(p, u, make_float2(9.999999404e-01f, 9.999999404e-01f));
  return __fmul2_rn(__fmul2_rn(s, make_float2(c4, c4)), p);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive columns of this thread's lane, one wait for all four loads
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
  uint32_t r[64];
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[16 * q + 0]), "=r"(r[16 * q + 1]), "=r"(r[16 * q + 2]), "=r"(r[16 * q + 3]), "=r"(r[16 * q + 4]),
          "=r"(r[16 * q + 5]), "=r"(r[16 * q + 6]), "=r"(r[16 * q + 7]), "=r"(r[16 * q + 8]), "=r"(r[16 * q + 9]),
          "=r"(r[16 * q + 10]), "=r"(r[16 * q + 11]), "=r"(r[16 * q + 12]), "=r"(r[16 * q + 13]), "=r"(r[16 * q + 14]),
          "=r"(r[16 * q + 15])
        : "r"(taddr + 16 * q));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 consecutive columns of this thread's lane, one wait for both loads
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
#pragma unroll
  for (int q = 0; q < 2; ++q)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[16 * q + 0]), "=r"(r[16 * q + 1]), "=r"(r[16 * q + 2]), "=r"(r[16 * q + 3]), "=r"(r[16 * q + 4]),
          "=r"(r[16 * q + 5]), "=r"(r[16 * q + 6]), "=r"(r[16 * q + 7]), "=r"(r[16 * q + 8]), "=r"(r[16 * q + 9]),
          "=r"(r[16 * q + 10]), "=r"(r[16 * q + 11]), "=r"(r[16 * q + 12]), "=r"(r[16 * q + 13]), "=r"(r[16 * q + 14]),
          "=r"(r[16 * q + 15])
        : "r"(taddr + 16 * q));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])) : "memory");
}

// The 64-key tiles a tile of query rows reads (and its first key), and into how many runs they are cut: `n_parts` runs for
// every tile when `run_tiles` is 0; otherwise as many runs of at most `run_tiles` key tiles as the tile needs, at most
// n_parts (short tiles then stay whole and write their rows themselves, long ones are shared between blocks).
__device__ __forceinline__ int tile_key_tiles(int row0, int nrows, const int* positions, const int* row_req, int window,
                                              int* kt_first) {
  const int pos0 = positions[row0];
  const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  *kt_first = (lo / BKV) * BKV;
  return (row_req[row0] < 0 || nrows <= 0) ? 0 : (pos0 + nrows - 1 - *kt_first) / BKV + 1;   // padding, or a tile without rows
}
__device__ __forceinline__ int tile_runs(int n_key_tiles, int n_parts, int run_tiles) {
  if (n_parts <= 1) return 1;
  if (run_tiles <= 0) return n_parts;
  const int p = (n_key_tiles + run_tiles - 1) / run_tiles;
  return p < 1 ? 1 : (p > n_parts ? n_parts : p);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                       const int* __restrict__ tile_row0, const int* __restrict__ tile_nrows,
                       const int* __restrict__ positions, const int* __restrict__ row_req,
                       const int* __restrict__ table, int table_stride, int page_size, int nh, int nkv,
                       float scale, float softcap, int window, __nv_bfloat16* __restrict__ out,
                       int* __restrict__ error_flag, int n_parts, int run_tiles, float* __restrict__ partial) {
  constexpr int NSUB = D / 64;                            // 64-element sub-tiles along the head dimension
  constexpr int Q_BYTES = BMQ * D * 2;
  constexpr int KV_BYTES = BKV * D * 2;                   // one K tile (or one V tile)
  constexpr int P_BYTES = BMQ * BKV * 2;
  constexpr int S_COLS = 64;
  constexpr int TMEM_COLS = (2 * S_COLS + D) <= 256 ? 256 : 512;
  constexpr uint32_t O_COL = 2 * S_COLS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;                             // [2][KV_BYTES]
  uint8_t* sV = sK + 2 * KV_BYTES;                        // [2][KV_BYTES]
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = (uint64_t*)(sP + P_BYTES);
  uint64_t* q_full = bars;                                // TMA
  uint64_t* k_full = bars + 1;                            // [2] TMA; keys and values have rings of their own, so that the
  uint64_t* v_full = bars + 3;                            // [2] next keys can load as soon as Q K^T has read the stage,
  uint64_t* k_free = bars + 5;                            // [2] commit after Q K^T of the tile in that stage
  uint64_t* v_free = bars + 7;                            // [2] commit after P V of the tile in that stage
  uint64_t* s_full = bars + 9;                            // [2] commit after Q K^T
  uint64_t* p_full = bars + 11;                           // the softmax group of the tile
  uint64_t* pv_done = bars + 12;                          // [2] commit after P V of tile i on barrier i % 2: a group waits
                                                          // for every other tile, and a parity tells only one phase back
  uint64_t* m_done = bars + 14;                           // [2] group g has published the row maxima after its tile
  uint64_t* s_free = bars + 16;                           // [2] group g has taken its scores out of S buffer g
  uint32_t* tmem_slot = (uint32_t*)(bars + 18);
  volatile int* s_abort = (volatile int*)(tmem_slot + 1);
  float* s_max = (float*)(tmem_slot + 2);                 // [128 rows] the running maximum O is scaled to; then [2][128] sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks are numbered (tile, run, head) with the head fastest and the last tile first: tiles late in a request have
  // the most keys, and blocks start in the order of their numbers.  With n_parts > 1 the keys of a tile are cut into
  // runs, one block each; the blocks of a tile with several runs leave unnormalised partial rows that a second kernel
  // merges, and a block whose run its tile does not have leaves at once.
  const int h = blockIdx.x % nh, slot = blockIdx.x / nh;
  const int tile = (int)(gridDim.x / (nh * n_parts)) - 1 - slot / n_parts, part = slot % n_parts;
  const int row0 = tile_row0[tile], nrows = tile_nrows[tile];
  const int kvh = h / (nh / nkv);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_free[s], 1); mbar_init(&v_free[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_full, SOFTMAX_THREADS / 2);
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    mbar_init(&m_done[0], SOFTMAX_THREADS / 2);
    mbar_init(&m_done[1], SOFTMAX_THREADS / 2);
    mbar_init(&s_free[0], SOFTMAX_THREADS / 2);
    mbar_init(&s_free[1], SOFTMAX_THREADS / 2);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  kf_pdl_trigger();

  // the step's integers were written before the step's first kernel: read before the grid dependency is waited for
  const int req = row_req[row0];
  const int pos0 = positions[row0];
  int kt_first;
  const int n_tiles_all = tile_key_tiles(row0, nrows, positions, row_req, window, &kt_first);
  const int my_parts = tile_runs(n_tiles_all, n_parts, run_tiles);
  const bool idle = part >= my_parts;                     // this tile has fewer runs than the launch has blocks per tile
  const int per_part = (n_tiles_all + my_parts - 1) / my_parts;
  const int kt_begin = kt_first + part * per_part * BKV;
  const int n_tiles = idle ? 0 : max(0, min(per_part, n_tiles_all - part * per_part));
  kf_pdl_wait();                                          // Q, and the keys and values of this step's rows, come from the kernel before

  if (warp == 8) {
    // ---- TMA producer of Q and the keys ----------------------------------------------------------------------
    if (lane == 0 && n_tiles > 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_kv) : "memory");
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int j = 0; j < NSUB; ++j) tma_load_2d(sQ + j * (BMQ * 128), &tm_q, q_full, h * D + j * 64, row0);
      const int* tab = table + (size_t)req * table_stride;
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i & 1;
        const int kt = kt_begin + i * BKV;
        int page = tab[kt / page_size];
        if (page < 0) page = 0;                            // a page already given back: every key of it is masked
        const int krow = ((page * 2 + 0) * nkv + kvh) * page_size + (kt % page_size);
        if (i >= 2 && !mbar_wait(&k_free[s], ((i >> 1) - 1) & 1)) { atomicExch(error_flag, ERR_ATTN_WAIT + 1); *s_abort = 1; break; }
        mbar_expect_tx(&k_full[s], KV_BYTES);
#pragma unroll
        for (int j = 0; j < NSUB; ++j) tma_load_2d(sK + s * KV_BYTES + j * (BKV * 128), &tm_kv, &k_full[s], j * 64, krow);
      }
    }
  } else if (warp == 11) {
    // ---- TMA producer of the values: a thread of its own, so that the next keys never wait for a value stage -----------
    if (lane == 0 && n_tiles > 0) {
      const int* tab = table + (size_t)req * table_stride;
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i & 1;
        const int kt = kt_begin + i * BKV;
        int page = tab[kt / page_size];
        if (page < 0) page = 0;
        const int vrow = ((page * 2 + 1) * nkv + kvh) * page_size + (kt % page_size);
        if (i >= 2 && !mbar_wait(&v_free[s], ((i >> 1) - 1) & 1)) { atomicExch(error_flag, ERR_ATTN_WAIT + 1); *s_abort = 1; break; }
        mbar_expect_tx(&v_full[s], KV_BYTES);
#pragma unroll
        for (int j = 0; j < NSUB; ++j) tma_load_2d(sV + s * KV_BYTES + j * (BKV * 128), &tm_kv, &v_full[s], j * 64, vrow);
      }
    }
  } else if (warp == 10) {
    // ---- issuer of S = Q K^T -------------------------------------------------------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t id_s = idesc(BKV, 0);
      bool ok = mbar_wait(q_full, 0);
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i & 1;
        ok = mbar_wait(&k_full[s], (i >> 1) & 1) && (i < 2 || mbar_wait(&s_free[s], ((i >> 1) - 1) & 1));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int j = 0; j < NSUB; ++j) {
          const uint64_t da = desc_kmajor(sQ + j * (BMQ * 128));
          const uint64_t db = desc_kmajor(sK + s * KV_BYTES + j * (BKV * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem_base + s * S_COLS, da + 2 * k, db + 2 * k, id_s, (j | k) ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_free[s]);
      }
      if (!ok) { atomicExch(error_flag, ERR_ATTN_WAIT + 2); *s_abort = 1; }
    }
  } else if (warp == 9) {
    // ---- issuer of O += P V -----------------------------------------------------------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t id_o = idesc(D, 1);
      bool ok = true;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i & 1;
        ok = mbar_wait(&v_full[s], (i >> 1) & 1) && mbar_wait(p_full, i & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < 4; ++k) {                      // 16 keys per MMA
          const uint64_t da = desc_kmajor(sP) + 2 * k;
          const uint64_t db = desc_mnmajor(sV + s * KV_BYTES + k * 2048, BKV * 128);
          umma(tmem_base + O_COL, da, db, id_o, (i | k) ? 1u : 0u);
        }
        umma_commit(&v_free[s]);
        umma_commit(&pv_done[i & 1]);
      }
      if (!ok) { atomicExch(error_flag, ERR_ATTN_WAIT + 2); *s_abort = 1; }
    }
  } else {
    // ---- softmax and epilogue: group `grp` takes every other key tile; one thread per query row -----------------------
    const int grp = warp >> 2, wq = warp & 3;
    const int half = grp;                                  // in the epilogue: which half of O's columns this thread stores
    const int r = wq * 32 + lane;                          // row of the tile = tensor-memory lane
    const int prow = pos0 + r;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(wq * 32) << 16);
    const float c0 = scale * LOG2E;                                        // no cap: s2 = s * c0
    const float c1 = softcap > 0.f ? scale * 2.f * LOG2E / softcap : 0.f;   // exp(2 x / cap) = exp2(s * c1)
    const float c3 = softcap * LOG2E;
    const float ct = softcap > 0.f ? scale / softcap : 0.f;
    const float c4 = c3 * ct;
    constexpr int HC = D / 2;                              // O columns of this thread in the epilogue
    float m_mine = -INFINITY, l_sum = 0.f;                 // this group's sum of exponentials, scaled to 2^-m_mine
    bool ok = true;
    // A thread runs every turn of its loop and arrives at every barrier of it, also after a wait has run out (the waits
    // are then skipped and the numbers are garbage that nobody stores): nobody is left waiting for it.
    for (int i = grp; i < n_tiles; i += 2) {
      ok = ok && mbar_wait(&s_full[grp], (i >> 1) & 1);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int kt = kt_begin + i * BKV;                   // first key of the tile
      float sv[64];
      tmem_ld64(lane_addr + grp * S_COLS, sv);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&s_free[grp]);                           // the buffer may take the scores of tile i + 2
      // Scores in base-2 units: s2 = log2(e) * cap * tanh(scale * s / cap) = c3 - 2 c3 / (exp2(s * c1) + 1), or
      // s * c0 without a cap.  A tile that every row of this warp sees whole skips the mask.
      const bool whole = (kt + BKV - 1 <= pos0 + wq * 32) && (window <= 0 || pos0 + wq * 32 + 31 - kt < window);
      if (softcap > 0.f) {
        // A cap is chosen beyond what scores usually reach: while every score of this warp's tile is within it
        // (|scale * s / cap| <= 1), tanh is a polynomial on the packed 32-bit pipe; otherwise it goes through exp2 and
        // 1 / x on the special-function unit, which bounds the tile with three of its operations per score.
        float am[4] = {0.f, 0.f, 0.f, 0.f};               // four chains: a single one is 64 dependent operations
#pragma unroll
        for (int c = 0; c < BKV; c += 8) {
          am[0] = max3(am[0], fabsf(sv[c]), fabsf(sv[c + 1])); am[1] = max3(am[1], fabsf(sv[c + 2]), fabsf(sv[c + 3]));
          am[2] = max3(am[2], fabsf(sv[c + 4]), fabsf(sv[c + 5])); am[3] = max3(am[3], fabsf(sv[c + 6]), fabsf(sv[c + 7]));
        }
        const float amax = fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3]));
        if (__all_sync(0xffffffffu, amax * ct <= 1.f)) {
#pragma unroll
          for (int c = 0; c < BKV; c += 2) {
            const float2 y = capped2(make_float2(sv[c], sv[c + 1]), ct, c4);
            sv[c] = y.x, sv[c + 1] = y.y;
          }
        } else {
#pragma unroll
          for (int c = 0; c < BKV; ++c) sv[c] = fmaf(-2.f * c3, rcp_fast(ex2_fast(sv[c] * c1) + 1.f), c3);
        }
      } else {
#pragma unroll
        for (int c = 0; c < BKV; ++c) sv[c] *= c0;
      }
      if (!whole) {
        // key kt + c is seen by this row iff first <= c <= last: one bit per key, tested with constant masks
        const int last = prow - kt;                                        // >= 64: all of the tile
        const int first = window > 0 ? last - window + 1 : 0;              // <= 0: from the tile's first key
        unsigned long long seen = last < 0 ? 0ull : (last >= 63 ? ~0ull : ((2ull << last) - 1ull));
        if (first > 0) seen &= first >= 64 ? 0ull : ~((1ull << first) - 1ull);
        const uint32_t seen_lo = (uint32_t)seen, seen_hi = (uint32_t)(seen >> 32);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          sv[c] = (seen_lo & (1u << c)) ? sv[c] : -INFINITY;
          sv[32 + c] = (seen_hi & (1u << c)) ? sv[32 + c] : -INFINITY;
        }
      }
      float mt[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BKV; c += 8) {
        mt[0] = max3(mt[0], sv[c], sv[c + 1]); mt[1] = max3(mt[1], sv[c + 2], sv[c + 3]);
        mt[2] = max3(mt[2], sv[c + 4], sv[c + 5]); mt[3] = max3(mt[3], sv[c + 6], sv[c + 7]);
      }
      const float m_tile = fmaxf(fmaxf(mt[0], mt[1]), fmaxf(mt[2], mt[3]));
      // the maximum O is scaled to after tile i - 1, from the other group; this tile's goes back the same way
      if (i > 0) ok = ok && mbar_wait(&m_done[grp ^ 1], ((i - 1) >> 1) & 1);
      const float m_used = i > 0 ? s_max[r] : -INFINITY;
      const bool raise = m_tile > m_used + RESCALE_STEP;   // also true for the first finite maximum
      const float m_new = raise ? m_tile : m_used;
      s_max[r] = m_new;
      mbar_arrive(&m_done[grp]);
      const float corr = raise ? ex2_fast(m_used - m_new) : 1.f;   // for O; exp2(-inf) = 0 when nothing was accumulated yet
      const float m_sub = (m_new == -INFINITY) ? 0.f : m_new;      // a row that has seen nothing yet: exp2(-inf - 0) = 0
      const float l_corr = (m_mine == m_new) ? 1.f : ex2_fast(m_mine - m_new);   // this group's sum follows the maximum
      float2 la[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};   // four chains of packed sums; the order is fixed
      const float2 neg_m = make_float2(-m_sub, -m_sub);
      uint32_t pk[BKV / 2];
#pragma unroll
      for (int c = 0; c < BKV; c += 2) {
        const float2 x = __fadd2_rn(make_float2(sv[c], sv[c + 1]), neg_m);
        const float2 pp = make_float2(ex2_fast(x.x), ex2_fast(x.y));
        la[(c >> 1) & 3] = __fadd2_rn(la[(c >> 1) & 3], pp);
        const __nv_bfloat162 b = __floats2bfloat162_rn(pp.x, pp.y);
        pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&b);
      }
      l_sum = l_sum * l_corr + (((la[0].x + la[0].y) + (la[1].x + la[1].y)) + ((la[2].x + la[2].y) + (la[3].x + la[3].y)));
      m_mine = m_new;
      if (i > 0) {                                          // P V of the previous tile must be done: O is at rest, P is free
        ok = ok && mbar_wait(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (__any_sync(0xffffffffu, raise)) {              // rescale this row of O (all lanes of the warp take part)
#pragma unroll 1
          for (int c = 0; c < D; c += 16) {
            float o[16];
            tmem_ld16(lane_addr + O_COL + c, o);
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] *= corr;
            tmem_st16(lane_addr + O_COL + c, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      // the P row -> shared memory, K-major with the 128-byte swizzle (chunk index XOR row % 8)
      uint8_t* prow_ptr = sP + r * 128;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint4 v = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        *reinterpret_cast<uint4*>(prow_ptr + ((q ^ (r & 7)) << 4)) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(p_full);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
    if (!ok) { atomicExch(error_flag, ERR_ATTN_WAIT + 3); *s_abort = 1; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // the row's sum is the two groups' sums, both brought to the last maximum; every softmax thread reaches this
    asm volatile("bar.sync 2, 256;" ::: "memory");          // every tile's maximum has been published
    const float m_used = n_tiles > 0 ? s_max[r] : -INFINITY;
    l_sum = (m_mine == m_used) ? l_sum : l_sum * ex2_fast(m_mine - m_used);
    asm volatile("bar.sync 2, 256;" ::: "memory");          // ... and read by both threads of the row
    s_max[half * BMQ + r] = l_sum;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    l_sum = s_max[r] + s_max[BMQ + r];
    if (idle) {
      // nothing to do and nothing to write
    } else if (my_parts > 1) {
      // ---- one of several runs of keys: leave O as it is (scaled by 2^-m), with m and the sum, for the merge ----------
      const bool run_ok = __all_sync(0xffffffffu, ok && n_tiles > 0 && *s_abort == 0);
      const bool have = run_ok && r < nrows && l_sum > 0.f;     // a row that saw no key in this run leaves m = -inf
      float* rec = partial + (((size_t)(row0 + (r < nrows ? r : 0)) * nh + h) * n_parts + part) * (D + 4);
      if (half == 0 && r < nrows) { rec[D] = have ? m_used : -INFINITY; rec[D + 1] = have ? l_sum : 0.f; }
      if (run_ok) {
#pragma unroll 1
        for (int c = 0; c < HC; c += 16) {
          float o[16];
          tmem_ld16(lane_addr + O_COL + half * HC + c, o);       // every lane of the warp takes part in the load
          if (have) {
#pragma unroll
            for (int e = 0; e < 16; e += 4)
              *reinterpret_cast<float4*>(rec + half * HC + c + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
          }
        }
      }
    } else if (ok && n_tiles > 0 && *s_abort == 0) {
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = out + ((size_t)(row0 + r) * nh + h) * D + half * HC;
#pragma unroll 1
      for (int c = 0; c < HC; c += 16) {
        float o[16];
        tmem_ld16(lane_addr + O_COL + half * HC + c, o);   // every lane of the warp takes part in the load
        if (r < nrows) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
            w[e] = *reinterpret_cast<const uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 9) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Merges the partial rows of the key runs: out = sum_p 2^(m_p - m) O_p / sum_p 2^(m_p - m) l_p, runs in index order.
// One block per (tile, row of the tile); a thread owns groups of four output elements over all heads.
template <int D>
__global__ void __launch_bounds__(128)
attn_prefill_merge_kernel(const float* __restrict__ partial, const int* __restrict__ tile_row0,
                          const int* __restrict__ tile_nrows, const int* __restrict__ positions,
                          const int* __restrict__ row_req, int window, int nh, int n_parts_max, int run_tiles,
                          __nv_bfloat16* __restrict__ out) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int tile = blockIdx.x, r = blockIdx.y;
  if (r >= tile_nrows[tile]) return;
  int kt_first;
  const int n_parts = tile_runs(tile_key_tiles(tile_row0[tile], tile_nrows[tile], positions, row_req, window, &kt_first),
                                n_parts_max, run_tiles);
  if (n_parts == 1) return;                                   // a tile with one run wrote its rows itself
  const int row = tile_row0[tile] + r;
  constexpr int REC = D + 4;
  for (int e = threadIdx.x; e < nh * (D / 4); e += blockDim.x) {
    const int h = e / (D / 4), c4 = e - h * (D / 4);
    const float* rec0 = partial + ((size_t)row * nh + h) * n_parts_max * REC;
    float m = -INFINITY;
    for (int p = 0; p < n_parts; ++p) m = fmaxf(m, rec0[(size_t)p * REC + D]);
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < n_parts; ++p) {
      const float mp = rec0[(size_t)p * REC + D];
      if (mp == -INFINITY) continue;                          // a run that saw no key: its O was never written
      const float w = ex2_fast(mp - m);
      l += rec0[(size_t)p * REC + D + 1] * w;
      const float4 o = *reinterpret_cast<const float4*>(rec0 + (size_t)p * REC + c4 * 4);
      acc.x += o.x * w; acc.y += o.y * w; acc.z += o.z * w; acc.w += o.w * w;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + ((size_t)row * nh + h) * D + c4 * 4) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
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

std::mutex g_mutex;
std::map<std::tuple<const void*, long, long, int>, CUtensorMap> g_maps;

// Row-major [rows, cols] bfloat16 with boxes of [box_rows, 64 elements], 128-byte swizzle.
bool tensor_map(const void* base, long rows, long cols, int box_rows, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto key = std::make_tuple(base, rows, cols, box_rows);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUtensorMap m;
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_maps.size() > 1024) g_maps.clear();
  g_maps[key] = m;
  *out = m;
  return true;
}

template <int D>
int launch(const CUtensorMap& tq, const CUtensorMap& tkv, const int* tile_row0, const int* tile_nrows, int n_tiles,
           const int* positions, const int* row_req, const int* table, int table_stride, int page_size, int nh, int nkv,
           float scale, float softcap, int window, void* out, int* error_flag, int n_parts, int run_tiles,
           float* partial, cudaStream_t stream) {
  const size_t smem = (size_t)BMQ * D * 2 + 4 * (size_t)BKV * D * 2 + (size_t)BMQ * BKV * 2 + 1024 + 256 + 4 * BMQ * 4;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  kf_launch(attn_prefill_tc_kernel<D>, dim3(n_tiles * n_parts * nh), dim3(THREADS), smem, stream, tq, tkv, tile_row0, tile_nrows,
            positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, (__nv_bfloat16*)out,
            error_flag, n_parts, run_tiles, partial);
  KF_CHECK_LAUNCH();
  if (n_parts > 1) {
    kf_launch(attn_prefill_merge_kernel<D>, dim3(n_tiles, BMQ), dim3(128), 0, stream, (const float*)partial, tile_row0,
              tile_nrows, positions, row_req, window, nh, n_parts, run_tiles, (__nv_bfloat16*)out);
    KF_CHECK_LAUNCH();
  }
  return KF_OK;
}

}  // namespace

KF_API int kf_attention_prefill_tc_supported(int d, int page_size, const void* q, const void* pages) {
  return (d == 64 || d == 128 || d == 256) && page_size % 64 == 0 && (((uintptr_t)q & 15) == 0) &&
         (((uintptr_t)pages & 15) == 0) && encode_fn() != nullptr;
}
KF_API int kf_attention_prefill_tc_tile_rows() { return BMQ; }

static int g_forced_parts = 0, g_forced_run_tiles = 0;
#ifdef KF_TUNING
// Measurement hook of a tuning build: a fixed plan instead of the planner's (0, 0 gives its choice back).
KF_API void kf_set_attention_prefill_plan(int parts, int run_tiles) { g_forced_parts = parts, g_forced_run_tiles = run_tiles; }
#endif

// Into how many runs the keys of a tile are cut, and how long a run may be (0: every tile gets `parts` runs).
// Few blocks (tiles x heads fill less than half of the GPU): every tile may be cut so that the blocks fill it; at most 8
// runs, never so many that a run of the longest tile has fewer than two 64-key tiles, and only if the shorter loop
// saves more than the partial rows and their merge cost.
// About one block per SM and long tiles (a whole prompt of 2,048 tokens x 8 heads: the launch lasts as long as the tile
// with the most keys, twice the average): cutting only the tiles longer than 1/2 or 5/8 of the longest in two
// (kf_set_attention_prefill_plan(2, 16 or 20)) measured within +-0.5 % of uncut over the 26-layer step, three or four
// runs slower: the partial rows cost a write, a read and a second kernel.  So such launches stay uncut.
KF_API int kf_attention_prefill_tc_plan(int n_tiles, int nh, int max_keys, int* run_tiles) {
  *run_tiles = 0;
  if (g_forced_parts > 0) { *run_tiles = g_forced_run_tiles; return g_forced_parts; }
  const long blocks = (long)n_tiles * nh;
  const int n_sm = kf_sm_count();
  if (blocks <= 0 || 2 * blocks > n_sm) return 1;
  int parts = (int)(n_sm / blocks);
  if (parts > 8) parts = 8;
  const int key_tiles = (max_keys + BKV - 1) / BKV;
  if (parts > key_tiles / 2) parts = key_tiles / 2;
  if (parts < 1) parts = 1;
  // A key tile takes a block about 0.93 us; partial rows, their merge kernel and its launch about 11 us together.  Of the
  // run counts that fill the GPU the one with the shortest estimate wins, so short prompts stay whole.
  int best = 1;
  float best_us = 0.93f * (float)key_tiles;
  for (int p = 2; p <= parts; ++p) {
    const float us = 0.93f * (float)((key_tiles + p - 1) / p) + 11.f;
    if (us < best_us) { best_us = us; best = p; }
  }
  return best;
}

// q, out: [T, nh*d] bfloat16; pages: [n_pages, 2, nkv, page_size, d] bfloat16.  tile_row0/tile_nrows: tiles of up to 128
// consecutive rows of one request (consecutive positions).  n_parts > 1 cuts a tile's keys into up to that many runs
// (every tile's when run_tiles is 0, else those of tiles with more than run_tiles key tiles);
// `partial` then holds T * nh * n_parts * (d + 4) floats.
KF_API int kf_attention_prefill_tc(const void* q, void* out, const void* pages, long n_pages, int T, const int* tile_row0,
                                   const int* tile_nrows, int n_tiles, const int* positions, const int* row_req,
                                   const int* table, int table_stride, int page_size, int nh, int nkv, int d, float scale,
                                   float softcap, int window, int* error_flag, int n_parts, int run_tiles, float* partial,
                                   cudaStream_t stream) {
  if (n_tiles <= 0) return KF_OK;
  if (nkv < 1 || nh % nkv != 0 || page_size % 64 != 0) return KF_ERR_SIZE;
  if (n_parts < 1 || n_parts > 8 || (n_parts > 1 && !partial) || run_tiles < 0) return KF_ERR_SIZE;
  CUtensorMap tq, tkv;
  if (!tensor_map(q, T, (long)nh * d, BMQ, &tq)) return KF_ERR_SETUP;
  if (!tensor_map(pages, n_pages * 2 * nkv * page_size, d, BKV, &tkv)) return KF_ERR_SETUP;
#define KF_ARGS tq, tkv, tile_row0, tile_nrows, n_tiles, positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, out, error_flag, n_parts, run_tiles, partial, stream
  switch (d) {
    case 64: return launch<64>(KF_ARGS);
    case 128: return launch<128>(KF_ARGS);
    case 256: return launch<256>(KF_ARGS);
  }
#undef KF_ARGS
  return KF_ERR_SIZE;
}
