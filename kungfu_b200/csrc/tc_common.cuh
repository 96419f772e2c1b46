// Device helpers shared by the tcgen05 products: mbarriers with bounded waits, TMA tile loads, shared-memory and
// instruction descriptors, the MMA and tensor-memory instructions and the fast activations.  Everything is inline; the one host function (the cached tensor maps) lives in gemm_tc.cu.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace kf_tc {

constexpr int BM = 128;            // output features per tile (tensor-memory lanes)
constexpr int BK = 64;             // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int WAIT_LIMIT = 40 * 1000 * 1000;

enum { EPI_F32 = 0, EPI_BF16 = 1, EPI_GATED = 2, EPI_ROPE = 3 };
enum { ERR_NONE = 0, ERR_WAIT_FULL = 1, ERR_WAIT_EMPTY = 2, ERR_WAIT_ACC = 3 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false if the phase did not complete within the limit.  try_wait itself may block for a while that
// the hardware chooses, so the limit is a time (about two seconds on the global timer, looked at every 256 turns)
// as well as a count.
constexpr unsigned long long WAIT_LIMIT_NS = 2000ull * 1000ull * 1000ull;
// The limit in force (one copy per translation unit).  A test shortens it through the translation unit's hook to see a
// wait give up; nothing else writes it.
static __device__ unsigned long long g_wait_limit_ns = WAIT_LIMIT_NS;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  unsigned long long t0 = 0;
  for (int i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 255) == 255) {
      const unsigned long long now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > g_wait_limit_ns) return false;
    }
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(const void* smem) {
  const uint32_t a = smem_u32(smem);
  uint64_t d = 0;
  d |= (uint64_t)((a & 0x3FFFF) >> 4);          // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset
  d |= (uint64_t)1 << 46;                       // version
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16: D = f32, A = B = bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// 32 consecutive columns of this thread's lane with one wait for both loads (the wait is most of a load's cost)
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
// Two 32-column ranges (gate and up accumulators) with one wait
__device__ __forceinline__ void tmem_ld32x2(uint32_t ta, uint32_t tb, float* v, float* u) {
  uint32_t r[64];
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[16 * q + 0]), "=r"(r[16 * q + 1]), "=r"(r[16 * q + 2]), "=r"(r[16 * q + 3]), "=r"(r[16 * q + 4]),
          "=r"(r[16 * q + 5]), "=r"(r[16 * q + 6]), "=r"(r[16 * q + 7]), "=r"(r[16 * q + 8]), "=r"(r[16 * q + 9]),
          "=r"(r[16 * q + 10]), "=r"(r[16 * q + 11]), "=r"(r[16 * q + 12]), "=r"(r[16 * q + 13]), "=r"(r[16 * q + 14]),
          "=r"(r[16 * q + 15])
        : "r"((q < 2 ? ta : tb) + 16 * (q & 1)));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) { v[i] = __uint_as_float(r[i]); u[i] = __uint_as_float(r[32 + i]); }
}

// Activations of the gated epilogue through the hardware exponential and reciprocal (relative error ~1e-6, far below
// the bfloat16 rounding of the result).  The 32-bit path of the engine uses tanhf/expf in its own kernel.
__device__ __forceinline__ float act_fast(float x, int act) {
  if (act == KF_ACT_GELU_TANH) {
    const float y = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(y * 2.885390081777927f));      // exp(2y)
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.f));
    return 0.5f * x * (2.f - 2.f * r);                                               // 0.5 x (1 + tanh y)
  }
  if (act == KF_ACT_SILU) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-x * 1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.f));
    return x * r;
  }
  return kf_act(x, act);
}

constexpr int SMEM_LIMIT = 220 * 1024;

// A 2-D map over a row-major [rows, cols] bfloat16 matrix with boxes of [box_rows, 64] and the 128-byte swizzle
// (cached per base address and shape).  False if the driver entry point is missing or refuses the shape.
bool tensor_map(const void* base, long rows, long cols, int box_rows, CUtensorMap* out);
bool tensor_maps_available();

}  // namespace kf_tc
