// Device helpers shared by the tcgen05 products: mbarriers with bounded waits, TMA tile loads, shared-memory and
// instruction descriptors, the MMA and tensor-memory instructions, the fast activations, and the rows-from-a-pending-norm
// prologue.  Everything is inline; the one host function (the cached tensor maps) lives in gemm_tc.cu.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace kf_tc {

constexpr int BM = 128;            // output features per tile (tensor-memory lanes)
constexpr int BK = 64;             // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int WAIT_LIMIT = 40 * 1000 * 1000;

enum { EPI_F32 = 0, EPI_BF16 = 1, EPI_GATED = 2 };
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
      else if (now - t0 > WAIT_LIMIT_NS) return false;
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

// The activation operand can come from a norm that is still pending: the previous product left its 32-bit output
// `branch`, and the rows this product reads are  n = rmsnorm(y; w_next)  with  y = res_in + rmsnorm(branch; w_post).
// Then every CTA computes the rows itself (the sums need whole rows, a few KB each) and writes its K range of n
// straight into shared memory in the layout the tensor core reads; the CTAs of feature tile 0 also store their K range
// of y to `res_out` (a buffer other than res_in: other CTAs still read res_in).  This saves the norm's own kernel.
struct NormIn {
  const float* branch;
  const float* res_in;
  float* res_out;
  const __nv_bfloat16* w_post;
  const __nv_bfloat16* w_next;
  float eps_post, eps_next;
  int plus_post, plus_next;
};

__device__ __forceinline__ void unpack_bf16x8(const uint4& r, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(p[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// Called by the 128 epilogue threads (w4 = 0..3 is the warp among them, tid = w4 * 32 + lane); red: 2 * 4 * BN floats
// of shared memory.  xs: [nkb][BN rows][128 bytes], 128-byte swizzle.  Work is split by columns, every thread walks
// all rows of its columns with the rows' loads independent of one another, so the latency of L2 is paid once per
// pass and not once per row: pass 1 sums branch^2, pass 2 sums y^2, pass 3 writes this CTA's K range.
// RB: rows held in registers (T <= RB <= BN); rows RB..BN-1 of the tile are zero-filled.
template <int BN, int RB = BN>
__device__ __forceinline__ void normed_rows_to_smem(const NormIn& ni, int T, int K, int kb_begin, int nkb, uint8_t* xs,
                                                    bool write_residual, int w4, int lane, float* red) {
  const int tid = w4 * 32 + lane;
  const int n4 = K >> 2;                                          // groups of 4 columns
  const float gp = ni.plus_post ? 1.f : 0.f, gn = ni.plus_next ? 1.f : 0.f;
  const float inv_k = 1.f / (float)K;
  float acc[RB];
  auto block_sums = [&](float* slot) {                            // acc[r] summed over the 128 threads -> acc[r]
#pragma unroll
    for (int r = 0; r < RB; ++r) acc[r] = kf_warp_sum(acc[r]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RB; ++r) slot[w4 * RB + r] = acc[r];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
    for (int r = 0; r < RB; ++r) acc[r] = slot[r] + slot[RB + r] + slot[2 * RB + r] + slot[3 * RB + r];
  };
  // ---- pass 1: sum of squares of the branch rows ---------------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < RB; ++r) acc[r] = 0.f;
  for (int c = tid; c < n4; c += 128) {
    float4 v[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r)
      v[r] = r < T ? *reinterpret_cast<const float4*>(ni.branch + (size_t)r * K + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < RB; ++r) acc[r] += v[r].x * v[r].x + v[r].y * v[r].y + v[r].z * v[r].z + v[r].w * v[r].w;
  }
  block_sums(red);
  float inv1[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) inv1[r] = 1.f / sqrtf(acc[r] * inv_k + ni.eps_post);
  // ---- pass 2: sum of squares of y = residual + branch * inv1 * g ------------------------------------------------------
#pragma unroll
  for (int r = 0; r < RB; ++r) acc[r] = 0.f;
  for (int c = tid; c < n4; c += 128) {
    const uint2 gw = *reinterpret_cast<const uint2*>(ni.w_post + c * 4);
    const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw.x));
    const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw.y));
    float4 va[RB], vx[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      va[r] = r < T ? *reinterpret_cast<const float4*>(ni.branch + (size_t)r * K + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      vx[r] = r < T ? *reinterpret_cast<const float4*>(ni.res_in + (size_t)r * K + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const float y0 = vx[r].x + va[r].x * inv1[r] * (g01.x + gp), y1 = vx[r].y + va[r].y * inv1[r] * (g01.y + gp);
      const float y2 = vx[r].z + va[r].z * inv1[r] * (g23.x + gp), y3 = vx[r].w + va[r].w * inv1[r] * (g23.y + gp);
      acc[r] += y0 * y0 + y1 * y1 + y2 * y2 + y3 * y3;
    }
  }
  block_sums(red + 4 * RB);
  float inv2[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) inv2[r] = 1.f / sqrtf(acc[r] * inv_k + ni.eps_next);
  // ---- pass 3: this CTA's K range, 8 columns (16 bytes of bfloat16) at a time ----------------------------------------
  for (int cc = tid; cc < nkb * 8; cc += 128) {
    const int c8 = kb_begin * 8 + cc;
    const bool in_k = c8 * 8 < K;
    float g1[8], g2[8];
    if (in_k) {
      unpack_bf16x8(*reinterpret_cast<const uint4*>(ni.w_post + c8 * 8), g1);
      unpack_bf16x8(*reinterpret_cast<const uint4*>(ni.w_next + c8 * 8), g2);
    }
    uint8_t* tile = xs + (size_t)(cc >> 3) * (BN * 128);
#pragma unroll
    for (int r0 = 0; r0 < RB; r0 += 4) {                           // four rows' loads in flight
      float4 a0[4], a1[4], x0[4], x1[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int r = r0 + q;
        if (in_k && r < T) {
          const float* a = ni.branch + (size_t)r * K + c8 * 8;
          const float* x = ni.res_in + (size_t)r * K + c8 * 8;
          a0[q] = *reinterpret_cast<const float4*>(a); a1[q] = *reinterpret_cast<const float4*>(a + 4);
          x0[q] = *reinterpret_cast<const float4*>(x); x1[q] = *reinterpret_cast<const float4*>(x + 4);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int r = r0 + q;
        uint4 packed = make_uint4(0, 0, 0, 0);
        if (in_k && r < T) {
          const float av[8] = {a0[q].x, a0[q].y, a0[q].z, a0[q].w, a1[q].x, a1[q].y, a1[q].z, a1[q].w};
          const float xv[8] = {x0[q].x, x0[q].y, x0[q].z, x0[q].w, x1[q].x, x1[q].y, x1[q].z, x1[q].w};
          float y[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = xv[i] + av[i] * inv1[r] * (g1[i] + gp);
          if (write_residual) {
            float* o = ni.res_out + (size_t)r * K + c8 * 8;
            *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(y[4], y[5], y[6], y[7]);
          }
          __nv_bfloat162 h[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            h[i] = __floats2bfloat162_rn(y[2 * i] * inv2[r] * (g2[2 * i] + gn), y[2 * i + 1] * inv2[r] * (g2[2 * i + 1] + gn));
          packed = make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                              *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
        }
        *reinterpret_cast<uint4*>(tile + (size_t)(r >> 3) * 1024 + (size_t)(r & 7) * 128 + (((cc & 7) ^ (r & 7)) << 4)) = packed;
      }
    }
#pragma unroll
    for (int r = RB; r < BN; ++r)
      *reinterpret_cast<uint4*>(tile + (size_t)(r >> 3) * 1024 + (size_t)(r & 7) * 128 + (((cc & 7) ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
  }
}

// Plain bfloat16 rows x[T, K] into the same layout (this CTA's K range; rows >= T and columns >= K are zeros).
template <int BN>
__device__ __forceinline__ void copy_rows_to_smem(const __nv_bfloat16* __restrict__ x, int T, int K, int kb_begin, int nkb,
                                                  uint8_t* xs, int tid) {
  for (int cc = tid; cc < nkb * 8; cc += 128) {
    const int c8 = kb_begin * 8 + cc;
    const bool in_k = c8 * 8 < K;
    uint4 v[BN];
#pragma unroll
    for (int r = 0; r < BN; ++r)
      v[r] = (in_k && r < T) ? *reinterpret_cast<const uint4*>(x + (size_t)r * K + c8 * 8) : make_uint4(0, 0, 0, 0);
    uint8_t* tile = xs + (size_t)(cc >> 3) * (BN * 128);
#pragma unroll
    for (int r = 0; r < BN; ++r)
      *reinterpret_cast<uint4*>(tile + (size_t)(r >> 3) * 1024 + (size_t)(r & 7) * 128 + (((cc & 7) ^ (r & 7)) << 4)) = v[r];
  }
}

// ---- mbarriers of other CTAs of the cluster ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrive `count` times on a barrier in the shared memory of CTA `rank`; writes of this thread before it (and what a CTA
// barrier ordered before them) are visible to whoever waits with acquire at cluster scope.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank, uint32_t count) {
  const uint32_t remote = map_to_cta(smem_u32(bar), rank);
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(remote), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  unsigned long long t0 = 0;
  for (int i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 255) == 255) {
      const unsigned long long now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) return false;
    }
  }
  return false;
}




constexpr int SMEM_LIMIT = 220 * 1024;

// A 2-D map over a row-major [rows, cols] bfloat16 matrix with boxes of [box_rows, 64] and the 128-byte swizzle
// (cached per base address and shape).  False if the driver entry point is missing or refuses the shape.
bool tensor_map(const void* base, long rows, long cols, int box_rows, CUtensorMap* out);
bool tensor_maps_available();

}  // namespace kf_tc
