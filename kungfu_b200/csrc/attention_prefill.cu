// Prompt-portion attention over paged bfloat16 keys and values on the tensor cores (mma.sync m16n8k16):
// causal, optional sliding window, optional softcap.
//
// A block is (tile of up to 64 consecutive rows of one request, query head); its 4 warps own 16 rows each.
// Keys are walked in tiles of BNK (64; 32 at head size 256) from the first key any row of the tile may see to
// the last row's position.  Key and value rows are gathered from the request's pages by 16-byte cp.async copies
// (a row that lies on a page the request no longer holds, or past the tile's last position, is zero-filled),
// double-buffered in shared memory with an XOR swizzle, and read back with ldmatrix.  S = Q K^T and O += P V run
// on m16n8k16 bfloat16 MMAs with 32-bit accumulators; scale, softcap, mask, the online softmax (base-2
// exponentials) and the running sums are 32-bit.  P is rounded to bfloat16 for the second product.
// Head sizes 16, 32, 64, 128, 256; others use the generic kernel.
// Reference counterpart: crates/kf-backend-cuda/src/kernels/flash.cu:14-26,52-248 (64 rows x 1 head per block,
// the same MMA shape on f16).  A tcgen05/TMEM version of this kernel is the next step for this engine.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

using namespace kf_mma;

constexpr int BM = 64;                 // query rows per tile
constexpr int PF_WARPS = 4;

template <int D, int BNK>
__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pages,
                    const int* __restrict__ tile_row0, const int* __restrict__ tile_nrows,
                    const int* __restrict__ positions, const int* __restrict__ row_req,
                    const int* __restrict__ table, int table_stride, int page_size, int nh, int nkv,
                    float scale, float softcap, int window, __nv_bfloat16* __restrict__ out) {
  kf_pdl_trigger();
  kf_pdl_wait();
  constexpr int CH = D / 8;                       // 16-byte chunks per row
  constexpr int NT_S = BNK / 8;                   // n-tiles of S per warp
  constexpr int NT_O = D / 8;                     // n-tiles of O per warp
  constexpr int KS_QK = D / 16;                   // k-steps of Q K^T
  constexpr int KS_PV = BNK / 16;                 // k-steps of P V
  extern __shared__ __align__(128) uint8_t pf_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(pf_smem);
  __nv_bfloat16* sK = sQ + BM * D;                // [2][BNK][D]
  __nv_bfloat16* sV = sK + 2 * BNK * D;           // [2][BNK][D]

  const int tile = blockIdx.x, h = blockIdx.y;
  const int row0 = tile_row0[tile], nrows = tile_nrows[tile];
  const int req = row_req[row0];
  if (req < 0 || nrows <= 0) return;                          // padding, or a tile without rows
  const int kvh = h / (nh / nkv);
  const int pos0 = positions[row0];                               // rows of a request are consecutive positions
  const int pos_last = pos0 + nrows - 1;
  const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int kt_begin = (lo / BNK) * BNK;
  const int n_ktiles = (pos_last - kt_begin) / BNK + 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int* tab = table + (size_t)req * table_stride;
  const size_t head_stride = (size_t)page_size * D;
  const size_t v_off = (size_t)nkv * head_stride;

  // ---- Q tile -> shared (rows past the tile are zero) -------------------------------------------------------
  for (int idx = tid; idx < BM * CH; idx += PF_WARPS * 32) {
    const int r = idx / CH, c = idx - r * CH;
    const bool ok = r < nrows;
    const __nv_bfloat16* src = q + ((size_t)(row0 + (ok ? r : 0)) * nh + h) * D + c * 8;
    cp_async16(tile_ptr<D>(sQ, r, c), src, ok);
  }
  auto load_kv = [&](int kt, int stage) {
    __nv_bfloat16* dk = sK + (size_t)stage * BNK * D;
    __nv_bfloat16* dv = sV + (size_t)stage * BNK * D;
    for (int idx = tid; idx < BNK * CH; idx += PF_WARPS * 32) {
      const int r = idx / CH, c = idx - r * CH;
      const int j = kt + r;
      bool ok = j <= pos_last;
      int page = 0;
      if (ok) { page = tab[j / page_size]; ok = page >= 0; }
      const __nv_bfloat16* src = pages + ((size_t)(ok ? page : 0) * 2 * nkv + kvh) * head_stride +
                                 (size_t)(ok ? j % page_size : 0) * D + c * 8;
      cp_async16(tile_ptr<D>(dk, r, c), src, ok);
      cp_async16(tile_ptr<D>(dv, r, c), src + v_off, ok);
    }
  };
  load_kv(kt_begin, 0);
  cp_async_commit();

  float o_acc[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n) { o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int prow[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};   // positions of this thread's two rows
  const float cap2 = softcap > 0.f ? 2.f * LOG2E / softcap : 0.f;

  for (int it = 0; it < n_ktiles; ++it) {
    const int stage = it & 1;
    const int kt = kt_begin + it * BNK;
    if (it + 1 < n_ktiles) load_kv(kt + BNK, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* k_s = sK + (size_t)stage * BNK * D;
    const __nv_bfloat16* v_s = sV + (size_t)stage * BNK * D;

    // ---- S = Q K^T for this warp's 16 rows -----------------------------------------------------------------
    float s_acc[NT_S][4];
#pragma unroll
    for (int n = 0; n < NT_S; ++n) { s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS_QK; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, tile_ptr<D>(sQ, warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np) {                     // two n-tiles (16 keys) per ldmatrix
        uint32_t b[4];
        ldmatrix_x4(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(k_s), np * 16 + (lane & 7) + ((lane >> 4) << 3),
                                   ks * 2 + ((lane >> 3) & 1)));
        mma_bf16(s_acc[2 * np], a, b[0], b[1]);
        mma_bf16(s_acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    // ---- scale, cap, mask; online softmax (base 2) -----------------------------------------------------------
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;                                      // 0: row g, 1: row g + 8
        const int j = kt + n * 8 + tq * 2 + (e & 1);
        float s = s_acc[n][e] * scale;
        if (softcap > 0.f) {
          const float ex = exp2f(s * cap2);
          s = softcap * (1.f - __fdividef(2.f, ex + 1.f));
        }
        const bool seen = j <= prow[r] && (window <= 0 || prow[r] - j < window);
        s = seen ? s * LOG2E : -INFINITY;
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
    for (int n = 0; n < NT_S; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = (m_new[r] == -INFINITY) ? 0.f : exp2f(s_acc[n][e] - m_new[r]);
        s_acc[n][e] = p;
        l_add[r] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + l_add[r];     // quad partial sums; merged at the end
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      o_acc[n][0] *= corr[0]; o_acc[n][1] *= corr[0];
      o_acc[n][2] *= corr[1]; o_acc[n][3] *= corr[1];
    }
    // ---- O += P V -----------------------------------------------------------------------------------------------
#pragma unroll
    for (int ks = 0; ks < KS_PV; ++ks) {
      uint32_t a[4];
      a[0] = pack_bf16(s_acc[2 * ks][0], s_acc[2 * ks][1]);
      a[1] = pack_bf16(s_acc[2 * ks][2], s_acc[2 * ks][3]);
      a[2] = pack_bf16(s_acc[2 * ks + 1][0], s_acc[2 * ks + 1][1]);
      a[3] = pack_bf16(s_acc[2 * ks + 1][2], s_acc[2 * ks + 1][3]);
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {                      // two n-tiles (16 value columns) per ldmatrix
        uint32_t b[4];
        ldmatrix_x4_trans(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(v_s), ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3),
                                         np * 2 + (lane >> 4)));
        mma_bf16(o_acc[2 * np], a, b[0], b[1]);
        mma_bf16(o_acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();                                               // the other stage may be overwritten next turn
  }
  cp_async_wait<0>();
  // ---- finish: row sums across the quad, normalise, store -------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int lr = warp * 16 + g + r * 8;
    if (lr >= nrows) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* orow = out + ((size_t)(row0 + lr) * nh + h) * D;
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
      const uint32_t v = pack_bf16(o_acc[n][2 * r] * inv, o_acc[n][2 * r + 1] * inv);
      *reinterpret_cast<uint32_t*>(orow + n * 8 + tq * 2) = v;
    }
  }
}

template <int D, int BNK>
int launch_prefill(const void* q, void* out, const void* pages, const int* tile_row0, const int* tile_nrows, int n_tiles,
                   const int* positions, const int* row_req, const int* table, int table_stride, int page_size,
                   int nh, int nkv, float scale, float softcap, int window, cudaStream_t stream) {
  const size_t smem = (size_t)(BM * D + 4 * BNK * D) * 2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<D, BNK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      kf_record_cuda_error(cudaGetLastError());
      return KF_ERR_SETUP;
    }
    configured = true;
  }
  kf_launch(attn_prefill_kernel<D, BNK>, dim3(n_tiles, nh), dim3(PF_WARPS * 32), smem, stream, 
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, tile_row0, tile_nrows, positions, row_req, table, table_stride,
      page_size, nh, nkv, scale, softcap, window, (__nv_bfloat16*)out);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

}  // namespace

KF_API int kf_attention_prefill_supported(int d) { return d == 16 || d == 32 || d == 64 || d == 128 || d == 256; }
KF_API int kf_attention_prefill_tile_rows() { return BM; }

// tile_row0[i], tile_nrows[i]: first row (index into the step's rows) and number of rows (1..64) of tile i; the rows of
// a tile belong to one request and hold consecutive positions.
KF_API int kf_attention_prefill(const void* q, void* out, const void* pages, const int* tile_row0, const int* tile_nrows,
                                int n_tiles, const int* positions, const int* row_req, const int* table, int table_stride,
                                int page_size, int nh, int nkv, int d, float scale, float softcap, int window,
                                cudaStream_t stream) {
  if (n_tiles <= 0) return KF_OK;
  if (nkv < 1 || nh % nkv != 0 || page_size < 1) return KF_ERR_SIZE;
#define KF_ARGS q, out, pages, tile_row0, tile_nrows, n_tiles, positions, row_req, table, table_stride, page_size, nh, nkv, scale, softcap, window, stream
  switch (d) {
    case 16: return launch_prefill<16, 64>(KF_ARGS);
    case 32: return launch_prefill<32, 64>(KF_ARGS);
    case 64: return launch_prefill<64, 64>(KF_ARGS);
    case 128: return launch_prefill<128, 64>(KF_ARGS);
    case 256: return launch_prefill<256, 32>(KF_ARGS);
  }
#undef KF_ARGS
  return KF_ERR_SIZE;
}
