// Fused scaled-dot-product attention forward (softmax(scale * Q K^T + mask) V) on tcgen05 tensor cores.
//
// The planner recognises the StableHLO chain dot_general -> multiply by a splat scale -> [iota / compare GE / select
// with -inf causal mask] -> reduce max -> subtract -> exponential -> reduce add -> divide -> convert -> dot_general
// (builders: crates/ryft-mlir/src/dialects/stable_hlo/operations/linear_algebra.rs:756-797, functional.rs:188-219,
// comparison.rs:136-164, control_flow.rs:263) and replaces it with this kernel; no score tensor touches HBM.
//
// One CTA per (batch*head, 128-row query tile); the tiles of one head are adjacent in the grid (K/V reuse in L2),
// longest causal prefix first.  192 threads:
//   warp 0      TMA producer: Q once, then K and V blocks of 128 keys into a 2-deep ring (per-CTA loads, no multicast)
//   warp 1      MMA issuer: S_j = Q K_j^T into one of two TMEM score buffers, O += P_j V_j into a TMEM accumulator;
//               S_{j+1} is issued before P_j is consumed so the tensor pipe works while the softmax warps run
//   warps 2-5   online softmax, one query row per thread: row max and exp2 from TMEM (two passes over 32-column
//               chunks), P_j written as bf16 into 128-byte-swizzled shared memory for the second MMA; the output
//               accumulator is rescaled only when the running max grew by more than 2^8 (exact: the same stale max is
//               used for the row sum), and is normalised by the row sum at the end
// Causal tiles above the diagonal are skipped; the diagonal block and ragged key tails are masked in registers.
// Bound: tensor pipe / MUFU (exp2); algorithmic FLOPs = 4 * BH * D * (number of unmasked score elements).
// Every mbarrier wait is bounded; on expiry the CTA unwinds, frees TMEM and reports through `status`.
#include "../../../include/b2x_kernels.h"
#include "common.cuh"
#include "sm100.cuh"

#include <cuda_bf16.h>

namespace b2x {

struct AttnParams {
  int64_t BH, Sq, Sk;
  int32_t n_q_tiles;
  int32_t causal;
  float scale_log2;   // scale * log2(e)
  __nv_bfloat16* out;
  uint32_t idesc_qk, idesc_pv;
};

constexpr int AT_M = 128;   // query rows per CTA
constexpr int AT_N = 128;   // keys per block

template <int D>
struct AttnSmem {
  static constexpr int Q_BYTES = AT_M * D * 2;
  static constexpr int KV_BYTES = AT_N * D * 2;
  static constexpr int P_BYTES = AT_M * AT_N * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;            // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;       // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(192, 1)
k_attention(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const __grid_constant__ AttnParams p, int32_t* status) {
  using namespace sm100;
  using SM = AttnSmem<D>;
  constexpr int DC = D / 64;                 // 64-wide (128-byte) chunks of the head dimension
  constexpr uint32_t TMEM_COLS = 512;        // S0 [0,128), S1 [128,256), O [256, 256 + D)
  constexpr uint32_t CHUNK_BYTES = 128 * 128;  // one [128 rows x 128 bytes] swizzled sub-tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + SM::BAR_OFF);
  // barriers: q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, pv_done, drain
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_q = b0, bar_kf = b0 + 8, bar_vf = b0 + 24, bar_kve = b0 + 40, bar_sf = b0 + 56, bar_se = b0 + 72, bar_pf = b0 + 88,
                 bar_pv = b0 + 96, bar_drain = b0 + 104;
  uint32_t* tmem_slot = (uint32_t*)(bars + 14);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // consecutive CTAs are the query tiles of one (batch, head), longest causal prefix first: they run together and find
  // that head's K and V in L2
  const int bh = (int)(blockIdx.x / p.n_q_tiles);
  const int qt = p.n_q_tiles - 1 - (int)(blockIdx.x % p.n_q_tiles);
  const int q0 = qt * AT_M;
  int64_t k_end = p.Sk;
  if (p.causal && (int64_t)q0 + AT_M < k_end) k_end = (int64_t)q0 + AT_M;
  const int nblk = (int)((k_end + AT_N - 1) / AT_N);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_kf + 8 * s, 1); mbar_init(bar_vf + 8 * s, 1); mbar_init(bar_kve + 8 * s, 1);
      mbar_init(bar_sf + 8 * s, 1); mbar_init(bar_se + 8 * s, 4);
    }
    mbar_init(bar_pf, 4); mbar_init(bar_pv, 1); mbar_init(bar_drain, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ---------------------------------------------- TMA producer --------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar_q, SM::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DC; c++) tma_load_3d(sbase + SM::Q_OFF + c * CHUNK_BYTES, &tmQ, bar_q, c * 64, q0, bh);
      bool ok = true;
      for (int j = 0; j < nblk && ok; j++) {
        const int st = j & 1;
        if (!mbar_wait(bar_kve + 8 * st, (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag, status, 11)) { ok = false; break; }
        mbar_expect_tx(bar_kf + 8 * st, SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; c++) tma_load_3d(sbase + SM::K_OFF + st * SM::KV_BYTES + c * CHUNK_BYTES, &tmK, bar_kf + 8 * st, c * 64, j * AT_N, bh);
        mbar_expect_tx(bar_vf + 8 * st, SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; c++) tma_load_3d(sbase + SM::V_OFF + st * SM::KV_BYTES + c * CHUNK_BYTES, &tmV, bar_vf + 8 * st, c * 64, j * AT_N, bh);
      }
      if (!ok) {
        for (int s = 0; s < 2; s++)
          for (uint32_t i = 0; i < (1u << 16); i++) {
            if ((mbar_try_wait(bar_kf + 8 * s, 0) || mbar_try_wait(bar_kf + 8 * s, 1)) && (mbar_try_wait(bar_vf + 8 * s, 0) || mbar_try_wait(bar_vf + 8 * s, 1))) break;
            __nanosleep(64);
          }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------- MMA issuer ------------------------------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 12);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1, sb = j & 1;
        if (!mbar_wait(bar_kf + 8 * st, (uint32_t)((j >> 1) & 1), abort_flag, status, 13)) return false;
        if (!mbar_wait(bar_se + 8 * sb, (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag, status, 14)) return false;
        tc_fence_after();
        const uint32_t qa = sbase + SM::Q_OFF, ka = sbase + SM::K_OFF + st * SM::KV_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; k++) {
          const uint32_t off = (uint32_t)(k >> 2) * CHUNK_BYTES + (uint32_t)(k & 3) * 32;
          umma_ss<false>(tmem_base + (uint32_t)(sb * 128), make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), p.idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(bar_sf + 8 * sb);
        return true;
      };
      if (ok && nblk > 0) ok = issue_qk(0);
      for (int j = 0; j < nblk && ok; j++) {
        if (j + 1 < nblk) { if (!issue_qk(j + 1)) { ok = false; break; } }
        const int st = j & 1;
        if (!mbar_wait(bar_vf + 8 * st, (uint32_t)((j >> 1) & 1), abort_flag, status, 15)) { ok = false; break; }
        if (!mbar_wait(bar_pf, (uint32_t)(j & 1), abort_flag, status, 16)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pa = sbase + SM::P_OFF, va = sbase + SM::V_OFF + st * SM::KV_BYTES;
#pragma unroll
        for (int k = 0; k < AT_N / 16; k++) {
          // A = P (K-major: keys contiguous); B = V (MN-major: head-dim chunks of 64 are CHUNK_BYTES apart, 8 key rows per 1 KiB)
          const uint32_t aoff = (uint32_t)(k >> 2) * CHUNK_BYTES + (uint32_t)(k & 3) * 32;
          umma_ss<false>(tmem_o, make_smem_desc(pa + aoff, 16, 1024), make_smem_desc(va + (uint32_t)k * 2048, CHUNK_BYTES, 1024), p.idesc_pv,
                         (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar_kve + 8 * st);
        tc_commit(bar_pv);
      }
      tc_commit(bar_drain);
      mbar_wait(bar_drain, 0, abort_flag, nullptr, 0);
    }
  } else {
    // ---------------------------------------------- softmax ---------------------------------------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;             // row of the tile == TMEM lane
    const int64_t qrow = (int64_t)q0 + row;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    uint8_t* prow = smem + SM::P_OFF + row * 128;
    for (int j = 0; j < nblk && ok; j++) {
      const int sb = j & 1;
      if (!mbar_wait(bar_sf + 8 * sb, (uint32_t)((j >> 1) & 1), abort_flag, status, 17)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)(sb * 128);
      // columns of this block that this row may attend to: [0, limit]
      int64_t lim = p.Sk - 1 - (int64_t)j * AT_N;
      if (p.causal) { const int64_t c = qrow - (int64_t)j * AT_N; lim = c < lim ? c : lim; }
      const bool need_mask = __any_sync(0xffffffffu, lim < AT_N - 1);
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < AT_N / 32; c++) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + (uint32_t)(c * 32), r);
        tc_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i++) { float v = __uint_as_float(r[i]); mx = (c * 32 + i <= lim) ? fmaxf(mx, v) : mx; }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) m_used = mx;
      else if ((mx - m_used) * p.scale_log2 > 8.0f) { alpha = fast_exp2((m_used - mx) * p.scale_log2); l *= alpha; m_used = mx; rescale = true; }
      // the previous P V product must have retired before O is touched or P is overwritten
      if (j > 0) {
        if (!mbar_wait(bar_pv, (uint32_t)((j - 1) & 1), abort_flag, status, 18)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; c++) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_o + lane_addr + (uint32_t)(c * 32), r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            // 32 columns back in two 16-column stores
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; i++) { lo[i] = r[i]; hi[i] = r[16 + i]; }
            tmem_st_32x16(tmem_o + lane_addr + (uint32_t)(c * 32), lo);
            tmem_st_32x16(tmem_o + lane_addr + (uint32_t)(c * 32 + 16), hi);
          }
          tc_wait_st();
        }
      }
      // pass 2: p = exp2(s * scale_log2 - m * scale_log2), row sum, bf16 P into swizzled shared memory
      const float mneg = -m_used * p.scale_log2;
      float psum = 0.f;
#pragma unroll 1
      for (int c = 0; c < AT_N / 32; c++) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + (uint32_t)(c * 32), r);
        tc_wait_ld();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; i++) {
          float e = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, mneg));
          if (need_mask) e = (c * 32 + i <= lim) ? e : 0.f;
          pv[i] = e;
          psum += e;
        }
        // 32 keys = 64 bytes = four 16-byte pieces of this row; piece index within the 128-byte line is XOR-swizzled
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; h++) {
            __nv_bfloat162 t = __floats2bfloat162_rn(pv[q * 8 + 2 * h], pv[q * 8 + 2 * h + 1]);
            w[h] = *reinterpret_cast<uint32_t*>(&t);
          }
          const int piece = c * 4 + q;                 // 0..15 over the 128 keys
          const int sub = piece >> 3, in = piece & 7;
          *reinterpret_cast<uint4*>(prow + sub * CHUNK_BYTES + ((in ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l += psum;
      // S buffer free for the block after next; P visible to the tensor-core (async) proxy
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_se + 8 * sb); mbar_arrive(bar_pf); }
    }
    // ---- epilogue: O / l -> bf16 -> global ----
    if (ok && nblk > 0) ok = mbar_wait(bar_pv, (uint32_t)((nblk - 1) & 1), abort_flag, status, 19);
    if (ok) {
      tc_fence_after();
      const float inv = (nblk > 0 && l > 0.f) ? __fdividef(1.0f, l) : 0.f;
      __nv_bfloat16* orow = p.out + ((int64_t)bh * p.Sq + qrow) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; c++) {
        uint32_t r[32];
        if (nblk > 0) { tmem_ld_32x32(tmem_o + lane_addr + (uint32_t)(c * 32), r); tc_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; i++) r[i] = 0;
        }
        if (qrow < p.Sq) {
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 4; h++) {
              __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + 2 * h]) * inv, __uint_as_float(r[q * 8 + 2 * h + 1]) * inv);
              w[h] = *reinterpret_cast<uint32_t*>(&t);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

template <int D>
static int launch_attention(const B2xAttentionArgs* a, int32_t* status, cudaStream_t stream) {
  using SM = AttnSmem<D>;
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!encode_3d(&tmQ, dt, 2, a->q, D, (uint64_t)a->Sq, (uint64_t)a->BH, D, (uint64_t)a->Sq * D, 64, AT_M)) return (int)cudaErrorInvalidValue;
  if (!encode_3d(&tmK, dt, 2, a->k, D, (uint64_t)a->Sk, (uint64_t)a->BH, D, (uint64_t)a->Sk * D, 64, AT_N)) return (int)cudaErrorInvalidValue;
  if (!encode_3d(&tmV, dt, 2, a->v, D, (uint64_t)a->Sk, (uint64_t)a->BH, D, (uint64_t)a->Sk * D, 64, AT_N)) return (int)cudaErrorInvalidValue;
  AttnParams p{};
  p.BH = a->BH; p.Sq = a->Sq; p.Sk = a->Sk;
  p.n_q_tiles = (int)((a->Sq + AT_M - 1) / AT_M);
  p.causal = a->causal;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)a->o;
  p.idesc_qk = sm100::make_idesc(1u, false, false, AT_M, AT_N);
  p.idesc_pv = sm100::make_idesc(1u, false, true, AT_M, D);
  auto kern = k_attention<D>;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    static bool configured[64] = {};
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  const int64_t grid = (int64_t)p.n_q_tiles * a->BH;
  if (grid <= 0) return 0;
  if (grid > 0x7fffffff) return (int)cudaErrorInvalidValue;
  kern<<<(unsigned)grid, 192, SM::TOTAL, stream>>>(tmQ, tmK, tmV, p, status);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace b2x

extern "C" int b2x_launch_attention(const B2xAttentionArgs* a, int32_t* status, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->BH <= 0 || a->Sq <= 0 || a->Sk <= 0) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)a->q & 15) || ((uintptr_t)a->k & 15) || ((uintptr_t)a->v & 15) || ((uintptr_t)a->o & 15)) return (int)cudaErrorInvalidValue;
  if (a->D == 128) return launch_attention<128>(a, status, stream);
  if (a->D == 64) return launch_attention<64>(a, status, stream);
  return (int)cudaErrorInvalidValue;
}
