// Fused scaled-dot-product attention forward (softmax(scale * Q K^T + mask) V) on tcgen05 tensor cores.
//
// The planner recognises the StableHLO chain dot_general -> multiply by a splat scale -> [iota / compare GE / select
// with -inf causal mask] -> reduce max -> subtract -> exponential -> reduce add -> divide -> convert -> dot_general
// (builders: crates/ryft-mlir/src/dialects/stable_hlo/operations/linear_algebra.rs:756-797, functional.rs:188-219,
// comparison.rs:136-164, control_flow.rs:263) and replaces it with this kernel; no score tensor touches HBM.
//
// Two kernels live here.  k_attention_pw (further down; the default) is persistent: one CTA per SM, two workers per CTA,
// each walking whole query tiles.  k_attention, described next, is the earlier one-tile-per-CTA form, kept as the
// fallback and for comparison (B2X_ATTENTION_KERNEL=tile).
//
// k_attention: one CTA per (batch*head, 128-row query tile); the tiles of one head are adjacent in the grid (K/V reuse in L2),
// longest causal prefix first.  The key blocks of a tile (128 keys each) are dealt alternately to two independent
// softmax streams: stream s owns blocks j = s, s + 2, ..., its own score buffer, probability buffer, K/V stage and
// output accumulator, and keeps its own running (max, sum).  While one stream exponentiates, the tensor pipe works
// for the other; the two partial results are merged once, at the end.  96 + 256 * TPR threads:
//   warp 0      TMA producer: Q once, then K_j and V_j into stage j & 1 as soon as that stage's previous K (after its
//               Q K^T retired) or V (after its P V retired) is free; each CTA loads its own tiles
//   warps 1,2   MMA issuers, one per stream: S_s = Q K_j^T into TMEM score buffer s, O_s += P_s V_j into accumulator s
//   warps 3..   softmax, 4 * TPR warps per stream.  TPR = 1 (the default): one thread per query row.  TPR = 2: two threads
//               share a query row, each owns 64 of the block's 128 keys (four softmax warps per scheduler instead of
//               two; measured slower).  With TPR = 2 a thread reads all 128 scores of its row from TMEM for the row maximum (both threads of
//               a row thus hold the same maximum without talking to each other) and keeps its own 64 in registers:
//               exp2, partial row sum, P as bf16 into 128-byte-swizzled shared memory for the second MMA.  The
//               accumulator is rescaled only when the running max grew by more than 2^8 (exact: the same stale max is
//               used for the row sum); the partial sums of a row meet in the final merge.
// Causal tiles above the diagonal are skipped; the diagonal block and ragged key tails are masked in registers.
// Bound: tensor pipe / MUFU (exp2), about equal for D = 128; algorithmic FLOPs = 4 * BH * D * (unmasked scores).
// Every wait is bounded; on expiry the CTA unwinds, frees TMEM and reports through `status`.
#include <atomic>
#include <cstdlib>
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

// PT: the probabilities go to the second MMA through TMEM (as its A operand) instead of shared memory; the P buffers
// then shrink to the 2 KB per stream that the final merge needs.
template <int D, bool PT>
struct AttnSmem {
  static constexpr int Q_BYTES = AT_M * D * 2;
  static constexpr int KV_BYTES = AT_N * D * 2;
  static constexpr int P_BYTES = PT ? 2048 : AT_M * AT_N * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;            // 2 stages (one per stream)
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;       // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * KV_BYTES;       // 2 buffers
  static constexpr int BAR_OFF = P_OFF + 2 * P_BYTES;      // 20 barriers, TMEM slot, abort flag
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two f32 lanes per instruction (sm_100 packed single precision) and the three-input maximum: the softmax warps are
// bound by instruction issue, and these halve the count of everything except the exponentials themselves.
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t splat2(float v) { return pack2(__float_as_uint(v), __float_as_uint(v)); }
__device__ __forceinline__ void unpack2(uint64_t v, uint32_t& lo, uint32_t& hi) { asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// NaN-propagating, so that a NaN score poisons its row as it does in an unfused softmax
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
template <int D, int TPR, bool PT>
__global__ void __launch_bounds__(96 + 256 * TPR, 1)
k_attention(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const __grid_constant__ AttnParams p, int32_t* status) {
  using namespace sm100;
  using SM = AttnSmem<D, PT>;
  constexpr int DC = D / 64;                 // 64-wide (128-byte) chunks of the head dimension
  constexpr uint32_t TMEM_COLS = 512;        // S0 [0,128), S1 [128,256), O0 [256, 256 + D), O1 [256 + D, 256 + 2 D)
  constexpr uint32_t CHUNK_BYTES = 128 * 128;  // one [128 rows x 128 bytes] swizzled sub-tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + SM::BAR_OFF);
  // barriers (each [2] is indexed by stream): q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2],
  // s_empty[2], p_full[2], pv_done[2], merge, drain
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_q = b0, bar_kf = b0 + 8, bar_ke = b0 + 24, bar_vf = b0 + 40, bar_ve = b0 + 56, bar_sf = b0 + 72, bar_se = b0 + 88,
                 bar_pf = b0 + 104, bar_pv = b0 + 120, bar_merge = b0 + 136, bar_drain = b0 + 144;   // drain[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 20);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  // per stream, row half and row (max * scale_log2, partial sum) for the final merge; stream s keeps them at the start of
  // its own probability buffer, which is idle once its last P V product has retired
  auto merge_slot = [&](int s, int half, int row) -> float2* { return (float2*)(smem + SM::P_OFF + s * SM::P_BYTES) + half * AT_M + row; };

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
      mbar_init(bar_kf + 8 * s, 1); mbar_init(bar_ke + 8 * s, 1); mbar_init(bar_vf + 8 * s, 1); mbar_init(bar_ve + 8 * s, 1);
      mbar_init(bar_sf + 8 * s, 1); mbar_init(bar_se + 8 * s, 4 * TPR); mbar_init(bar_pf + 8 * s, 4 * TPR); mbar_init(bar_pv + 8 * s, 1);
    }
    mbar_init(bar_merge, 8 * TPR); mbar_init(bar_drain, 1); mbar_init(bar_drain + 8, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------- TMA producer --------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar_q, SM::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DC; c++) tma_load_3d(sbase + SM::Q_OFF + c * CHUNK_BYTES, &tmQ, bar_q, c * 64, q0, bh);
      // K_j and V_j go into stage j & 1; each is issued as soon as its stage is free, whichever comes first
      int jk = 0, jv = 0;
      uint32_t idle = 0;
      bool ok = true;
      while (jk < nblk || jv < nblk) {
        bool progress = false;
        if (jk < nblk) {
          const int s = jk & 1, it = jk >> 1;
          if (it == 0 || mbar_try_wait(bar_ke + 8 * s, (uint32_t)((it - 1) & 1))) {
            mbar_expect_tx(bar_kf + 8 * s, SM::KV_BYTES);
#pragma unroll
            for (int c = 0; c < DC; c++) tma_load_3d(sbase + SM::K_OFF + s * SM::KV_BYTES + c * CHUNK_BYTES, &tmK, bar_kf + 8 * s, c * 64, jk * AT_N, bh);
            jk++; progress = true;
          }
        }
        if (jv < nblk) {
          const int s = jv & 1, it = jv >> 1;
          if (it == 0 || mbar_try_wait(bar_ve + 8 * s, (uint32_t)((it - 1) & 1))) {
            mbar_expect_tx(bar_vf + 8 * s, SM::KV_BYTES);
#pragma unroll
            for (int c = 0; c < DC; c++) tma_load_3d(sbase + SM::V_OFF + s * SM::KV_BYTES + c * CHUNK_BYTES, &tmV, bar_vf + 8 * s, c * 64, jv * AT_N, bh);
            jv++; progress = true;
          }
        }
        if (progress) { idle = 0; continue; }
        if (++idle > (1u << 22)) { *abort_flag = 1; if (status) atomicCAS(status, 0, 11); ok = false; break; }
        if (idle > 16) { if (*abort_flag) { ok = false; break; } __nanosleep(idle > 4096 ? 256 : 32); }
      }
      if (!ok) {
        // let copies already in flight land before the CTA's shared memory goes away
        for (int s = 0; s < 2; s++)
          for (uint32_t i = 0; i < (1u << 16); i++) {
            if ((mbar_try_wait(bar_kf + 8 * s, 0) || mbar_try_wait(bar_kf + 8 * s, 1)) && (mbar_try_wait(bar_vf + 8 * s, 0) || mbar_try_wait(bar_vf + 8 * s, 1))) break;
            __nanosleep(64);
          }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------------------------------------- MMA issuers -----------------------------------------------------
    // One issuing thread per stream, so that a stream whose probabilities are late never holds up the other stream's
    // next score block.  The two threads touch disjoint TMEM columns and shared-memory buffers (Q is only read).
    if (lane == 0) {
      const int s = warp - 1;
      const int n_mine = nblk > s ? (nblk - s + 1) / 2 : 0;
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 12);
      auto issue_qk = [&](int it) -> bool {
        if (!mbar_wait(bar_kf + 8 * s, (uint32_t)(it & 1), abort_flag, status, 13)) return false;
        tc_fence_after();
        const uint32_t qa = sbase + SM::Q_OFF, ka = sbase + SM::K_OFF + s * SM::KV_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; k++) {
          const uint32_t off = (uint32_t)(k >> 2) * CHUNK_BYTES + (uint32_t)(k & 3) * 32;
          umma_ss<false>(tmem_base + (uint32_t)(s * 128), make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), p.idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(bar_sf + 8 * s);    // scores ready for the stream
        tc_commit(bar_ke + 8 * s);    // K stage free
        return true;
      };
      if (ok && n_mine > 0) ok = issue_qk(0);
      for (int it = 0; it < n_mine && ok; it++) {
        if constexpr (!PT) {
          // the stream has copied this block's scores into registers: its score buffer can take its next block
          if (it + 1 < n_mine) {
            if (!mbar_wait(bar_se + 8 * s, (uint32_t)(it & 1), abort_flag, status, 14)) { ok = false; break; }
            if (!issue_qk(it + 1)) { ok = false; break; }
          }
        }
        if (!mbar_wait(bar_vf + 8 * s, (uint32_t)(it & 1), abort_flag, status, 15)) { ok = false; break; }
        if (!mbar_wait(bar_pf + 8 * s, (uint32_t)(it & 1), abort_flag, status, 16)) { ok = false; break; }
        tc_fence_after();
        const uint32_t va = sbase + SM::V_OFF + s * SM::KV_BYTES;
        const uint32_t o_tmem = tmem_base + 256u + (uint32_t)(s * D);
        if constexpr (PT) {
          // A = P from TMEM: row = lane, 16 keys of a k-step = 8 columns (two bf16 per column) at the start of the stream's
          // score buffer; B = V (MN-major: head-dim chunks of 64 are CHUNK_BYTES apart, 8 key rows per 1 KiB)
          const uint32_t p_tmem = tmem_base + (uint32_t)(s * 128);
#pragma unroll
          for (int k = 0; k < AT_N / 16; k++)
            umma_ts_f16(o_tmem, p_tmem + (uint32_t)(k * 8), make_smem_desc(va + (uint32_t)k * 2048, CHUNK_BYTES, 1024), p.idesc_pv, (it > 0 || k > 0) ? 1u : 0u);
        } else {
          const uint32_t pa = sbase + SM::P_OFF + s * SM::P_BYTES;
#pragma unroll
          for (int k = 0; k < AT_N / 16; k++) {
            // A = P (K-major: keys contiguous); B = V (MN-major: head-dim chunks of 64 are CHUNK_BYTES apart, 8 key rows per 1 KiB)
            const uint32_t aoff = (uint32_t)(k >> 2) * CHUNK_BYTES + (uint32_t)(k & 3) * 32;
            umma_ss<false>(o_tmem, make_smem_desc(pa + aoff, 16, 1024), make_smem_desc(va + (uint32_t)k * 2048, CHUNK_BYTES, 1024), p.idesc_pv,
                           (it > 0 || k > 0) ? 1u : 0u);
          }
        }
        tc_commit(bar_ve + 8 * s);    // V stage free
        tc_commit(bar_pv + 8 * s);    // the stream's accumulator and probability buffer may be touched again
        if constexpr (PT) {
          // the probabilities sit in the score buffer: the next score block may overwrite it only after the product above
          // has read them, which the tensor pipe guarantees by executing this thread's MMAs in issue order
          if (it + 1 < n_mine && !issue_qk(it + 1)) { ok = false; break; }
        }
      }
      // everything this thread issued must retire before TMEM is released
      tc_commit(bar_drain + 8 * s);
      mbar_wait(bar_drain + 8 * s, 0, abort_flag, nullptr, 0);
    }
  } else {
    // ---------------------------------------------- softmax ---------------------------------------------------------
    constexpr int WPS = 4 * TPR;                  // softmax warps per stream
    constexpr int KW = AT_N / TPR;                // keys of a block that this thread exponentiates
    constexpr int KC = KW / 32;                   // ... in chunks of 32
    const int s = (warp - 3) / WPS;               // stream
    const int half = ((warp - 3) % WPS) >> 2;     // which part of the row's keys
    const int quad = warp & 3;                    // TMEM lanes [32 * quad, 32 * quad + 32): fixed by the warp's number
    const int row = quad * 32 + lane;             // row of the tile == TMEM lane
    const int64_t qrow = (int64_t)q0 + row;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)(s * 128);
    const uint32_t o_addr = tmem_base + lane_addr + 256u + (uint32_t)(s * D);
    float m_used = -INFINITY, l = 0.f;
    bool ok = true, poisoned = false;
    const uint32_t prow_s = sbase + (uint32_t)(SM::P_OFF + s * SM::P_BYTES + row * 128);
    const int n_mine = nblk > s ? (nblk - s + 1) / 2 : 0;    // blocks s, s + 2, ...
    for (int it = 0; it < n_mine && ok; it++) {
      const int j = 2 * it + s;
      if (!mbar_wait(bar_sf + 8 * s, (uint32_t)(it & 1), abort_flag, status, 17)) { ok = false; break; }
      tc_fence_after();
      // columns of this block that this row may attend to: [0, lim]
      int64_t lim = p.Sk - 1 - (int64_t)j * AT_N;
      if (p.causal) { const int64_t c = qrow - (int64_t)j * AT_N; lim = c < lim ? c : lim; }
      const bool need_mask = __any_sync(0xffffffffu, lim < AT_N - 1);
      uint32_t r[KC][32];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if constexpr (TPR == 2) {
        // the other part of the row: only its maximum is needed (one chunk at a time: its 32 registers are free again
        // before this thread's own scores are loaded)
#pragma unroll 1
        for (int c = 0; c < KC; c++) {
          const int col0 = (half ^ 1) * KW + c * 32;
          uint32_t t[32];
          tmem_ld_32x32(s_addr + (uint32_t)col0, t);
          tc_wait_ld();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; i++) if (col0 + i > lim) t[i] = 0xff800000u;
          }
#pragma unroll
          for (int i = 0; i < 16; i++) mx4[i & 3] = max3(mx4[i & 3], __uint_as_float(t[2 * i]), __uint_as_float(t[2 * i + 1]));
        }
      }
#pragma unroll
      for (int c = 0; c < KC; c++) tmem_ld_32x32(s_addr + (uint32_t)(half * KW + c * 32), r[c]);
      tc_wait_ld();
      if constexpr (!PT) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_se + 8 * s);
      } else if constexpr (TPR == 2) {
        // both threads of a row have read the scores before either overwrites part of them with probabilities
        asm volatile("bar.sync %0, 64;" ::"r"(1 + s * 4 + quad) : "memory");
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < KC; c++)
#pragma unroll
          for (int i = 0; i < 32; i++) if (half * KW + c * 32 + i > lim) r[c][i] = 0xff800000u;
      }
      float mx;
      {
#pragma unroll
        for (int c = 0; c < KC; c++)
#pragma unroll
          for (int i = 0; i < 16; i++) mx4[i & 3] = max3(mx4[i & 3], __uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
        mx = max3(mx4[0], mx4[1], max3(mx4[2], mx4[3], -INFINITY));
      }
      // a NaN score makes the whole row NaN (as max and sum do in the unfused program); keep the arithmetic finite
      // and poison the row sum at the end
      if (mx != mx) { poisoned = true; mx = 0.f; }
      float alpha = 1.f;
      bool rescale = false;
      if (it == 0) m_used = mx;
      else if ((mx - m_used) * p.scale_log2 > 8.0f) { alpha = fast_exp2((m_used - mx) * p.scale_log2); l *= alpha; m_used = mx; rescale = true; }
      // this stream's previous P V product must have retired before its accumulator is touched or its P overwritten
      if (it > 0) {
        if (!mbar_wait(bar_pv + 8 * s, (uint32_t)((it - 1) & 1), abort_flag, status, 18)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
          // each thread of a row rescales its share of the accumulator's columns (both took the same decision)
#pragma unroll 1
          for (int c = half * (D / 16 / TPR); c < (half + 1) * (D / 16 / TPR); c++) {
            // 16 columns at a time: the block's scores stay in registers meanwhile
            uint32_t o[16];
            tmem_ld_32x16(o_addr + (uint32_t)(c * 16), o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(o_addr + (uint32_t)(c * 16), o);
          }
          tc_wait_st();
        }
      }
      // p = exp2(s * scale_log2 - m * scale_log2) (a masked score is -inf and gives exactly 0), row sum, bf16 P into
      // swizzled shared memory; a fully masked row (m = -inf) gives 0 everywhere
      const float mneg = (m_used == -INFINITY) ? 0.f : -m_used * p.scale_log2;
      const uint32_t sc_bits = __float_as_uint(p.scale_log2), mn_bits = __float_as_uint(mneg);
      const uint64_t sc2 = pack2(sc_bits, sc_bits), mn2 = pack2(mn_bits, mn_bits);
      uint64_t ps2[2] = {0ull, 0ull};
#pragma unroll
      for (int c = 0; c < KC; c++) {
        uint32_t pw[16];                                  // 32 keys as bf16 pairs
        // 32 keys = 64 bytes = four 16-byte pieces of this row; piece index within the 128-byte line is XOR-swizzled
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; h++) {
            const int i = q * 8 + 2 * h;
            const uint64_t x2 = fma2(pack2(r[c][i], r[c][i + 1]), sc2, mn2);
            uint32_t t0, t1;
            unpack2(x2, t0, t1);
            const float e0 = fast_exp2(__uint_as_float(t0)), e1 = fast_exp2(__uint_as_float(t1));
            ps2[h & 1] = add2(ps2[h & 1], pack2(__float_as_uint(e0), __float_as_uint(e1)));
            __nv_bfloat162 t = __floats2bfloat162_rn(e0, e1);
            w[h] = *reinterpret_cast<uint32_t*>(&t);
          }
          if constexpr (PT) {
#pragma unroll
            for (int h = 0; h < 4; h++) pw[q * 4 + h] = w[h];
          } else {
            const int piece = (half * KW) / 8 + c * 4 + q;   // 0..15 over the 128 keys
            const int sub = piece >> 3, in = piece & 7;
            sts_v4(prow_s + (uint32_t)(sub * CHUNK_BYTES + ((in ^ (row & 7)) << 4)), w[0], w[1], w[2], w[3]);
          }
        }
        // key k of the block lives in column k / 2 of the stream's score buffer (low half of the word: the even key)
        if constexpr (PT) tmem_st_32x16(s_addr + (uint32_t)((half * KW) / 2 + c * 16), pw);
      }
      {
        uint32_t a0, a1, b0, b1;
        unpack2(ps2[0], a0, a1); unpack2(ps2[1], b0, b1);
        l += (__uint_as_float(a0) + __uint_as_float(a1)) + (__uint_as_float(b0) + __uint_as_float(b1));
      }
      if constexpr (PT) {
        tc_wait_st();
        tc_fence_before();
      } else {
        // P visible to the tensor-core (async) proxy
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pf + 8 * s);
    }
    // ---- merge the two streams and write O / l as bf16 ----
    if (ok && n_mine > 0) ok = mbar_wait(bar_pv + 8 * s, (uint32_t)((n_mine - 1) & 1), abort_flag, status, 19);
    if (poisoned) l = __int_as_float(0x7fc00000);
    *merge_slot(s, half, row) = make_float2((n_mine > 0 && m_used != -INFINITY) ? m_used * p.scale_log2 : -INFINITY, n_mine > 0 ? l : 0.f);
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_merge);
    if (ok) ok = mbar_wait(bar_merge, 0, abort_flag, status, 20);
    if (ok) {
      tc_fence_after();
      float2 mine = *merge_slot(s, 0, row), other = *merge_slot(s ^ 1, 0, row);
      if constexpr (TPR == 2) { mine.y += merge_slot(s, 1, row)->y; other.y += merge_slot(s ^ 1, 1, row)->y; }
      const float mm = fmaxf(mine.x, other.x);
      const float a_mine = (mine.x == -INFINITY) ? 0.f : fast_exp2(mine.x - mm);
      const float a_other = (other.x == -INFINITY) ? 0.f : fast_exp2(other.x - mm);
      const float lsum = mine.y * a_mine + other.y * a_other;
      const float inv = !(lsum <= 0.f) ? __fdividef(1.0f, lsum) : 0.f;   // a NaN sum stays NaN
      const float w_mine = a_mine * inv, w_other = a_other * inv;
      const bool have_mine = n_mine > 0, have_other = (nblk > (s ^ 1));
      const uint32_t o_mine = o_addr, o_other = tmem_base + lane_addr + 256u + (uint32_t)((s ^ 1) * D);
      __nv_bfloat16* orow = p.out + ((int64_t)bh * p.Sq + qrow) * D;
      // the 2 * TPR threads of a row share the head dimension: thread (s, half) writes columns [g * W, (g + 1) * W) with
      // g = s * TPR + half and W = D / (2 * TPR)
      constexpr int W = D / (2 * TPR);
      const int g = s * TPR + half;
      // 16 columns at a time: the merge is a cold path and must not set the kernel's register count
#pragma unroll 1
      for (int c = g * (W / 16); c < (g + 1) * (W / 16); c++) {
        uint32_t x[16], y[16];
        if (have_mine) tmem_ld_32x16(o_mine + (uint32_t)(c * 16), x);
        if (have_other) tmem_ld_32x16(o_other + (uint32_t)(c * 16), y);
        tc_wait_ld();
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
          float v = 0.f;
          if (have_mine) v = __uint_as_float(x[i]) * w_mine;
          if (have_other) v = fmaf(__uint_as_float(y[i]), w_other, v);
          f[i] = v;
        }
        if (qrow < p.Sq) {
#pragma unroll
          for (int q = 0; q < 2; q++) {
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 4; h++) {
              __nv_bfloat162 t = __floats2bfloat162_rn(f[q * 8 + 2 * h], f[q * 8 + 2 * h + 1]);
              w[h] = *reinterpret_cast<uint32_t*>(&t);
            }
            *reinterpret_cast<uint4*>(orow + c * 16 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------------------------------
// Persistent form: one CTA per SM, two independent workers per CTA.  A worker owns a whole query tile at a time (drawn
// from a device-wide counter in head-major, longest-prefix-first order), walks all of its key blocks, normalises and
// writes its rows, and draws the next tile; the other worker does the same on its own tile.  While one worker starts a
// tile (Q and first K in flight, first scores not there yet) or finishes one (last P V product, write-out), the tensor
// pipe and the special-function pipe work for the other, which the one-tile-per-CTA form above cannot offer: there every
// CTA pays its start-up and drain with the SM otherwise idle.  No merge of partial results is needed.
//
// Per worker: Q, one K stage, one V stage, half a probability buffer (64 keys: the P V product of a block is issued in two
// halves, and the second half's probabilities are computed while the first half multiplies), a 128-column score buffer
// and a D-column accumulator in TMEM.  384 threads:
//   warps 0,1   TMA producers (one per worker): draw the tile, publish it to the worker's other warps, load Q, K_j, V_j
//   warps 2,3   MMA issuers (one per worker)
//   warps 4..7  softmax of worker 0, warps 8..11 softmax of worker 1 (one thread per query row)
// Barrier phases are counted over the whole kernel (blocks, half-steps and tiles processed so far), not per tile.
template <int D>
struct AttnPwSmem {
  static constexpr int Q_BYTES = AT_M * D * 2;
  static constexpr int KV_BYTES = AT_N * D * 2;
  static constexpr int P_BYTES = AT_M * 64 * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + KV_BYTES;
  static constexpr int P_OFF = V_OFF + KV_BYTES;
  static constexpr int W_BYTES = P_OFF + P_BYTES;          // one worker
  static constexpr int BAR_OFF = 2 * W_BYTES;              // 2 x 16 barriers, TMEM slot, abort flag, tile rings
  static constexpr int TOTAL = BAR_OFF + 512 + 1024;
};

template <int D>
__global__ void __launch_bounds__(384, 1)
k_attention_pw(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ AttnParams p, int32_t* sched, int32_t* status) {
  using namespace sm100;
  using SM = AttnPwSmem<D>;
  constexpr int DC = D / 64;
  constexpr uint32_t TMEM_COLS = 512;          // S0 [0,128), S1 [128,256), O0 [256, 256 + D), O1 [256 + D, 256 + 2 D)
  constexpr uint32_t CHUNK_BYTES = 128 * 128;  // one [128 rows x 128 bytes] swizzled sub-tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + SM::BAR_OFF);
  uint32_t* tmem_slot = (uint32_t*)(bars + 32);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int w = warp < 4 ? (warp & 1) : ((warp - 4) >> 2);   // worker
  volatile int* ring = (volatile int*)(tmem_slot + 2) + 2 * w;   // the worker's current and next tile
  const uint32_t wb = smem_u32(bars) + (uint32_t)w * 128u;
  const uint32_t bar_qf = wb, bar_qe = wb + 8, bar_kf = wb + 16, bar_ke = wb + 24, bar_vf = wb + 32, bar_ve = wb + 40, bar_sf = wb + 48,
                 bar_se = wb + 56, bar_pf = wb + 64, bar_pv = wb + 72, bar_of = wb + 80, bar_tf = wb + 88 /* [2] */, bar_te = wb + 104 /* [2] */,
                 bar_drain = wb + 120;
  const uint32_t wbase = sbase + (uint32_t)w * SM::W_BYTES;
  const int total = (int)(p.BH * p.n_q_tiles);

  if (threadIdx.x == 0) {
    for (int v = 0; v < 2; v++) {
      const uint32_t b = smem_u32(bars) + (uint32_t)v * 128u;
      mbar_init(b, 1); mbar_init(b + 8, 1); mbar_init(b + 16, 1); mbar_init(b + 24, 1); mbar_init(b + 32, 1); mbar_init(b + 40, 1);
      mbar_init(b + 48, 1); mbar_init(b + 56, 4); mbar_init(b + 64, 4); mbar_init(b + 72, 1); mbar_init(b + 80, 4);
      mbar_init(b + 88, 1); mbar_init(b + 96, 1); mbar_init(b + 104, 5); mbar_init(b + 112, 5); mbar_init(b + 120, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile t: consecutive tiles are the query tiles of one (batch, head), longest causal prefix first
  auto decode = [&](int t, int& bh, int& q0, int& nblk) {
    bh = t / p.n_q_tiles;
    q0 = (p.n_q_tiles - 1 - t % p.n_q_tiles) * AT_M;
    int64_t k_end = p.Sk;
    if (p.causal && (int64_t)q0 + AT_M < k_end) k_end = (int64_t)q0 + AT_M;
    nblk = (int)((k_end + AT_N - 1) / AT_N);
  };

  if (warp < 2) {
    // ---------------------------------------------- TMA producer --------------------------------------------------
    if (lane == 0) {
      uint32_t kc = 0, vc = 0;       // K and V blocks loaded so far
      bool ok = true;
      for (int n = 0; ok; n++) {
        // the ring slot's previous tile has been read by the issuer and the four softmax warps
        if (n >= 2 && !mbar_wait(bar_te + 8 * (n & 1), (uint32_t)(((n >> 1) - 1) & 1), abort_flag, status, 21)) { ok = false; break; }
        int t = atomicAdd(sched, 1);
        if (t >= total) t = -1;
        ring[n & 1] = t;
        mbar_arrive(bar_tf + 8 * (n & 1));
        if (t < 0) break;
        int bh, q0, nblk;
        decode(t, bh, q0, nblk);
        // Q is free once the previous tile's last Q K^T has retired
        if (n > 0 && !mbar_wait(bar_qe, (uint32_t)((n - 1) & 1), abort_flag, status, 22)) { ok = false; break; }
        mbar_expect_tx(bar_qf, SM::Q_BYTES);
#pragma unroll
        for (int c = 0; c < DC; c++) tma_load_3d(wbase + SM::Q_OFF + c * CHUNK_BYTES, &tmQ, bar_qf, c * 64, q0, bh);
        int jk = 0, jv = 0;
        uint32_t idle = 0;
        while (jk < nblk || jv < nblk) {
          bool progress = false;
          if (jk < nblk && (kc == 0 || mbar_try_wait(bar_ke, (kc - 1) & 1))) {
            mbar_expect_tx(bar_kf, SM::KV_BYTES);
#pragma unroll
            for (int c = 0; c < DC; c++) tma_load_3d(wbase + SM::K_OFF + c * CHUNK_BYTES, &tmK, bar_kf, c * 64, jk * AT_N, bh);
            jk++; kc++; progress = true;
          }
          if (jv < nblk && (vc == 0 || mbar_try_wait(bar_ve, (vc - 1) & 1))) {
            mbar_expect_tx(bar_vf, SM::KV_BYTES);
#pragma unroll
            for (int c = 0; c < DC; c++) tma_load_3d(wbase + SM::V_OFF + c * CHUNK_BYTES, &tmV, bar_vf, c * 64, jv * AT_N, bh);
            jv++; vc++; progress = true;
          }
          if (progress) { idle = 0; continue; }
          if (++idle > (1u << 22)) { *abort_flag = 1; if (status) atomicCAS(status, 0, 11); ok = false; break; }
          if (idle > 16) { if (*abort_flag) { ok = false; break; } __nanosleep(idle > 4096 ? 256 : 32); }
        }
      }
      if (!ok) {
        // the other roles stop at their next wait; let copies already in flight land before shared memory goes away
        for (uint32_t i = 0; i < 4096; i++) __nanosleep(256);
      }
    }
  } else if (warp < 4) {
    // ---------------------------------------------- MMA issuer ------------------------------------------------------
    if (lane == 0) {
      uint32_t kc = 0, vc = 0, hc = 0;     // score blocks issued, V blocks consumed, P V half-steps issued
      const uint32_t s_tmem = tmem_base + (uint32_t)(w * 128), o_tmem = tmem_base + 256u + (uint32_t)(w * D);
      const uint32_t qa = wbase + SM::Q_OFF, ka = wbase + SM::K_OFF, va = wbase + SM::V_OFF, pa = wbase + SM::P_OFF;
      bool ok = true;
      auto issue_qk = [&](bool last_of_tile) -> bool {
        if (!mbar_wait(bar_kf, kc & 1, abort_flag, status, 13)) return false;
        // the worker's softmax has copied the previous block's scores into registers
        if (kc > 0 && !mbar_wait(bar_se, (kc - 1) & 1, abort_flag, status, 14)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; k++) {
          const uint32_t off = (uint32_t)(k >> 2) * CHUNK_BYTES + (uint32_t)(k & 3) * 32;
          umma_ss<false>(s_tmem, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), p.idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(bar_sf);
        tc_commit(bar_ke);
        if (last_of_tile) tc_commit(bar_qe);
        kc++;
        return true;
      };
      for (int n = 0; ok; n++) {
        if (!mbar_wait(bar_tf + 8 * (n & 1), (uint32_t)((n >> 1) & 1), abort_flag, status, 23)) { ok = false; break; }
        const int t = ring[n & 1];
        mbar_arrive(bar_te + 8 * (n & 1));
        if (t < 0) break;
        int bh, q0, nblk;
        decode(t, bh, q0, nblk);
        if (!mbar_wait(bar_qf, (uint32_t)(n & 1), abort_flag, status, 12)) { ok = false; break; }
        if (!issue_qk(nblk == 1)) { ok = false; break; }
        for (int it = 0; it < nblk && ok; it++) {
          // the block's scores are in the softmax warps' registers early: the next score block goes ahead of this
          // block's products
          if (it + 1 < nblk && !issue_qk(it + 2 == nblk)) { ok = false; break; }
          if (!mbar_wait(bar_vf, vc & 1, abort_flag, status, 15)) { ok = false; break; }
          // the previous tile's rows have been read out of the accumulator
          if (it == 0 && n > 0 && !mbar_wait(bar_of, (uint32_t)((n - 1) & 1), abort_flag, status, 24)) { ok = false; break; }
#pragma unroll
          for (int h = 0; h < 2; h++) {
            if (!mbar_wait(bar_pf, hc & 1, abort_flag, status, 16)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; k++) {
              // A = P (K-major: 64 keys contiguous per row); B = V (MN-major: head-dim chunks of 64 are CHUNK_BYTES apart)
              const int kk = 4 * h + k;
              umma_ss<false>(o_tmem, make_smem_desc(pa + (uint32_t)k * 32, 16, 1024), make_smem_desc(va + (uint32_t)kk * 2048, CHUNK_BYTES, 1024), p.idesc_pv,
                             (it > 0 || kk > 0) ? 1u : 0u);
            }
            tc_commit(bar_pv);     // the half's probabilities have been read; the accumulator holds them
            hc++;
          }
          if (!ok) break;
          tc_commit(bar_ve);
          vc++;
        }
      }
      // everything this thread issued must retire before TMEM is released
      tc_commit(bar_drain);
      mbar_wait(bar_drain, 0, abort_flag, nullptr, 0);
    }
  } else {
    // ---------------------------------------------- softmax ---------------------------------------------------------
    const int quad = warp & 3;                    // TMEM lanes [32 * quad, 32 * quad + 32): fixed by the warp's number
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)(w * 128);
    const uint32_t o_addr = tmem_base + lane_addr + 256u + (uint32_t)(w * D);
    const uint32_t prow_s = wbase + (uint32_t)(SM::P_OFF + row * 128);
    const uint32_t sw = (uint32_t)(row & 7);
    uint32_t sc = 0, hc = 0;                      // score blocks consumed, probability half-steps published
    bool ok = true;
    // 32 scores -> exp2, partial row sums, 16 words of bf16 pairs
    auto exps = [&](const uint32_t (&r)[32], uint64_t sc2, uint64_t mn2, uint64_t (&ps2)[2], uint32_t (&pw)[16]) {
#pragma unroll
      for (int h = 0; h < 16; h++) {
        const uint64_t x2 = fma2(pack2(r[2 * h], r[2 * h + 1]), sc2, mn2);
        uint32_t t0, t1;
        unpack2(x2, t0, t1);
        const float e0 = fast_exp2(__uint_as_float(t0)), e1 = fast_exp2(__uint_as_float(t1));
        ps2[h & 1] = add2(ps2[h & 1], pack2(__float_as_uint(e0), __float_as_uint(e1)));
        __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
        pw[h] = *reinterpret_cast<uint32_t*>(&b);
      }
    };
    // chunk c (32 keys = four 16-byte pieces) of the 64-key half into the swizzled probability buffer
    auto store = [&](int c, const uint32_t (&pw)[16]) {
#pragma unroll
      for (int q = 0; q < 4; q++)
        sts_v4(prow_s + ((((uint32_t)((c & 1) * 4 + q)) ^ sw) << 4), pw[4 * q], pw[4 * q + 1], pw[4 * q + 2], pw[4 * q + 3]);
    };
    auto publish = [&]() {
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pf);
      hc++;
    };
    for (int n = 0; ok; n++) {
      if (!mbar_wait(bar_tf + 8 * (n & 1), (uint32_t)((n >> 1) & 1), abort_flag, status, 25)) { ok = false; break; }
      const int t = ring[n & 1];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_te + 8 * (n & 1));
      if (t < 0) break;
      int bh, q0, nblk;
      decode(t, bh, q0, nblk);
      const int64_t qrow = (int64_t)q0 + row;
      float m_used = -INFINITY, l = 0.f;
      bool poisoned = false;
      for (int it = 0; it < nblk && ok; it++) {
        if (!mbar_wait(bar_sf, sc & 1, abort_flag, status, 17)) { ok = false; break; }
        tc_fence_after();
        // columns of this block that this row may attend to: [0, lim]
        int64_t lim = p.Sk - 1 - (int64_t)it * AT_N;
        if (p.causal) { const int64_t c = qrow - (int64_t)it * AT_N; lim = c < lim ? c : lim; }
        const bool need_mask = __any_sync(0xffffffffu, lim < AT_N - 1);
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; c++) tmem_ld_32x32(s_addr + (uint32_t)(c * 32), r[c]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_se);
        sc++;
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 4; c++)
#pragma unroll
            for (int i = 0; i < 32; i++) if (c * 32 + i > lim) r[c][i] = 0xff800000u;
        }
        float mx;
        {
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 4; c++)
#pragma unroll
            for (int i = 0; i < 16; i++) mx4[i & 3] = max3(mx4[i & 3], __uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
          mx = max3(mx4[0], mx4[1], max3(mx4[2], mx4[3], -INFINITY));
        }
        // a NaN score makes the whole row NaN (as max and sum do in the unfused program); keep the arithmetic finite
        // and poison the row sum at the end
        if (mx != mx) { poisoned = true; mx = 0.f; }
        float alpha = 1.f;
        bool rescale = false;
        if (it == 0) m_used = mx;
        else if ((mx - m_used) * p.scale_log2 > 8.0f) { alpha = fast_exp2((m_used - mx) * p.scale_log2); l *= alpha; m_used = mx; rescale = true; }
        if (it > 0) {
          // the previous block's second half-product has retired: the probability buffer is free and the accumulator at rest
          if (!mbar_wait(bar_pv, (hc - 1) & 1, abort_flag, status, 18)) { ok = false; break; }
          tc_fence_after();
          if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
            for (int c = 0; c < D / 16; c++) {
              uint32_t o[16];
              tmem_ld_32x16(o_addr + (uint32_t)(c * 16), o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st_32x16(o_addr + (uint32_t)(c * 16), o);
            }
            tc_wait_st();
          }
        }
        const float mneg = (m_used == -INFINITY) ? 0.f : -m_used * p.scale_log2;
        const uint32_t sc_bits = __float_as_uint(p.scale_log2), mn_bits = __float_as_uint(mneg);
        const uint64_t sc2 = pack2(sc_bits, sc_bits), mn2 = pack2(mn_bits, mn_bits);
        uint64_t ps2[2] = {0ull, 0ull};
        {
          uint32_t pw[16];
          exps(r[0], sc2, mn2, ps2, pw); store(0, pw);
          exps(r[1], sc2, mn2, ps2, pw); store(1, pw);
        }
        publish();
        {
          // the second half: its first 32 keys are exponentiated while the first half multiplies
          uint32_t pw[16];
          exps(r[2], sc2, mn2, ps2, pw);
          if (!mbar_wait(bar_pv, (hc - 1) & 1, abort_flag, status, 19)) { ok = false; break; }
          store(0, pw);
          exps(r[3], sc2, mn2, ps2, pw); store(1, pw);
        }
        publish();
        {
          uint32_t a0, a1, b0, b1;
          unpack2(ps2[0], a0, a1); unpack2(ps2[1], b0, b1);
          l += (__uint_as_float(a0) + __uint_as_float(a1)) + (__uint_as_float(b0) + __uint_as_float(b1));
        }
      }
      if (!ok) break;
      // ---- the tile's last product has retired: normalise and write the rows as bf16 ----
      if (!mbar_wait(bar_pv, (hc - 1) & 1, abort_flag, status, 20)) { ok = false; break; }
      tc_fence_after();
      if (poisoned) l = __int_as_float(0x7fc00000);
      const float inv = !(l <= 0.f) ? __fdividef(1.0f, l) : 0.f;   // a NaN sum stays NaN
      __nv_bfloat16* orow = p.out + ((int64_t)bh * p.Sq + qrow) * D;
#pragma unroll 1
      for (int c = 0; c < D / 16; c++) {
        uint32_t x[16];
        tmem_ld_32x16(o_addr + (uint32_t)(c * 16), x);
        tc_wait_ld();
        if (qrow < p.Sq) {
#pragma unroll
          for (int q = 0; q < 2; q++) {
            uint32_t wd[4];
#pragma unroll
            for (int h = 0; h < 4; h++) {
              __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(x[q * 8 + 2 * h]) * inv, __uint_as_float(x[q * 8 + 2 * h + 1]) * inv);
              wd[h] = *reinterpret_cast<uint32_t*>(&b);
            }
            *reinterpret_cast<uint4*>(orow + c * 16 + q * 8) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_of);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  // the last CTA to leave puts the tile counter back for the stream's next launch
  if (threadIdx.x == 0 && atomicAdd(sched + 1, 1) == (int)gridDim.x - 1) { sched[0] = 0; sched[1] = 0; __threadfence(); }
}

int32_t* sched_slot(cudaStream_t stream);   // defined in gemm_tc.cu: a (tile counter, finished CTAs) pair per stream

// Returns -1 when the stream has no scheduler pair (the caller then uses the one-tile-per-CTA form).
template <int D>
static int launch_attention_pw(const B2xAttentionArgs* a, int32_t* status, cudaStream_t stream) {
  using SM = AttnPwSmem<D>;
  int32_t* sched = sched_slot(stream);
  if (!sched) return -1;
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
  auto kern = k_attention_pw<D>;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    static std::atomic<bool> configured[64];
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
  }
  const int64_t tiles = (int64_t)p.n_q_tiles * a->BH;
  if (tiles <= 0) return 0;
  if (tiles > 0x7fffff00) return (int)cudaErrorInvalidValue;
  const int64_t ctas = (tiles + 1) / 2 < kNumSms ? (tiles + 1) / 2 : kNumSms;
  kern<<<(unsigned)ctas, 384, SM::TOTAL, stream>>>(tmQ, tmK, tmV, p, sched, status);
  count_launch();
  return (int)cudaGetLastError();
}

template <int D, int TPR, bool PT>
static int launch_attention(const B2xAttentionArgs* a, int32_t* status, cudaStream_t stream) {
  using SM = AttnSmem<D, PT>;
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
  auto kern = k_attention<D, TPR, PT>;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    static std::atomic<bool> configured[64];
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
  }
  const int64_t grid = (int64_t)p.n_q_tiles * a->BH;
  if (grid <= 0) return 0;
  if (grid > 0x7fffffff) return (int)cudaErrorInvalidValue;
  kern<<<(unsigned)grid, 96 + 256 * TPR, SM::TOTAL, stream>>>(tmQ, tmK, tmV, p, status);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace b2x

extern "C" int b2x_launch_attention(const B2xAttentionArgs* a, int32_t* status, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->BH <= 0 || a->Sq <= 0 || a->Sk <= 0) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)a->q & 15) || ((uintptr_t)a->k & 15) || ((uintptr_t)a->v & 15) || ((uintptr_t)a->o & 15)) return (int)cudaErrorInvalidValue;
  // Variants kept for comparison, both measured slower on the 4096 x 128 causal case (0.85 ms and 0.72 ms against 0.68 ms):
  // B2X_ATTENTION_P=tmem (probabilities through TMEM as the second MMA's A operand: frees the P buffers, but a stream's next
  // score block must then wait for its P V product), B2X_ATTENTION_THREADS_PER_ROW=2 (two threads share a query row)
  // The persistent two-worker form is the default (0.64 ms on the 4096 x 128 causal case against 0.68 ms);
  // B2X_ATTENTION_KERNEL=tile selects the one-tile-per-CTA form and its variants below.
  const char* form = getenv("B2X_ATTENTION_KERNEL");
  if (!(form && form[0] == 't') && (a->D == 128 || a->D == 64)) {
    const int rc = a->D == 128 ? launch_attention_pw<128>(a, status, stream) : launch_attention_pw<64>(a, status, stream);
    if (rc != -1) return rc;
  }
  const char* tpr = getenv("B2X_ATTENTION_THREADS_PER_ROW");
  const char* pv = getenv("B2X_ATTENTION_P");
  const bool two = tpr && tpr[0] == '2';
  const bool via_smem = !(pv && pv[0] == 't');
  if (a->D == 128) {
    if (via_smem) return two ? launch_attention<128, 2, false>(a, status, stream) : launch_attention<128, 1, false>(a, status, stream);
    return two ? launch_attention<128, 2, true>(a, status, stream) : launch_attention<128, 1, true>(a, status, stream);
  }
  if (a->D == 64) {
    if (via_smem) return two ? launch_attention<64, 2, false>(a, status, stream) : launch_attention<64, 1, false>(a, status, stream);
    return two ? launch_attention<64, 2, true>(a, status, stream) : launch_attention<64, 1, true>(a, status, stream);
  }
  return (int)cudaErrorInvalidValue;
}
