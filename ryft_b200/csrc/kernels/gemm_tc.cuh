// stablehlo.dot_general on the 5th-generation tensor cores: a persistent, warp-specialised tcgen05 GEMM.
//
//   C[b][m][n] = sum_k A[b][m][k] * B[b][k][n],  A and B bf16 / f16 (kind::f16) or f32 read as TF32 (kind::tf32),
//   f32 accumulation in TMEM, result handed to the fused elementwise epilogue program (vm.cuh) which does the stores.
//
// One CTA per SM (grid = min(tiles, 148)), 64 + 32 * TC_EPI_WARPS threads:
//   warp 0     TMA producer: per k-block one 128 x BK tile of A and one BN x BK tile of B into a STAGES-deep ring of
//              128-byte-swizzled shared-memory buffers (cp.async.bulk.tensor, each CTA loads its own tiles);
//   warp 1     MMA issuer: one elected lane issues tcgen05.mma (128 x BN x 16) over the ring, commits each stage back
//              to the producer and each finished accumulator to the epilogue; also owns TMEM allocation;
//   warps 2..  epilogue: tcgen05.ld the 128 x BN f32 accumulator (each warp its 32 lanes and every fourth 32-column
//              chunk, so that four warps per scheduler hide each other's latencies), run the epilogue program on
//              8-wide row vectors and store.  Two accumulators (2 x BN TMEM columns) let tile i's epilogue overlap
//              tile i+1's main loop.
// Either operand may be K-major (k contiguous) or MN-major (m or n contiguous); the second form covers the
// transposed contractions of a backward pass without materialising a transpose.
// Bound: tensor pipe for K >= ~1024 (algorithmic FLOPs = 2*B*M*N*K); HBM (output bytes) for short K.
// Every mbarrier wait is bounded (sm100.cuh); on expiry the CTA unwinds, frees TMEM and reports through `status`.
#pragma once
#include <atomic>
#include <type_traits>
#include <cstdlib>
#include <cstring>
#include "../../../include/b2x_kernels.h"
#include "common.cuh"
#include "sm100.cuh"
#include "vm.cuh"

namespace b2x {

struct TcParams {
  int64_t batch, M, N, K;
  int32_t a_mn_major, b_mn_major;
  // The MN-major operand's map is the folded 4-D form (encode_mn_major_4d): one load per stage instead of one per
  // 128-byte-wide sub-tile.  The producer is one thread; with five or six loads per k-block it needed 700-750 cycles per
  // k-block, more than the 512 cycles the tensor pipe takes to consume one, and the MLP step ran 8-12 % slower.
  int32_t a_mn_4d, b_mn_4d;
  // Tall tiles (256 x 256, only the <256, 4> kernels on long-K 16-bit problems): a stage is 256 rows of A and 256 of B
  // (64 KB, three stages in the same 192 KB ring), every k-step issues two MMAs that share the B sub-tile, one into each
  // 256-column accumulator, and epilogue group g drains accumulator g = rows [128 g, 128 g + 128) of the tile.  Operand
  // bytes per FLOP drop by a third (62.5 instead of 94 bytes per clock and SM at full tensor rate) and a stage covers
  // 1024 cycles of tensor work instead of 512; the price is that the epilogue no longer overlaps the next tile's MMAs.
  int32_t tall;
  // Short-K problems (a tile is at most three k-blocks, only the <256, 4> kernels): three stages instead of four, and the
  // freed 48 KB double the bulk-store epilogue's staging tiles, so that a warp fills one while the TMA engine still reads the
  // other (with one tile it waited 200-350 cycles per strip for the previous store to have read it).
  int32_t short_k;
  int32_t num_m_tiles, num_n_tiles;
  int64_t num_tiles;
  int32_t k_blocks;
  int32_t tma_store;   // the single-store epilogue writes through the output tensor map
  int32_t epi_groups;  // 2: one group of eight epilogue warps per accumulator; 1: all sixteen on every tile (short K)
  int32_t transposed;  // multi-store epilogues on short-K problems go through shared memory (see tc_transposed_epilogue)
  int32_t group_m;     // m-tiles per raster group: a group's A slab stays in L2 while its n-tiles stream by
  uint32_t idesc;
  int32_t* sched;      // [0] next tile to hand out, [1] CTAs that have finished (the last one resets both)
  int32_t withhold;    // test switch: CTA 0 never announces its first tile, so that the waits of its other roles run out
};

constexpr int TC_BM = 128;
constexpr int TC_EPI_WARPS = 16;                    // four per TMEM lane quarter, i.e. four per warp scheduler
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;
// The epilogue warps form two groups of eight, one per TMEM accumulator: group g finishes tiles g, g + 2, ... of the CTA
// on its own.  The groups drift out of phase (one reads TMEM or stores while the other is in its MUFU-heavy part), and
// each warp's per-tile set-up is amortised over twice as many columns as with all sixteen warps on every tile.
// That holds when a tile's main loop is long.  With a short K (config 2: two k-blocks per tile) the epilogue is the
// bottleneck and a group would sit idle while the MMA refills its accumulator, so there all sixteen warps finish every
// tile together and the accumulators alternate (TcParams::epi_groups = 1).

// Tile order: batches outermost; inside a batch, groups of `group_m` m-tiles, and inside a group m fastest.  Tiles that
// run at the same time then share a few rows of A and a few columns of B, and consecutive waves reuse the group's A
// slab out of L2 instead of streaming all of A from HBM once per wave.
__device__ __forceinline__ void tc_tile_coords(const struct TcParams& p, int64_t t, int BN, int* b, int* m0, int* n0);

__device__ __forceinline__ void tc_tile_coords(const TcParams& p, int64_t t, int BN, int* b, int* m0, int* n0) {
  // the launcher rejects problems with 2^31 or more tiles, so 32-bit divisions suffice
  const uint32_t per_batch = (uint32_t)p.num_m_tiles * (uint32_t)p.num_n_tiles;
  const uint32_t t32 = (uint32_t)t;
  const uint32_t bb = t32 / per_batch;
  const uint32_t r = t32 - bb * per_batch;
  const uint32_t per_group = (uint32_t)p.group_m * (uint32_t)p.num_n_tiles;
  const uint32_t g = r / per_group;
  const uint32_t in = r - g * per_group;
  const uint32_t gm = (uint32_t)min(p.group_m, p.num_m_tiles - (int)g * p.group_m);
  const uint32_t nn = in / gm;
  *b = (int)bb;
  *m0 = (int)(g * (uint32_t)p.group_m + (in - nn * gm)) * (p.tall ? 2 * TC_BM : TC_BM);
  *n0 = (int)nn * BN;
}

// A warp-wide store with one row per lane keeps the load/store unit busy for 32 cycles (one per cache line touched);
// with four lanes per row it is 8, but the round trip through shared memory costs about as much as one such store.
// Measured on the MLP step: a two-store epilogue behind a K = 4096 GEMM gains 11 %; single-store programs, and epilogues
// behind a K = 16384 GEMM (which have four times as long per tile), lose a few per cent to the extra work.  So the
// transposed path is compiled for programs with two or more stores and taken when K <= 8192.
template <int ID>
__host__ __device__ constexpr bool tc_transposed_epilogue() {
  if constexpr (ID == 0) return false;
  else return vm_static_stores<ID>() >= 2;
}

// Single-store programs writing 16- or 32-bit elements put their result tile into shared memory and let the TMA engine
// store it: the load/store unit then sees one shared-memory pass (a few wavefronts per warp) instead of 32 cache lines
// per warp-wide store, and ragged M / N edges are clipped by the tensor map.
template <int ID>
__host__ __device__ constexpr bool tc_tma_store_epilogue() {
  if constexpr (ID == 0) return false;
  else if constexpr (vm_static_stores<ID>() != 1) return false;
  else {
    const uint8_t e = VmStatic<ID>::elem(vm_static_store_tensor<ID>());
    return e == EL_BF16 || e == EL_F16 || e == EL_F32 || e == EL_S32 || e == EL_U32 || e == EL_S16 || e == EL_U16;
  }
}
template <int ID>
__host__ __device__ constexpr int tc_store_elem_size() {
  if constexpr (!tc_tma_store_epilogue<ID>()) return 0;
  else {
    const uint8_t e = VmStatic<ID>::elem(vm_static_store_tensor<ID>());
    return (e == EL_F32 || e == EL_S32 || e == EL_U32) ? 4 : 2;
  }
}

template <int BN, int STAGES, bool TF32, bool STAGING>
struct TcSmem {
  static constexpr int A_BYTES = TC_BM * 128;   // 128 rows (or k-lines x chunks) of 128 bytes
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;             // 1024-byte aligned (swizzled store boxes)
  // per epilogue warp 16 rows of 32 f32 columns; only kernels that contain the transposed epilogue pay for it (shared
  // memory a kernel does not ask for stays available to the SM as L1 cache)
  static constexpr int STAGING_BYTES = STAGING ? TC_EPI_WARPS * 2048 : 0;
  static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING_BYTES;       // barriers, TMEM slot, tile ring: 384 bytes
  static constexpr int TOTAL = BAR_OFFSET + 384 + 1024;                   // + slack for 1024-byte alignment
};

template <int BN, int STAGES, bool TF32, int ID>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmOut,
          const __grid_constant__ TcParams p,
          const __grid_constant__ B2xVmProgram epi, int32_t* status) {
  using namespace sm100;
  using SM = TcSmem<BN, STAGES, TF32, tc_transposed_epilogue<ID>() || tc_tma_store_epilogue<ID>()>;
  constexpr int ES = TF32 ? 4 : 2;
  constexpr int BK = 128 / ES;            // elements per 128-byte line: 64 (16-bit) or 32 (tf32)
  constexpr int UMMA_K = 32 / ES;         // 16 or 8
  constexpr int CHUNK = 128 / ES;         // MN-elements per 128-byte line in MN-major layout
  // Accumulators in TMEM.  Four 128-column accumulators (a pair for each of two epilogue groups, 128-wide tiles on
  // short-K problems) were measured on config 2: 107 us against 92 us with two 256-column ones and one group, so two it is.
  constexpr int NACC = 2;
  constexpr uint32_t TMEM_COLS = (NACC * BN <= 32) ? 32 : (NACC * BN <= 64 ? 64 : (NACC * BN <= 128 ? 128 : (NACC * BN <= 256 ? 256 : 512)));

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + SM::BAR_OFFSET);
  // barrier slots: full[STAGES], empty[STAGES], tmem_full[NACC], tmem_empty[NACC], drain, sched_full[4], sched_empty[4]
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES, bar_tfull = bar_empty + 8 * STAGES,
                 bar_tempty = bar_tfull + 8 * NACC, bar_drain = bar_tempty + 8 * NACC, bar_sfull = bar_drain + 8, bar_sempty = bar_sfull + 32;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 2 * NACC + 1 + 8);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  // Tiles are handed out dynamically: the producer draws the next tile index from a global counter and publishes it
  // to the other roles through this ring, so a CTA that starts late (its SM was busy with another kernel, e.g. a
  // collective) simply takes fewer tiles.
  // A ring entry is {tile, batch, m0, n0}: the producer decomposes the tile index once for all roles.
  volatile int32_t* tile_ring = (volatile int32_t*)(tmem_slot + 2);
  constexpr int RING = 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int a = 0; a < NACC; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, TC_EPI_WARPS / p.epi_groups); }
    mbar_init(bar_drain, 1);
    for (int r = 0; r < RING; r++) { mbar_init(bar_sfull + 8 * r, 1); mbar_init(bar_sempty + 8 * r, (p.tall ? TC_EPI_WARPS : TC_EPI_WARPS / p.epi_groups) + 1); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // stage geometry: the ring is STAGES * STAGE_BYTES either way (tall tiles are only routed to the <256, 4> kernels,
  // whose 4 x 48 KB ring is 3 x 64 KB)
  const int n_stages = (p.tall || p.short_k) ? 3 : STAGES;
  const uint32_t a_bytes = p.tall ? 2u * SM::A_BYTES : (uint32_t)SM::A_BYTES;
  const uint32_t stage_bytes = a_bytes + (uint32_t)SM::B_BYTES;


  if (warp == 0) {
    // ------------------------------------------------ TMA producer ------------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // The next tile is drawn one tile ahead: the atomic's round trip to L2 overlaps the loads of the current tile
      // instead of standing between two tiles (it is a large part of a tile's time when K is one or two blocks).
      int64_t t_next = (int64_t)atomicAdd(p.sched, 1);
      for (int64_t local = 0; ok; local++) {
        const int slot = (int)(local & (RING - 1));
        if (!mbar_wait(bar_sempty + 8 * slot, (uint32_t)(((local / RING) & 1) ^ 1), abort_flag, status, 5)) { ok = false; break; }
        int64_t t = t_next;
        if (t >= p.num_tiles) t = -1;
        else t_next = (int64_t)atomicAdd(p.sched, 1);
        int b = 0, m0 = 0, n0 = 0;
        if (t >= 0) tc_tile_coords(p, t, BN, &b, &m0, &n0);
        tile_ring[slot * 4 + 0] = (int32_t)t; tile_ring[slot * 4 + 1] = b; tile_ring[slot * 4 + 2] = m0; tile_ring[slot * 4 + 3] = n0;
        if (!(p.withhold && local == 0 && blockIdx.x == 0)) mbar_arrive(bar_sfull + 8 * slot);
        if (t < 0 && (p.epi_groups == 1 || p.tall)) break;
        if (t < 0) {
          // the other epilogue group reads the ring entry after this one: it gets its own end marker
          const int64_t nxt = local + 1;
          const int slot2 = (int)(nxt & (RING - 1));
          if (mbar_wait(bar_sempty + 8 * slot2, (uint32_t)(((nxt / RING) & 1) ^ 1), abort_flag, status, 5)) {
            tile_ring[slot2 * 4] = -1;
            mbar_arrive(bar_sfull + 8 * slot2);
          }
          break;
        }
        for (int kb = 0; kb < p.k_blocks; kb++) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status, 1)) { ok = false; break; }
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, stage_bytes);
          const uint32_t sa = smem_base + stage * stage_bytes, sb = sa + a_bytes;
          const int k0 = kb * BK;
          if (!p.a_mn_major) tma_load_3d(sa, &tmA, full, k0, m0, b);
          else if (p.a_mn_4d) tma_load_4d(sa, &tmA, full, 0, k0, m0 / CHUNK, b);
          else {
#pragma unroll
            for (int c = 0; c < TC_BM / CHUNK; c++) tma_load_3d(sa + c * (BK * 128), &tmA, full, m0 + c * CHUNK, k0, b);
            if (p.tall) {
#pragma unroll
              for (int c = TC_BM / CHUNK; c < 2 * TC_BM / CHUNK; c++) tma_load_3d(sa + c * (BK * 128), &tmA, full, m0 + c * CHUNK, k0, b);
            }
          }
          if (!p.b_mn_major) tma_load_3d(sb, &tmB, full, k0, n0, b);
          else if (p.b_mn_4d) tma_load_4d(sb, &tmB, full, 0, k0, n0 / CHUNK, b);
          else {
#pragma unroll
            for (int c = 0; c < BN / CHUNK; c++) tma_load_3d(sb + c * (BK * 128), &tmB, full, n0 + c * CHUNK, k0, b);
          }
          if (++stage == n_stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // unwind: let copies already in flight land before the CTA's shared memory goes away
        for (int s = 0; s < STAGES; s++) {
          for (uint32_t i = 0; i < (1u << 16); i++) { if (mbar_try_wait(bar_full + 8 * s, 0) || mbar_try_wait(bar_full + 8 * s, 1)) break; __nanosleep(64); }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer ----------------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t local = 0; ok; local++) {
        const int slot = (int)(local & (RING - 1));
        if (!mbar_wait(bar_sfull + 8 * slot, (uint32_t)((local / RING) & 1), abort_flag, status, 6)) { ok = false; break; }
        const int32_t t = tile_ring[slot * 4];
        mbar_arrive(bar_sempty + 8 * slot);
        if (t < 0) break;
        const int acc = p.tall ? 0 : (int)(local % NACC);
        const uint32_t acc_phase = p.tall ? (uint32_t)(local & 1) : (uint32_t)((local / NACC) & 1);
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, status, 2)) { ok = false; break; }
        if (p.tall && !mbar_wait(bar_tempty + 8, acc_phase ^ 1, abort_flag, status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < p.k_blocks; kb++) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * stage_bytes, sb = sa + a_bytes;
          // K-major: 8-row groups 1024 B apart, k advances 32 B inside the swizzle atom.
          // MN-major: 64/32-element chunks BK*128 B apart, 8 k-lines per 1024 B group, k advances UMMA_K lines.
          const uint64_t a_desc0 = p.a_mn_major ? make_smem_desc(sa, BK * 128, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t b_desc0 = p.b_mn_major ? make_smem_desc(sb, BK * 128, 1024) : make_smem_desc(sb, 16, 1024);
          const uint32_t a_adv = p.a_mn_major ? (UMMA_K * 128) >> 4 : 32 >> 4;
          const uint32_t b_adv = p.b_mn_major ? (UMMA_K * 128) >> 4 : 32 >> 4;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            umma_ss<TF32>(d_tmem, a_desc0 + (uint64_t)(k * a_adv), b_desc0 + (uint64_t)(k * b_adv), p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
            // tall tiles: rows 128..255 of the stage's A (16 KB further in either layout) against the same B sub-tile
            if (p.tall) umma_ss<TF32>(d_tmem + (uint32_t)BN, a_desc0 + (uint64_t)(k * a_adv) + (uint64_t)(SM::A_BYTES >> 4), b_desc0 + (uint64_t)(k * b_adv), p.idesc,
                                      (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * stage);   // frees the stage once the MMAs above have read it
          if (++stage == n_stages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(bar_tfull + 8 * acc);  // accumulator complete
        if (ok && p.tall) tc_commit(bar_tfull + 8);
      }
      // drain: everything issued must retire before TMEM is released
      tc_commit(bar_drain);
      mbar_wait(bar_drain, 0, abort_flag, nullptr, 0);
    }
  } else {
    // ------------------------------------------------ epilogue ------------------------------------------------------
    const int quad = warp & 3;              // TMEM lanes [32*quad, 32*quad + 32)
    const int group_warps = TC_EPI_WARPS / p.epi_groups;
    const int group = (warp - 2) / group_warps;                  // with two groups: the accumulator this warp serves
    const int part = ((warp - 2) % group_warps) >> 2;            // column chunks part, part + col_parts, ...
    const int col_parts = group_warps / 4;
    bool ok = true;
    uint32_t stg_sel = 0;
    const VmRowPlan rplan = vm_row_plan(epi, (uint32_t)p.N);
    for (int64_t local = p.tall ? 0 : group; ok; local += p.tall ? 1 : p.epi_groups) {
      const int slot = (int)(local & (RING - 1));
      if (!mbar_wait(bar_sfull + 8 * slot, (uint32_t)((local / RING) & 1), abort_flag, status, 7)) { ok = false; break; }
      const int64_t t = tile_ring[slot * 4];
      const int b = tile_ring[slot * 4 + 1], m0 = tile_ring[slot * 4 + 2] + (p.tall ? group * TC_BM : 0), n0 = tile_ring[slot * 4 + 3];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sempty + 8 * slot);
      if (t < 0) break;
      const int acc = p.tall ? group : (int)(local % NACC);
      const uint32_t acc_phase = p.tall ? (uint32_t)(local & 1) : (uint32_t)((local / NACC) & 1);
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, status, 4)) { ok = false; break; }
      tc_fence_after();
      const int64_t row = (int64_t)m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      if constexpr (tc_transposed_epilogue<ID>()) {
        // Transposed epilogue: the accumulator chunk goes through shared memory so that four adjacent lanes own one
        // row's 32 columns.  Every global access of the program is then contiguous over 4 lanes x 8 elements (128 bytes
        // of f32, 64 of bf16) instead of one 16-byte piece per row.
        const int wrow0 = m0 + quad * 32;
        int nrows = (int)min((int64_t)32, p.M - (int64_t)wrow0);
        VmRowBlock blk;
        blk.ok = false;
        if (p.transposed) vm_row_block(epi, rplan, (uint64_t)((int64_t)b * p.M + (nrows > 0 ? wrow0 : 0)), (uint32_t)(nrows > 0 ? nrows : 1), (uint32_t)p.N, blk);
        if (__all_sync(0xffffffffu, blk.ok)) {
          const uint32_t stg = smem_base + SM::STAGING_OFFSET + (uint32_t)(warp - 2) * 2048u;
#pragma unroll 1
          for (int c = part; c < BN / 32; c += col_parts) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 32), r);
            tc_wait_ld();
            const int col = n0 + c * 32 + (lane & 3) * 8;
#pragma unroll
            for (int half = 0; half < 2; half++) {
              __syncwarp();
              if ((lane >> 4) == half) {
                const uint32_t rowaddr = stg + (uint32_t)(lane & 15) * 128u;
#pragma unroll
                for (int j = 0; j < 8; j++) sts_v4(rowaddr + (uint32_t)((j ^ (lane & 7)) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              }
              __syncwarp();
#pragma unroll
              for (int run = 0; run < 2; run++) {
                const int rloc = run * 8 + (lane >> 2);
                const int rowidx = half * 16 + rloc;
                const int j0 = (lane & 3) * 2;
                uint32_t a0[8], out[8];
                lds_v4(stg + (uint32_t)rloc * 128u + (uint32_t)((j0 ^ (rloc & 7)) << 4), a0[0], a0[1], a0[2], a0[3]);
                lds_v4(stg + (uint32_t)rloc * 128u + (uint32_t)(((j0 + 1) ^ (rloc & 7)) << 4), a0[4], a0[5], a0[6], a0[7]);
                if (rowidx < nrows && col < p.N) vm_run_block_row<8, ID>(epi, blk, (uint32_t)rowidx, (uint32_t)col, a0, out);
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
          continue;
        }
      }
      if constexpr (tc_tma_store_epilogue<ID>()) {
        if (p.tma_store) {
          // Thread = row for the arithmetic; the result goes into this warp's 2 KB staging tile (32 rows of 64 bytes,
          // 64-byte swizzle: the 16-byte piece index is XORed with bits 1..2 of the row, which also keeps the 16-byte
          // shared stores of a quarter warp on distinct banks) and from there to global memory with one bulk tensor
          // store per 64-byte-wide column strip.
          constexpr int OES = tc_store_elem_size<ID>();
          constexpr int STRIP = 64 / OES;                   // columns per strip: 32 (16-bit) or 16 (32-bit)
          // short_k: two staging tiles per warp in the ring's unused fourth stage, used alternately
          const uint32_t stg0 = p.short_k ? smem_base + 3u * (uint32_t)SM::STAGE_BYTES + (uint32_t)(warp - 2) * 2048u
                                          : smem_base + SM::STAGING_OFFSET + (uint32_t)(warp - 2) * 2048u;
          const uint32_t stg1 = p.short_k ? smem_base + SM::STAGING_OFFSET + (uint32_t)(warp - 2) * 2048u : stg0;
          const uint32_t sw = (uint32_t)((lane >> 1) & 3);
          VmRow vrow;
          vm_row_begin(epi, rplan, (uint64_t)((int64_t)b * p.M + (row_ok ? row : 0)), (uint32_t)p.N, vrow);
          const bool row_vec = __all_sync(0xffffffffu, vrow.vec);
          if (row_vec) {
#pragma unroll 1
            for (int c = part; c < BN / 32; c += col_parts) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 32), r);
              tc_wait_ld();
#pragma unroll
              for (int strip = 0; strip < 32 / STRIP; strip++) {
                // the store that last read this staging tile must be done with it: the previous one, or with two tiles the
                // one before that
                const uint32_t stg = stg_sel ? stg1 : stg0;
                const uint32_t my = stg + (uint32_t)lane * 64u;
                if (lane == 0) { if (p.short_k) bulk_wait_read_1(); else bulk_wait_read(); }
                __syncwarp();
#pragma unroll
                for (int v = strip * (STRIP / 8); v < (strip + 1) * (STRIP / 8); v++) {
                  const int col = n0 + c * 32 + v * 8;
                  if (row_ok && col < p.N) {
                    uint32_t a0[8], out[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) a0[j] = r[v * 8 + j];
                    // pieces of this vector inside the 64-byte row: 16-bit -> piece v, 32-bit -> pieces 2 (v & 1), + 1
                    const uint32_t p0 = OES == 2 ? (uint32_t)(v & 3) : (uint32_t)((v & 1) * 2);
                    vm_run_row_stage<ID>(epi, vrow, (uint32_t)col, my + ((p0 ^ sw) << 4), my + (((p0 + 1) ^ sw) << 4), a0, out);
                  }
                }
                fence_async_shared();
                __syncwarp();
                const bool do_store = n0 + c * 32 + strip * STRIP < p.N && m0 + quad * 32 < p.M;   // the same for the whole warp
                if (lane == 0 && do_store) {
                  tma_store_3d(&tmOut, stg, n0 + c * 32 + strip * STRIP, m0 + quad * 32, b);
                  bulk_commit();
                }
                if (do_store && p.short_k) stg_sel ^= 1u;   // issued stores alternate between the two tiles
              }
            }
            // the last strip's store is still reading the staging tile: the next tile waits for it before its first
            // strip, the kernel's exit waits for all of them
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            continue;
          }
        }
      }
      // Thread = row.
      VmRow vrow;
      vm_row_begin(epi, rplan, (uint64_t)((int64_t)b * p.M + (row_ok ? row : 0)), (uint32_t)p.N, vrow);
      // one decision per warp: tcgen05.ld below is warp-collective, so all lanes must take the same loop
      const bool row_vec = __all_sync(0xffffffffu, vrow.vec);
      auto chunks = [&](auto vec_tag) {
        constexpr bool VEC = decltype(vec_tag)::value;
        if constexpr (ID != 0) {
          // specialised epilogue: straight-line code, four 8-wide vectors per 32-column TMEM load
#pragma unroll 1
          for (int c = part; c < BN / 32; c += col_parts) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 32), r);
            tc_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int v = 0; v < 4; v++) {
                const int col = n0 + c * 32 + v * 8;
                if (col < p.N) {
                  uint32_t a0[8], out[8];
#pragma unroll
                  for (int j = 0; j < 8; j++) a0[j] = r[v * 8 + j];
                  if constexpr (VEC) vm_run_row_vec<8, ID>(epi, vrow, (uint32_t)col, a0, out);
                  else vm_run_row<8, ID>(epi, vrow, (uint32_t)col, a0, out);
                }
              }
            }
          }
        } else {
          // interpreted epilogue: one inlined copy of the interpreter, fed 8 columns at a time
#pragma unroll 1
          for (int c = part; c < BN / 8; c += col_parts) {
            uint32_t a0[8], out[8];
            tmem_ld_32x8(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 8), a0);
            tc_wait_ld();
            const int col = n0 + c * 8;
            if (row_ok && col < p.N) vm_run_row<8, 0>(epi, vrow, (uint32_t)col, a0, out);
          }
        }
      };
      if (ID != 0 && row_vec) chunks(std::true_type{}); else chunks(std::false_type{});
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  if constexpr (tc_tma_store_epilogue<ID>()) {
    if (warp >= 2 && lane == 0) bulk_wait_all();   // this thread's result stores are complete before the CTA retires
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) { p.sched[0] = 0; p.sched[1] = 0; __threadfence(); }
  }
}

// Scheduler counters: (next tile, finished CTAs) pairs in device memory, one pair per stream that launches GEMMs.
// A pair returns to zero when its launch retires, so no memset is needed between launches.
constexpr int kSchedSlots = 256;
int32_t* sched_slot(cudaStream_t stream);   // defined in gemm_tc.cu

template <int BN, int STAGES, bool TF32, int ID>
static int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p_in, const B2xVmProgram& epi, int32_t* status, cudaStream_t stream) {
  TcParams p = p_in;
  p.sched = sched_slot(stream);
  if (!p.sched) return (int)cudaErrorLaunchOutOfResources;
  // B2X_DEBUG_WITHHOLD_ARRIVE=1 (tests of the bounded waits): one arrival is left out, the kernel gives up after about a
  // second, reports through `status` and returns by itself
  {
    const char* w = getenv("B2X_DEBUG_WITHHOLD_ARRIVE");
    p.withhold = (w && w[0] == '1') ? 1 : 0;
  }
  using SM = TcSmem<BN, STAGES, TF32, tc_transposed_epilogue<ID>() || tc_tma_store_epilogue<ID>()>;
  CUtensorMap tmOut;
  memset(&tmOut, 0, sizeof(tmOut));
  p.tma_store = 0;
  if constexpr (tc_tma_store_epilogue<ID>()) {
    // the stored tensor must be the dense row-major [batch, M, N] result
    constexpr int T = vm_static_store_tensor<ID>();
    constexpr int OES = tc_store_elem_size<ID>();
    const B2xVmTensor& o = epi.tensors[T];
    bool dense = o.stride[epi.n_dims - 1] == 1;
    int64_t total = 1;
    for (int d = epi.n_dims - 1; d >= 0; d--) { dense = dense && o.stride[d] == total; total *= epi.dim[d]; }
    dense = dense && total == p.batch * p.M * p.N && ((uintptr_t)o.ptr & 15) == 0 && (p.N * OES) % 16 == 0;
    if (dense && encode_3d(&tmOut, OES == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, OES, o.ptr, (uint64_t)p.N, (uint64_t)p.M,
                           (uint64_t)p.batch, (uint64_t)p.N, (uint64_t)(p.M * p.N), 64 / OES, 32, CU_TENSOR_MAP_SWIZZLE_64B))
      p.tma_store = 1;
  }
  auto kern = k_gemm_tc<BN, STAGES, TF32, ID>;
  {
    // per device: the attribute belongs to the function on the current device
    int dev = 0;
    cudaGetDevice(&dev);
    static std::atomic<bool> configured[64];
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
  }
  int64_t grid = p.num_tiles < kNumSms ? p.num_tiles : kNumSms;
  kern<<<(unsigned)grid, TC_THREADS, SM::TOTAL, stream>>>(tmA, tmB, tmOut, p, epi, status);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace b2x

namespace b2x {
// Launches a build-time specialised epilogue when one exists for (program id, tile width); returns -1 otherwise.
int launch_tc_static(int id, int BN, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, const B2xVmProgram& epi, int32_t* status,
                     cudaStream_t stream);
// Same for f32 operands (3xTF32); only the plain f32 store is specialised there.
int launch_tc_static_tf32(int id, int BN, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, const B2xVmProgram& epi, int32_t* status,
                          cudaStream_t stream);
// Whether a specialised kernel exists for (program id, tile width), and how many stores that program has.
bool tc_static_has(int id, int BN);
bool tc_static_has_tf32(int id, int BN);
int tc_static_stores(int id);
}  // namespace b2x
