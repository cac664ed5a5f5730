// Entry points of the tcgen05 GEMM (kernel: gemm_tc.cuh) and the f32 hi/lo split used by the 3xTF32 scheme.
#include "gemm_tc.cuh"

#include <atomic>
#include <map>
#include <mutex>

namespace b2x {

static __device__ int32_t g_sched[kSchedSlots * 2];

// Scheduler pair for launches on `stream` of the current device.  Launches on one stream run in order, and a pair is
// back at zero when its launch retires, so every stream can keep one pair for good; launches that may overlap (different
// streams) never share a tile counter.  Only the address of the array is taken here; device code reads and resets it.
// Returns nullptr when more than kSchedSlots different streams have launched GEMMs on this device.
int32_t* sched_slot(cudaStream_t stream) {
  static std::mutex mu;
  static int32_t* base[64] = {};
  static std::map<cudaStream_t, int> slot_of[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!base[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sched) != cudaSuccess) return nullptr;
    base[dev] = (int32_t*)p;
  }
  auto it = slot_of[dev].find(stream);
  if (it == slot_of[dev].end()) {
    if ((int)slot_of[dev].size() >= kSchedSlots) return nullptr;
    it = slot_of[dev].emplace(stream, (int)slot_of[dev].size()).first;
  }
  return base[dev] + 2 * it->second;
}

// ---- f32 -> hi/lo TF32 split for the 3xTF32 scheme ------------------------------------------------------------------
// out rows are K-major with 3K elements: sel 0 -> [hi | hi | lo], sel 1 -> [hi | lo | hi].  One launch splits both
// operands: a CTA takes 32 x 32 (row, k) tiles of either.  A source that is contiguous along k is read and written
// with lane = k; any other source is read with lane = row and turned through shared memory, so that the writes are
// contiguous along k as well.
struct SplitSide {
  const float* src; float* dst;
  int64_t rows, K, sb, sr, sk;
  int64_t tiles_r, tiles_k, n_tiles;
  int sel;
};
__device__ __forceinline__ void split_write(float* o, int64_t K, int64_t k, float x, int sel) {
  const float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
  const float lo = __uint_as_float(__float_as_uint(x - hi) & 0xffffe000u);
  o[k] = hi;
  o[K + k] = sel == 0 ? hi : lo;
  o[2 * K + k] = sel == 0 ? lo : hi;
}
__global__ void __launch_bounds__(256) k_split_f32(const __grid_constant__ SplitSide A, const __grid_constant__ SplitSide B) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t total = A.n_tiles + B.n_tiles;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const bool second = t >= A.n_tiles;
    const SplitSide& S = second ? B : A;
    int64_t u = second ? t - A.n_tiles : t;
    const int64_t tk = u % S.tiles_k; u /= S.tiles_k;
    const int64_t tr = u % S.tiles_r;
    const int64_t b = u / S.tiles_r;
    const int64_t r0 = tr * 32, k0 = tk * 32;
    const float* src = S.src + b * S.sb;
    float* dst = S.dst + b * S.rows * (3 * S.K);
    if (S.sk == 1) {
      const int64_t k = k0 + tx;
#pragma unroll
      for (int i = ty; i < 32; i += 8) {
        const int64_t r = r0 + i;
        if (r < S.rows && k < S.K) split_write(dst + r * (3 * S.K), S.K, k, __ldg(src + r * S.sr + k), S.sel);
      }
    } else {
      const int64_t r_in = r0 + tx;
#pragma unroll
      for (int i = ty; i < 32; i += 8) {
        const int64_t k = k0 + i;
        tile[i][tx] = (r_in < S.rows && k < S.K) ? __ldg(src + r_in * S.sr + k * S.sk) : 0.0f;
      }
      __syncthreads();
      const int64_t k = k0 + tx;
#pragma unroll
      for (int i = ty; i < 32; i += 8) {
        const int64_t r = r0 + i;
        if (r < S.rows && k < S.K) split_write(dst + r * (3 * S.K), S.K, k, tile[tx][i], S.sel);
      }
      __syncthreads();
    }
  }
}

}  // namespace b2x

extern "C" int b2x_launch_split_f32(const B2xGemmArgs* a, float* a_split, float* b_split, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->elem != EL_F32) return (int)cudaErrorInvalidValue;
  auto side = [&](const void* src, float* dst, int64_t rows, int64_t sb, int64_t sr, int64_t sk, int sel) {
    SplitSide s{};
    s.src = (const float*)src; s.dst = dst; s.rows = rows; s.K = a->K; s.sb = sb; s.sr = sr; s.sk = sk; s.sel = sel;
    s.tiles_r = (rows + 31) / 32; s.tiles_k = (a->K + 31) / 32; s.n_tiles = a->batch * s.tiles_r * s.tiles_k;
    return s;
  };
  const SplitSide A = side(a->a, a_split, a->M, a->a_batch_stride, a->a_row_stride, a->a_k_stride, 0);
  const SplitSide B = side(a->b, b_split, a->N, a->b_batch_stride, a->b_row_stride, a->b_k_stride, 1);
  int64_t grid = A.n_tiles + B.n_tiles;
  if (grid > (int64_t)kNumSms * 8) grid = (int64_t)kNumSms * 8;
  if (grid < 1) return 0;
  k_split_f32<<<(unsigned)grid, 256, 0, stream>>>(A, B);
  count_launch(1);
  return (int)cudaGetLastError();
}

namespace b2x {
// Everything the launcher decides from the problem's shape and the epilogue program, before any device work.
struct TcRoute {
  bool tf32 = false, a_mn = false, b_mn = false;
  int es = 2, BK = 64, CHUNK = 64, BN = 256;
  int64_t a_ld = 0, b_ld = 0;
  int static_id = 0;        // build-time specialised epilogue that will run (0: the interpreter)
  TcParams p{};
};

static int tc_route(const B2xGemmArgs* a, const B2xVmProgram* epilogue, TcRoute* r) {
  if (a->batch <= 0 || a->M <= 0 || a->N <= 0 || a->K <= 0) return (int)cudaErrorInvalidValue;
  r->tf32 = a->elem == EL_F32;
  if (!r->tf32 && a->elem != EL_BF16 && a->elem != EL_F16) return (int)cudaErrorInvalidValue;
  const int es = r->es = r->tf32 ? 4 : 2;
  const int BK = r->BK = 128 / es;
  r->CHUNK = 128 / es;
  const int64_t al = 16 / es;
  r->a_mn = !(a->a_k_stride == 1) && a->a_row_stride == 1;
  r->b_mn = !(a->b_k_stride == 1) && a->b_row_stride == 1;
  if (!r->a_mn && a->a_k_stride != 1) return (int)cudaErrorInvalidValue;
  if (!r->b_mn && a->b_k_stride != 1) return (int)cudaErrorInvalidValue;
  r->a_ld = r->a_mn ? a->a_k_stride : a->a_row_stride;
  r->b_ld = r->b_mn ? a->b_k_stride : a->b_row_stride;
  if (r->a_ld % al || r->b_ld % al || (a->batch > 1 && (a->a_batch_stride % al || a->b_batch_stride % al))) return (int)cudaErrorInvalidValue;
  if (a->N % 8) return (int)cudaErrorInvalidValue;
  // widest tile that the result allows; a problem with fewer tiles than half the SMs takes narrower ones, so that
  // more SMs share the operand traffic (each CTA streams its own A and B tiles)
  int BN = a->N >= 256 ? 256 : (a->N >= 128 ? 128 : 64);
  {
    const int64_t m_tiles = (a->M + TC_BM - 1) / TC_BM;
    while (BN > 64 && m_tiles * ((a->N + BN - 1) / BN) * a->batch < kNumSms / 2) BN /= 2;
  }
  r->BN = BN;
  TcParams& p = r->p;
  p.batch = a->batch; p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_mn_major = r->a_mn; p.b_mn_major = r->b_mn;
  p.num_m_tiles = (int)((a->M + TC_BM - 1) / TC_BM);
  p.num_n_tiles = (int)((a->N + BN - 1) / BN);
  p.num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles * a->batch;
  if (p.num_tiles >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  p.k_blocks = (int)((a->K + BK - 1) / BK);
  p.transposed = a->K <= 8192 ? 1 : 0;
  p.epi_groups = p.k_blocks <= 8 ? 1 : 2;
  // Tall (256 x 256) tiles: long-K 16-bit problems whose tall tiles still fill the last round of the 148 SMs.  Their
  // epilogue is not overlapped, so K must be long enough to make it small; B2X_GEMM_TALL=0 / 1 switches them off / forces
  // them wherever the kernel can run them.
  p.tall = 0;
  // short K: three stages, the fourth holds the second set of staging tiles of the bulk-store epilogue (gemm_tc.cuh)
  p.short_k = (BN == 256 && !r->tf32 && p.k_blocks <= 3) ? 1 : 0;
  { static const int sk = [] { const char* e = getenv("B2X_GEMM_SHORT_K"); return e ? atoi(e) : -1; }(); if (sk == 0) p.short_k = 0; }
  int64_t bm = TC_BM;
  if (!r->tf32 && BN == 256 && a->M >= 2 * TC_BM) {
    static const int mode = [] { const char* e = getenv("B2X_GEMM_TALL"); return e ? atoi(e) : -1; }();
    // how full the rounds of the 148 SMs are with either tile height; tall tiles were measured 20-25 % faster per FLOP
    // (MLP step, K = 4096 ... 16384), so they are taken unless their last round wastes more than that
    const int64_t tall_tiles = ((a->M + 2 * TC_BM - 1) / (2 * TC_BM)) * p.num_n_tiles * a->batch;
    auto fill = [](int64_t tiles) { const int64_t rounds = (tiles + kNumSms - 1) / kNumSms; return (double)tiles / (double)(rounds * kNumSms); };
    const bool pays = fill(tall_tiles) * 1.2 > fill(p.num_tiles);
    if (mode == 1 || (mode != 0 && p.k_blocks >= 32 && pays)) {
      p.tall = 1;
      p.epi_groups = 2;
      p.transposed = 1;   // the epilogue of a tall tile is not hidden behind the next tile, so the form with fewer store cycles wins at every K
      bm = 2 * TC_BM;
      p.num_m_tiles = (int)((a->M + bm - 1) / bm);
      p.num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles * a->batch;
    }
  }
  {
    // A slab of a group ~ 32 MiB (a quarter of the 126 MB L2)
    const int64_t slab_per_m_tile = bm * a->K * es;
    int64_t gm = (32ll << 20) / (slab_per_m_tile > 0 ? slab_per_m_tile : 1);
    if (gm < 4) gm = 4;
    if (gm > 64) gm = 64;
    if (gm > p.num_m_tiles) gm = p.num_m_tiles;
    p.group_m = (int)gm;
  }
  p.idesc = sm100::make_idesc(r->tf32 ? 2u : (a->elem == EL_BF16 ? 1u : 0u), r->a_mn, r->b_mn, TC_BM, (uint32_t)BN);
  const int id = vm_static_enabled() ? vm_static_lookup(vm_signature_hash(*epilogue)) : 0;
  r->static_id = (id && (r->tf32 ? tc_static_has_tf32(id, BN) : tc_static_has(id, BN))) ? id : 0;
  return 0;
}
}  // namespace b2x

extern "C" int b2x_gemm_tc_route(const B2xGemmArgs* a, const B2xVmProgram* epilogue, int32_t out[12]) {
  using namespace b2x;
  TcRoute r;
  int rc = tc_route(a, epilogue, &r);
  if (rc) return rc;
  out[0] = r.BN; out[1] = r.static_id; out[2] = r.p.epi_groups;
  out[3] = (r.static_id && r.p.transposed && tc_static_stores(r.static_id) >= 2) ? 1 : 0;
  out[4] = r.p.group_m; out[5] = r.p.num_m_tiles; out[6] = r.p.num_n_tiles; out[7] = r.p.k_blocks;
  out[8] = r.static_id ? tc_static_stores(r.static_id) : 0;
  out[9] = (int32_t)(r.p.num_tiles < kNumSms ? r.p.num_tiles : kNumSms);
  out[10] = r.p.tall ? 2 * TC_BM : TC_BM;
  out[11] = 0;
  return 0;
}

extern "C" int b2x_launch_gemm_tc(const B2xGemmArgs* a, const B2xVmProgram* epilogue, int32_t* status, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  TcRoute r;
  int rc = tc_route(a, epilogue, &r);
  if (rc) return rc;
  if (((uintptr_t)a->a & 15) || ((uintptr_t)a->b & 15)) return (int)cudaErrorInvalidValue;
  const bool tf32 = r.tf32, a_mn = r.a_mn, b_mn = r.b_mn;
  const int es = r.es, BK = r.BK, CHUNK = r.CHUNK, BN = r.BN;
  const int64_t a_ld = r.a_ld, b_ld = r.b_ld;
  CUtensorMapDataType dt = tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (a->elem == EL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUtensorMap tmA, tmB;
  bool ok;
  TcParams p = r.p;
  // B2X_GEMM_LOADS=3d keeps one load per 128-byte-wide sub-tile of an MN-major operand (for comparison)
  static const bool folded = [] { const char* e = getenv("B2X_GEMM_LOADS"); return !(e && e[0] == '3'); }();
  p.a_mn_4d = p.b_mn_4d = 0;
  const uint32_t bm = p.tall ? 2 * TC_BM : TC_BM;   // rows of A per stage
  if (!a_mn) ok = encode_3d(&tmA, dt, es, a->a, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->batch, (uint64_t)a_ld, (uint64_t)a->a_batch_stride, BK, bm);
  else {
    ok = folded && encode_mn_major_4d(&tmA, dt, es, a->a, (uint64_t)a->M, (uint64_t)a->K, (uint64_t)a->batch, (uint64_t)a_ld, (uint64_t)a->a_batch_stride, CHUNK, BK, bm);
    if (ok) p.a_mn_4d = 1;
    else ok = encode_3d(&tmA, dt, es, a->a, (uint64_t)a->M, (uint64_t)a->K, (uint64_t)a->batch, (uint64_t)a_ld, (uint64_t)a->a_batch_stride, CHUNK, BK);
  }
  if (!ok) return (int)cudaErrorInvalidValue;
  if (!b_mn) ok = encode_3d(&tmB, dt, es, a->b, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->batch, (uint64_t)b_ld, (uint64_t)a->b_batch_stride, BK, BN);
  else {
    ok = folded && encode_mn_major_4d(&tmB, dt, es, a->b, (uint64_t)a->N, (uint64_t)a->K, (uint64_t)a->batch, (uint64_t)b_ld, (uint64_t)a->b_batch_stride, CHUNK, BK, BN);
    if (ok) p.b_mn_4d = 1;
    else ok = encode_3d(&tmB, dt, es, a->b, (uint64_t)a->N, (uint64_t)a->K, (uint64_t)a->batch, (uint64_t)b_ld, (uint64_t)a->b_batch_stride, CHUNK, BK);
  }
  if (!ok) return (int)cudaErrorInvalidValue;
  if (tf32) {
    if (r.static_id) {
      rc = launch_tc_static_tf32(r.static_id, BN, tmA, tmB, p, *epilogue, status, stream);
      if (rc >= 0) return rc;
    }
    if (BN == 256) return launch_tc<256, 4, true, 0>(tmA, tmB, p, *epilogue, status, stream);
    if (BN == 128) return launch_tc<128, 6, true, 0>(tmA, tmB, p, *epilogue, status, stream);
    return launch_tc<64, 8, true, 0>(tmA, tmB, p, *epilogue, status, stream);
  }
  if (r.static_id) {
    rc = launch_tc_static(r.static_id, BN, tmA, tmB, p, *epilogue, status, stream);
    if (rc >= 0) return rc;
  }
  if (BN == 256) return launch_tc<256, 4, false, 0>(tmA, tmB, p, *epilogue, status, stream);
  if (BN == 128) return launch_tc<128, 6, false, 0>(tmA, tmB, p, *epilogue, status, stream);
  return launch_tc<64, 8, false, 0>(tmA, tmB, p, *epilogue, status, stream);
}
