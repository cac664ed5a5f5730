// stablehlo.reduce kernels: the input is viewed as [A, R, B] and reduced over R, with the producing elementwise
// chain evaluated on the fly (vm.cuh) so that the reduced tensor is read from HBM exactly once.
//
//   B == 1 (row reduction): a group of T threads (a warp or a whole CTA) owns one (row, split) piece, walks it with
//     128-bit vector loads, folds lanes in registers, then warp shuffles and one shared-memory step.
//   B  > 1 (column reduction): threads are laid out [ry][bx]; each owns V adjacent columns and strides over R, so a
//     warp reads one contiguous span per row; the ry partials meet in shared memory.
// Long reductions with few outputs are cut into S splits whose partials land in scratch.  A row reduction folds them in
// the same launch: every CTA takes a ticket when its partials are written, and the CTA that draws the last ticket folds
// all of them, in index order, so the result does not depend on which CTA that is.  A column reduction folds them with
// a second launch.  The final value of each output can be handed to a fused consumer program (its VM_SRC_ACC0), which
// then does the stores.  HBM-bound: algorithmic bytes = one read of every operand of the prologue.
#include <cstdio>
#include <map>
#include <mutex>

#include "../../../include/b2x_kernels.h"
#include "common.cuh"
#include "vm.cuh"

namespace b2x {

__device__ __forceinline__ uint32_t red_combine(uint32_t a, uint32_t b, int monoid, int cls) {
  switch (monoid) {
    case 0: return cls == VM_F32 ? f2u(u2f(a) + u2f(b)) : a + b;
    case 1: return cls == VM_F32 ? f2u(u2f(a) * u2f(b)) : a * b;
    case 2: return cls == VM_F32 ? f2u(vm_fmax(u2f(a), u2f(b))) : (cls == VM_S32 ? (uint32_t)max((int)a, (int)b) : max(a, b));
    case 3: return cls == VM_F32 ? f2u(vm_fmin(u2f(a), u2f(b))) : (cls == VM_S32 ? (uint32_t)min((int)a, (int)b) : min(a, b));
    case 4: return a & b;
    case 5: return a | b;
    default: return a ^ b;
  }
}
__host__ __device__ inline uint32_t red_identity(int monoid, int cls) {
  switch (monoid) {
    case 0: case 5: case 6: return 0u;
    case 1: return cls == VM_F32 ? 0x3f800000u : 1u;
    case 2: return cls == VM_F32 ? 0xff800000u : (cls == VM_S32 ? 0x80000000u : 0u);
    case 3: return cls == VM_F32 ? 0x7f800000u : (cls == VM_S32 ? 0x7fffffffu : 0xffffffffu);
    default: return 0xffffffffu;
  }
}

// MC selects a combine whose monoid and value class are known at compile time (the two that dominate: f32 sum and f32
// max); 0 = decided at run time.
template <int MC>
__device__ __forceinline__ uint32_t red_combine_t(uint32_t a, uint32_t b, int monoid, int cls) {
  if constexpr (MC == 1) return f2u(u2f(a) + u2f(b));
  else if constexpr (MC == 2) return f2u(vm_fmax(u2f(a), u2f(b)));
  else return red_combine(a, b, monoid, cls);
}
inline int red_combine_class(int monoid, int cls) { return cls == VM_F32 ? (monoid == 0 ? 1 : (monoid == 2 ? 2 : 0)) : 0; }

struct ReduceKArgs {
  int64_t A, R, B;
  int64_t chunk;       // elements of R per split (multiple of the vector width for row reductions)
  int32_t S;
  int32_t monoid, cls;
  int32_t out_elem, init_elem;
  uint32_t init_imm;
  const void* init_ptr;
  void* out;           // final output (S == 1) or partials (S > 1, raw 32-bit)
  // single-launch split reduction: partials go to `out`, the last CTA folds them into `final_out`
  void* final_out;
  int32_t* ticket;     // CTAs that have written their partials; the last one resets it
  int32_t has_post;    // the final value goes to the consumer program Q instead of (or besides) `final_out`
  // The consumer program digested on the host when it is `load acc0; <up to four of mul/add/sub/div by an immediate>;
  // store T0` in f32 (the mean of a loss, a scaled norm): post_n >= 0, and the kernel applies it inline instead of
  // starting the interpreter for one value (2.4 us on the one thread the whole launch waits for).
  int32_t post_n;
  uint8_t post_op[4];
  uint32_t post_imm[4];
  float* post_dst;
  int64_t post_stride;
};

// Hands one finished output to the fused consumer program: element `index` of the result, value in ACC0.
static __device__ __noinline__ void red_post(const B2xVmProgram& Q, int64_t index, uint32_t v) {
  uint32_t a0[1] = {v}, out[1];
  vm_run<1, 0>(Q, (uint64_t)index, a0, out);
}

// Combines a reduced value with the init operand, rounds it to the result element type and stores it (or passes it on).
__device__ __forceinline__ void red_finish(const ReduceKArgs& K, const B2xVmProgram& Q, void* dst, int64_t index, uint32_t v) {
  uint32_t init = K.init_imm;
  if (K.init_ptr) {
    uint32_t raw;
    const int es = vm_elem_size((uint8_t)K.init_elem);
    if (es == 4) raw = *(const uint32_t*)K.init_ptr; else if (es == 2) raw = *(const uint16_t*)K.init_ptr; else raw = *(const uint8_t*)K.init_ptr;
    init = vm_decode(raw, (uint8_t)K.init_elem);
  }
  v = red_combine(init, v, K.monoid, K.cls);
  uint32_t enc = vm_encode(v, (uint8_t)K.out_elem);
  if (K.has_post) {
    const uint32_t dv = vm_decode(enc, (uint8_t)K.out_elem);
    if (K.post_n < 0) { red_post(Q, index, dv); return; }
    float f = u2f(dv);
    for (int i = 0; i < K.post_n; i++) {
      const float y = u2f(K.post_imm[i]);
      switch (K.post_op[i]) {
        case VM_MUL: f = __fmul_rn(f, y); break;
        case VM_ADD: f = __fadd_rn(f, y); break;
        case VM_SUB: f = __fsub_rn(f, y); break;
        default: f = __fdiv_rn(f, y); break;
      }
    }
    K.post_dst[index * K.post_stride] = f;
    return;
  }
  const int es = vm_elem_size((uint8_t)K.out_elem);
  if (es == 4) ((uint32_t*)dst)[index] = enc; else if (es == 2) ((uint16_t*)dst)[index] = (uint16_t)enc; else ((uint8_t*)dst)[index] = (uint8_t)enc;
}

__device__ __forceinline__ void red_write(const ReduceKArgs& K, const B2xVmProgram& Q, int64_t index, uint32_t v) {
  if (K.S > 1) { ((uint32_t*)K.out)[index] = v; return; }
  red_finish(K, Q, K.out, index, v);
}

// Tail of a split row reduction: this CTA's partials are in memory; it takes a ticket, and whoever draws the last one
// folds all partials (in index order, so the result does not depend on which CTA that is) and finishes the outputs.
__device__ __forceinline__ void red_fold_by_last_cta(const ReduceKArgs& K, const B2xVmProgram& Q, uint32_t* smem, int* s_last, uint32_t ident) {
  if (!(K.S > 1 && K.ticket != nullptr)) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) *s_last = (atomicAdd(K.ticket, 1) == (int)gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  const uint32_t* parts = (const uint32_t*)K.out;
  for (int64_t a = 0; a < K.A; a++) {
    uint32_t v = ident;
    // four loads in flight per thread: the fold is one round trip to L2 for up to 1024 partials, and the order in which
    // a thread combines its partials stays fixed
    for (int64_t i0 = threadIdx.x; i0 < K.S; i0 += 1024) {
      uint32_t x[4];
#pragma unroll
      for (int u = 0; u < 4; u++) x[u] = i0 + u * 256 < K.S ? __ldcg(parts + a * K.S + i0 + u * 256) : ident;
#pragma unroll
      for (int u = 0; u < 4; u++) v = red_combine(v, x[u], K.monoid, K.cls);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = red_combine(v, __shfl_xor_sync(0xffffffffu, v, off), K.monoid, K.cls);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t t = smem[0];
#pragma unroll
      for (int w = 1; w < 8; w++) t = red_combine(t, smem[w], K.monoid, K.cls);
      red_finish(K, Q, K.final_out, a, t);
    }
  }
  if (threadIdx.x == 0) { *K.ticket = 0; __threadfence(); }
}

// The same tail for the direct kernels (f32 sum or maximum, partials written by thread 0 only): the combine is fixed at
// compile time, only the writer fences before it takes the ticket, and a plain f32 result without an init tensor or an
// interpreted consumer is finished without the generic encode / decode path.
template <int MC>
__device__ __forceinline__ void red_fold_direct(const ReduceKArgs& K, const B2xVmProgram& Q, uint32_t* smem, int* s_last, uint32_t ident) {
  if (!(K.S > 1 && K.ticket != nullptr)) return;
  if (threadIdx.x == 0) {
    __threadfence();                      // release: this CTA's partials before its ticket
    const bool last = atomicAdd(K.ticket, 1) == (int)gridDim.x - 1;
    if (last) __threadfence();            // acquire: every other CTA's partials after their tickets
    *s_last = last ? 1 : 0;
  }
  __syncthreads();
  if (!*s_last) return;
  // the partials are read through L2 (ld.cg); the barrier above orders these reads behind thread 0's fence
  const uint32_t* parts = (const uint32_t*)K.out;
  for (int64_t a = 0; a < K.A; a++) {
    uint32_t v = ident;
    for (int64_t i0 = threadIdx.x; i0 < K.S; i0 += 1024) {
      uint32_t x[4];
#pragma unroll
      for (int u = 0; u < 4; u++) x[u] = i0 + u * 256 < K.S ? __ldcg(parts + a * K.S + i0 + u * 256) : ident;
#pragma unroll
      for (int u = 0; u < 4; u++) v = red_combine_t<MC>(v, x[u], K.monoid, K.cls);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = red_combine_t<MC>(v, __shfl_xor_sync(0xffffffffu, v, off), K.monoid, K.cls);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t t = smem[0];
#pragma unroll
      for (int w = 1; w < 8; w++) t = red_combine_t<MC>(t, smem[w], K.monoid, K.cls);
      if (K.init_ptr == nullptr && K.out_elem == EL_F32 && K.init_elem == EL_F32 && (!K.has_post || K.post_n >= 0)) {
        float f = u2f(red_combine_t<MC>(K.init_imm, t, K.monoid, K.cls));
        if (K.has_post) {
          for (int i = 0; i < K.post_n; i++) {
            const float y = u2f(K.post_imm[i]);
            switch (K.post_op[i]) {
              case VM_MUL: f = __fmul_rn(f, y); break;
              case VM_ADD: f = __fadd_rn(f, y); break;
              case VM_SUB: f = __fsub_rn(f, y); break;
              default: f = __fdiv_rn(f, y); break;
            }
          }
          K.post_dst[a * K.post_stride] = f;
        } else {
          ((float*)K.final_out)[a] = f;
        }
      } else {
        red_finish(K, Q, K.final_out, a, t);
      }
    }
  }
  if (threadIdx.x == 0) { *K.ticket = 0; __threadfence(); }
}

// Row reduction.  T = threads cooperating on one (row, split) piece: 32 or 256.
template <int V, int T, int ID, int MC>
__global__ void __launch_bounds__(256, ID != 0 ? 4 : 1) k_reduce_rows(const __grid_constant__ B2xVmProgram P, const __grid_constant__ ReduceKArgs K,
                                                                       const __grid_constant__ B2xVmProgram Q) {
  __shared__ uint32_t smem[8];
  __shared__ int s_last;
  constexpr int PIECES_PER_CTA = 256 / T;
  const int lane_in_piece = threadIdx.x % T;
  const int64_t n_pieces = K.A * K.S;
  uint32_t zero[V];
#pragma unroll
  for (int j = 0; j < V; j++) zero[j] = 0;
  const uint32_t ident = red_identity(K.monoid, K.cls);
  // the program's dims are [A, R] (or one merged dim): the coordinates of a vector are (a, r) without a division
  const bool rows2 = P.n_dims == 2 && P.dim[1] == K.R;
  // rows of K.R elements addressed through the row-wise driver (usable when R fits its 32-bit column index)
  const bool row_driver = ID != 0 && V == 8 && K.R > 0 && K.R < (1ll << 28);
  VmRowPlan rplan;
  if (row_driver) rplan = vm_row_plan(P, (uint32_t)K.R); else rplan.fast = false;
  for (int64_t piece0 = (int64_t)blockIdx.x * PIECES_PER_CTA; piece0 < n_pieces; piece0 += (int64_t)gridDim.x * PIECES_PER_CTA) {
    const int64_t piece = piece0 + threadIdx.x / T;
    uint32_t total = ident;
    if (piece < n_pieces) {
      // The S pieces of a row interleave: piece s takes the blocks s, s + S, s + 2S, ... of T * V elements, so that at
      // any moment the pieces of a row read neighbouring addresses (the whole grid sweeps the row together, which is what
      // DRAM likes) instead of S streams that are far apart.  With S == 1 this is the plain walk over the row.
      const int64_t a = piece / K.S, s = piece % K.S;
      constexpr int64_t BLOCK = (int64_t)T * V;
      const int64_t STEP = BLOCK * K.S;
      const int64_t r1 = K.R;
      int64_t r = s * BLOCK + (int64_t)lane_in_piece * V;
      if constexpr (ID != 0 && V == 8) {
        // Specialised programs are short, so the address arithmetic decides the instruction count: the row's operand
        // addresses are set up once (vm_row_begin) and a vector then costs one 32-bit multiply-add per tensor.  Four
        // vectors per trip keep all their loads in flight together.
        VmRow vrow;
        vrow.vec = false;
        if (row_driver && rplan.affine) vm_row_begin(P, rplan, (uint64_t)a, (uint32_t)K.R, vrow);
        if (vrow.vec && vm_row_all_contiguous(P, vrow)) {
          // every operand is contiguous along the row: branch-free fetches, all four vectors' loads in flight at once
          uint32_t tot[4] = {ident, ident, ident, ident};
          for (; r + 3 * STEP < r1; r += 4 * STEP) {
            uint32_t acc[4][V];
#pragma unroll
            for (int u = 0; u < 4; u++) vm_run_row_contig<V, ID>(P, vrow, (uint32_t)(r + u * STEP), zero, acc[u]);
#pragma unroll
            for (int j = 0; j < V; j++) {
#pragma unroll
              for (int u = 0; u < 4; u++) tot[u] = red_combine_t<MC>(tot[u], acc[u][j], K.monoid, K.cls);
            }
          }
          total = red_combine_t<MC>(red_combine_t<MC>(tot[0], tot[1], K.monoid, K.cls), red_combine_t<MC>(tot[2], tot[3], K.monoid, K.cls), K.monoid, K.cls);
          for (; r < r1; r += STEP) {
            uint32_t acc[V];
            vm_run_row_contig<V, ID>(P, vrow, (uint32_t)r, zero, acc);
#pragma unroll
            for (int j = 0; j < V; j++) total = red_combine_t<MC>(total, acc[j], K.monoid, K.cls);
          }
        } else if (vrow.vec) {
          uint32_t tot[4] = {ident, ident, ident, ident};
          for (; r + 3 * STEP < r1; r += 4 * STEP) {
            uint32_t acc[4][V];
#pragma unroll
            for (int u = 0; u < 4; u++) vm_run_row_vec<V, ID>(P, vrow, (uint32_t)(r + u * STEP), zero, acc[u]);
#pragma unroll
            for (int j = 0; j < V; j++) {
#pragma unroll
              for (int u = 0; u < 4; u++) tot[u] = red_combine_t<MC>(tot[u], acc[u][j], K.monoid, K.cls);
            }
          }
          total = red_combine_t<MC>(red_combine_t<MC>(tot[0], tot[1], K.monoid, K.cls), red_combine_t<MC>(tot[2], tot[3], K.monoid, K.cls), K.monoid, K.cls);
          for (; r < r1; r += STEP) {
            uint32_t acc[V];
            vm_run_row_vec<V, ID>(P, vrow, (uint32_t)r, zero, acc);
#pragma unroll
            for (int j = 0; j < V; j++) total = red_combine_t<MC>(total, acc[j], K.monoid, K.cls);
          }
        }
      }
      for (; r < r1; r += STEP) {
        uint32_t acc[V];
        vm_run_at<V, ID>(P, (uint64_t)(a * K.R + r), rows2, a, r, zero, acc);
#pragma unroll
        for (int j = 0; j < V; j++) total = red_combine_t<MC>(total, acc[j], K.monoid, K.cls);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) total = red_combine_t<MC>(total, __shfl_xor_sync(0xffffffffu, total, off), K.monoid, K.cls);
    if (T == 32) {
      if (lane_in_piece == 0 && piece < n_pieces) red_write(K, Q, piece, total);
    } else {
      __syncthreads();
      if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = total;
      __syncthreads();
      if (threadIdx.x == 0) {
        uint32_t t = smem[0];
#pragma unroll
        for (int w = 1; w < 8; w++) t = red_combine(t, smem[w], K.monoid, K.cls);
        if (piece < n_pieces) red_write(K, Q, piece, t);
      }
    }
  }
  red_fold_by_last_cta(K, Q, smem, &s_last, ident);
}

// The plainest reductions - sum, sum of squares and maximum of one dense f32 or bf16 tensor, CTA-per-piece - without the
// fused-elementwise machinery: the loop is eight loads and sixteen arithmetic instructions per trip, which is what lets
// a 134 MB reduction run at the memory system's speed rather than at the instruction scheduler's.  Same pieces, same
// tickets and the same fold as k_reduce_rows; ES = bytes per element (4: f32, 2: bf16), SQ = square each element first,
// MC = 1 sum / 2 maximum (NaN-propagating).
template <int ES, bool SQ, int MC>
__global__ void __launch_bounds__(256) k_reduce_rows_direct(const char* __restrict__ base, const __grid_constant__ ReduceKArgs K,
                                                            const __grid_constant__ B2xVmProgram Q) {
  __shared__ uint32_t smem[8];
  __shared__ int s_last;
  const int64_t n_pieces = K.A * K.S;
  const uint32_t ident = red_identity(K.monoid, K.cls);
  auto fold8 = [&](float& t, const uint4& lo, const uint4& hi) {
    float x[8];
    if constexpr (ES == 4) {
      x[0] = u2f(lo.x); x[1] = u2f(lo.y); x[2] = u2f(lo.z); x[3] = u2f(lo.w); x[4] = u2f(hi.x); x[5] = u2f(hi.y); x[6] = u2f(hi.z); x[7] = u2f(hi.w);
    } else {
      x[0] = u2f(lo.x << 16); x[1] = u2f(lo.x & 0xffff0000u); x[2] = u2f(lo.y << 16); x[3] = u2f(lo.y & 0xffff0000u);
      x[4] = u2f(lo.z << 16); x[5] = u2f(lo.z & 0xffff0000u); x[6] = u2f(lo.w << 16); x[7] = u2f(lo.w & 0xffff0000u);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float v = SQ ? x[j] * x[j] : x[j];      // the product is rounded before it is added, as the program says
      if constexpr (MC == 1) t = __fadd_rn(t, v); else t = vm_fmax(t, v);
    }
  };
  for (int64_t piece = blockIdx.x; piece < n_pieces; piece += gridDim.x) {
    const int64_t a = piece / K.S, s = piece % K.S;
    constexpr int64_t BLOCK = 256 * 8;
    const int64_t STEP = BLOCK * K.S;
    const char* row = base + a * K.R * ES;
    int64_t r = s * BLOCK + (int64_t)threadIdx.x * 8;
    // U blocks in flight per thread (with four CTAs per SM, two measured faster than four or one on a 134 MB read)
    constexpr int U = ES == 4 ? 2 : 4;
    float tot[4] = {u2f(ident), u2f(ident), u2f(ident), u2f(ident)};
    for (; r + (U - 1) * STEP < K.R; r += U * STEP) {
      uint4 lo[U], hi[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint4* p = (const uint4*)(row + (r + u * STEP) * ES);
        lo[u] = __ldg(p);
        if constexpr (ES == 4) hi[u] = __ldg(p + 1); else hi[u] = make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; u++) fold8(tot[u], lo[u], hi[u]);
    }
    for (; r < K.R; r += STEP) {
      const uint4* p = (const uint4*)(row + r * ES);
      uint4 lo = __ldg(p), hi = make_uint4(0, 0, 0, 0);
      if constexpr (ES == 4) hi = __ldg(p + 1);
      fold8(tot[0], lo, hi);
    }
    uint32_t total = red_combine_t<MC>(red_combine_t<MC>(f2u(tot[0]), f2u(tot[1]), K.monoid, K.cls), red_combine_t<MC>(f2u(tot[2]), f2u(tot[3]), K.monoid, K.cls),
                                       K.monoid, K.cls);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) total = red_combine_t<MC>(total, __shfl_xor_sync(0xffffffffu, total, off), K.monoid, K.cls);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t t = smem[0];
#pragma unroll
      for (int w = 1; w < 8; w++) t = red_combine_t<MC>(t, smem[w], K.monoid, K.cls);
      red_write(K, Q, piece, t);
    }
  }
  red_fold_direct<MC>(K, Q, smem, &s_last, ident);
}

// Which direct kernel, if any, computes this prologue: 0 none, 1 the tensor itself, 2 its square.  The program must be
// `load T0` or `load T0; save t; mul t` in f32 arithmetic over one dense, 16-byte aligned f32 or bf16 tensor.
static int direct_kind(const B2xVmProgram& P, const ReduceKArgs& K, int vec) {
  if (vec != 8 || P.n_tensors != 1 || K.cls != VM_F32 || K.B != 1) return 0;
  const B2xVmTensor& T = P.tensors[0];
  if (T.elem != EL_F32 && T.elem != EL_BF16) return 0;
  const int es = T.elem == EL_F32 ? 4 : 2;
  const bool dense = (P.n_dims == 1 && T.stride[0] == 1 && P.dim[0] == K.A * K.R) ||
                     (P.n_dims == 2 && P.dim[1] == K.R && T.stride[1] == 1 && T.stride[0] == K.R);
  if (!dense || ((uintptr_t)T.ptr & 15) || (K.A > 1 && (K.R * es) % 16 != 0) || K.R % 8 != 0) return 0;
  auto plain = [](const B2xVmInstr& I) { return I.tc == VM_F32 && I.rnd == VM_RN_NONE; };
  const B2xVmInstr* c = P.code;
  if (!(c[0].op == VM_LOAD && c[0].src_kind == VM_SRC_TENSOR && c[0].src_idx == 0 && plain(c[0]))) return 0;
  if (P.n_instr == 1) return 1;
  if (P.n_instr == 3 && c[1].op == VM_SAVE && c[2].op == VM_MUL && c[2].src_kind == VM_SRC_TEMP && c[2].src_idx == c[1].aux && plain(c[2])) return 2;
  return 0;
}

// Column reduction.  blockDim = (BX, RY) with BX * RY = 256; thread (bx, ry) owns V adjacent columns.
template <int V>
__global__ void __launch_bounds__(256) k_reduce_cols(const __grid_constant__ B2xVmProgram P, const __grid_constant__ ReduceKArgs K, const __grid_constant__ B2xVmProgram Q, int n_bblocks) {
  __shared__ uint32_t smem[256 * V];
  const int BX = blockDim.x, RY = blockDim.y;
  const int64_t n_work = K.A * K.S * (int64_t)n_bblocks;
  uint32_t zero[V];
#pragma unroll
  for (int j = 0; j < V; j++) zero[j] = 0;
  const uint32_t ident = red_identity(K.monoid, K.cls);
  for (int64_t w = blockIdx.x; w < n_work; w += gridDim.x) {
    const int bb = (int)(w % n_bblocks);
    const int64_t as = w / n_bblocks;
    const int64_t a = as / K.S, s = as % K.S;
    const int64_t b0 = ((int64_t)bb * BX + threadIdx.x) * V;
    const int64_t r0 = s * K.chunk, r1 = min(K.R, r0 + K.chunk);
    uint32_t tot[V];
#pragma unroll
    for (int j = 0; j < V; j++) tot[j] = ident;
    if (b0 < K.B) {
      for (int64_t r = r0 + threadIdx.y; r < r1; r += RY) {
        uint32_t acc[V];
        vm_run<V>(P, (uint64_t)((a * K.R + r) * K.B + b0), zero, acc);
#pragma unroll
        for (int j = 0; j < V; j++) tot[j] = red_combine(tot[j], acc[j], K.monoid, K.cls);
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < V; j++) smem[(threadIdx.y * BX + threadIdx.x) * V + j] = tot[j];
    __syncthreads();
    if (threadIdx.y == 0 && b0 < K.B) {
      for (int y = 1; y < RY; y++) {
#pragma unroll
        for (int j = 0; j < V; j++) tot[j] = red_combine(tot[j], smem[(y * BX + threadIdx.x) * V + j], K.monoid, K.cls);
      }
#pragma unroll
      for (int j = 0; j < V; j++) red_write(K, Q, (a * K.S + s) * K.B + b0 + j, tot[j]);
    }
  }
}

static int launch_one(const B2xVmProgram& P, ReduceKArgs K, const B2xVmProgram& Q, int vec, cudaStream_t stream) {
  const int64_t cap = (int64_t)kNumSms * 24;   // at least the split target: one CTA per piece, dealt out by the hardware
  if (K.B == 1) {
    const int64_t pieces = K.A * K.S;
    const int64_t len = (K.chunk < K.R ? K.chunk : K.R);
    const bool warp_rows = (len / vec) <= 64;
    const int per_cta = warp_rows ? 8 : 1;
    int64_t blocks = (pieces + per_cta - 1) / per_cta;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid((unsigned)blocks), block(256);
    {
      const int mc0 = red_combine_class(K.monoid, K.cls);
      const int dk = (!warp_rows && (mc0 == 1 || mc0 == 2) && vm_static_enabled()) ? direct_kind(P, K, vec) : 0;
      if (dk) {
        const char* base = (const char*)P.tensors[0].ptr;
        const bool f32 = P.tensors[0].elem == EL_F32;
#define B2X_DIRECT(ES_, SQ_, MC_) k_reduce_rows_direct<ES_, SQ_, MC_><<<grid, block, 0, stream>>>(base, K, Q)
        if (f32) { if (dk == 2) { if (mc0 == 1) B2X_DIRECT(4, true, 1); else B2X_DIRECT(4, true, 2); } else { if (mc0 == 1) B2X_DIRECT(4, false, 1); else B2X_DIRECT(4, false, 2); } }
        else { if (dk == 2) { if (mc0 == 1) B2X_DIRECT(2, true, 1); else B2X_DIRECT(2, true, 2); } else { if (mc0 == 1) B2X_DIRECT(2, false, 1); else B2X_DIRECT(2, false, 2); } }
#undef B2X_DIRECT
        count_launch();
        return (int)cudaGetLastError();
      }
    }
#define B2X_ROWS_MC(VV, II, MM)                                                           \
    if (warp_rows) k_reduce_rows<VV, 32, II, MM><<<grid, block, 0, stream>>>(P, K, Q);    \
    else k_reduce_rows<VV, 256, II, MM><<<grid, block, 0, stream>>>(P, K, Q);
    // specialised programs also get a combine fixed at compile time for f32 sum / f32 max
#define B2X_ROWS(VV, II)                                                                  \
    if (II != 0 && mc == 1) { B2X_ROWS_MC(VV, II, (II != 0 ? 1 : 0)) }                    \
    else if (II != 0 && mc == 2) { B2X_ROWS_MC(VV, II, (II != 0 ? 2 : 0)) }               \
    else { B2X_ROWS_MC(VV, II, 0) }
    const int mc = red_combine_class(K.monoid, K.cls);
    if (vec == 8) {
      switch (vm_static_enabled() ? vm_static_lookup(vm_signature_hash(P)) : 0) {
#define X(I) case I: B2X_ROWS(8, I) break;
        B2X_VM_STATIC_REDUCE(X)
#undef X
        default: B2X_ROWS(8, 0) break;
      }
    } else if (vec == 4) { B2X_ROWS(4, 0) } else { B2X_ROWS(1, 0) }
#undef B2X_ROWS_MC
#undef B2X_ROWS
  } else {
    int64_t bvecs = (K.B + vec - 1) / vec;
    int bx = 1;
    while (bx < 256 && bx < bvecs) bx <<= 1;
    int ry = 256 / bx;
    int n_bblocks = (int)((bvecs + bx - 1) / bx);
    int64_t blocks = K.A * K.S * (int64_t)n_bblocks;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid((unsigned)blocks), block(bx, ry);
    if (vec == 8) k_reduce_cols<8><<<grid, block, 0, stream>>>(P, K, Q, n_bblocks);
    else if (vec == 4) k_reduce_cols<4><<<grid, block, 0, stream>>>(P, K, Q, n_bblocks);
    else k_reduce_cols<1><<<grid, block, 0, stream>>>(P, K, Q, n_bblocks);
  }
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace b2x

// Ticket counters of the single-launch split reduction: one per stream that launches reductions, in device memory that
// is part of the library image.  A counter is back at zero when its launch retires (the last CTA resets it), and
// launches on one stream run in order, so a stream keeps its counter for good and launches that may overlap never
// share one.
namespace b2x {
constexpr int kTicketSlots = 256;
static __device__ int32_t g_reduce_tickets[kTicketSlots];
static int32_t* ticket_slot(cudaStream_t stream) {
  static std::mutex mu;
  static int32_t* base[64] = {};
  static std::map<cudaStream_t, int> slot_of[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!base[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_reduce_tickets) != cudaSuccess) return nullptr;
    base[dev] = (int32_t*)p;
  }
  auto it = slot_of[dev].find(stream);
  if (it == slot_of[dev].end()) {
    if ((int)slot_of[dev].size() >= kTicketSlots) return nullptr;
    it = slot_of[dev].emplace(stream, (int)slot_of[dev].size()).first;
  }
  return base[dev] + it->second;
}
}  // namespace b2x

extern "C" int b2x_reduce_splits(int64_t A, int64_t R, int64_t B) {
  // Enough independent pieces to fill 148 SMs in one wave of four resident CTAs per SM (the specialised row kernels are
  // built for at most 64 registers), each piece long enough to keep several vectors per thread in flight for several
  // trips.
  int64_t outputs = A * ((B + 255) / 256 > 1 ? (B + 255) / 256 : 1);
  if (outputs <= 0 || outputs >= 296 || R < 4096) return 1;   // an empty result has nothing to split
  int64_t s = (592 + outputs - 1) / outputs;
  if (s > R / 2048) s = R / 2048;
  if (s > 4096) s = 4096;
  return (int)(s < 1 ? 1 : s);
}

extern "C" int b2x_reduce_launches(int64_t A, int64_t R, int64_t B) {
  if (A <= 0 || B <= 0) return 0;
  return (b2x_reduce_splits(A, R, B) > 1 && R > 0 && B != 1) ? 2 : 1;
}

extern "C" int b2x_launch_reduce(const B2xVmProgram* prologue, const B2xReduceArgs* a, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->A <= 0 || a->B <= 0) return 0;
  const int vec = a->vec;
  if (vec != 1 && vec != 4 && vec != 8) return (int)cudaErrorInvalidValue;
  const int S = b2x_reduce_splits(a->A, a->R, a->B);
  ReduceKArgs K{};
  K.A = a->A; K.R = a->R; K.B = a->B;
  K.monoid = a->monoid; K.cls = a->cls;
  K.out_elem = a->out_elem; K.init_elem = a->init_elem;
  K.init_imm = a->init_imm; K.init_ptr = a->init_ptr;
  K.has_post = a->host_post != nullptr ? 1 : 0;
  K.post_n = -1;
  if (a->host_post && a->cls == VM_F32 && a->out_elem == EL_F32) {
    const B2xVmProgram& q = *a->host_post;
    const int n = q.n_instr;
    bool simple = n >= 2 && n <= 6 && q.n_tensors == 1 && q.n_dims == 1 && q.tensors[0].elem == EL_F32 && q.code[0].op == VM_LOAD &&
                  q.code[0].src_kind == VM_SRC_ACC0 && q.code[n - 1].op == VM_STORE && q.code[n - 1].src_kind == VM_SRC_TENSOR &&
                  q.code[n - 1].src_idx == 0 && q.code[n - 1].rnd == VM_RN_NONE;
    for (int i = 1; simple && i < n - 1; i++) {
      const B2xVmInstr& I = q.code[i];
      simple = (I.op == VM_MUL || I.op == VM_ADD || I.op == VM_SUB || I.op == VM_DIV) && I.src_kind == VM_SRC_IMM && I.tc == VM_F32 && I.rnd == VM_RN_NONE;
    }
    if (simple) {
      K.post_n = n - 2;
      for (int i = 1; i < n - 1; i++) { K.post_op[i - 1] = q.code[i].op; K.post_imm[i - 1] = q.code[i].imm; }
      K.post_dst = (float*)q.tensors[0].ptr;
      K.post_stride = q.tensors[0].stride[0];
    }
  }
  static const B2xVmProgram kNoPost{};
  const B2xVmProgram& Q = a->host_post ? *a->host_post : kNoPost;
  if (S <= 1 || a->R == 0) {
    K.S = 1; K.chunk = a->R > 0 ? a->R : 1; K.out = a->out;
    return launch_one(*prologue, K, Q, vec, stream);
  }
  if (!a->scratch) return (int)cudaErrorInvalidValue;
  int64_t chunk = (a->R + S - 1) / S;
  chunk = (chunk + vec - 1) / vec * vec;
  K.S = S; K.chunk = chunk; K.out = a->scratch;
  if (a->B == 1) {
    // row reduction: the launch folds its own partials (see k_reduce_rows)
    K.final_out = a->out;
    K.ticket = ticket_slot(stream);
    if (!K.ticket) return (int)cudaErrorLaunchOutOfResources;
    return launch_one(*prologue, K, Q, vec, stream);
  }
  ReduceKArgs K1 = K;
  K1.has_post = 0;
  int rc = launch_one(*prologue, K1, kNoPost, vec, stream);
  if (rc) return rc;
  // fold the [A, S, B] partials
  B2xVmProgram F{};
  F.n_instr = 1; F.n_tensors = 1; F.n_dims = 1;
  F.dim[0] = a->A * S * a->B;
  F.tensors[0].ptr = a->scratch;
  F.tensors[0].stride[0] = 1;
  F.tensors[0].elem = a->cls == VM_F32 ? EL_F32 : (a->cls == VM_S32 ? EL_S32 : EL_U32);
  F.code[0].op = VM_LOAD; F.code[0].src_kind = VM_SRC_TENSOR; F.code[0].src_idx = 0; F.code[0].tc = a->cls;
  ReduceKArgs K2 = K;
  K2.R = S; K2.S = 1; K2.chunk = S; K2.out = a->out;
  int v2 = (a->B % 8 == 0) ? 8 : (a->B % 4 == 0 ? 4 : 1);
  return launch_one(F, K2, Q, v2, stream);
}

// ---- reduction entry point that allocates nothing ---------------------------------------------------------------------
// Some callers of this library run where device memory cannot be requested: inside a framework that owns the whole
// allocator and forbids foreign cudaMalloc calls, in a latency-critical serving loop where an allocation would stall
// the device, or after the process has handed all free memory to a pool.  A long reduction with few outputs needs a
// small buffer for its partial results; here that buffer is a fixed array inside the library image, so such callers
// can still reduce.  The price is a size limit and no concurrency between calls (see include/b2x_kernels.h).
namespace b2x {
static __device__ __align__(256) uint32_t g_reduce_partials[B2X_REDUCE_NOALLOC_MAX_PARTIALS];
static std::mutex g_partials_mu;
static void* g_partials_addr[64] = {};

// Device address of the partials array for the current device; looked up once per device.  The array's name is only a
// host-side handle, never a device pointer, so the address must come from the runtime.
static int partials_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_partials_mu);
  if (!g_partials_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_reduce_partials);
    if (e != cudaSuccess) return (int)e;
    g_partials_addr[dev] = p;
  }
  *out = g_partials_addr[dev];
  return 0;
}
}  // namespace b2x

extern "C" int b2x_launch_reduce_noalloc(const B2xVmProgram* prologue, const B2xReduceArgs* a, b2x_stream_t stream, char* err, size_t err_cap) {
  using namespace b2x;
  auto fail = [&](int code, const char* fmt, long long x, long long y) {
    if (err && err_cap) snprintf(err, err_cap, fmt, x, y);
    return code;
  };
  if (err && err_cap) err[0] = 0;
  if (a->A <= 0 || a->B <= 0) return 0;   // empty result: nothing to launch
  const int S = b2x_reduce_splits(a->A, a->R, a->B);
  const long long need = S > 1 ? (long long)a->A * S * a->B : 0;
  if (need > B2X_REDUCE_NOALLOC_MAX_PARTIALS)
    return fail((int)cudaErrorInvalidValue, "this reduction needs %lld partial results but the built-in buffer holds %lld; use b2x_launch_reduce with caller scratch",
                need, (long long)B2X_REDUCE_NOALLOC_MAX_PARTIALS);
  void* partials = nullptr;
  int rc = partials_address(&partials);
  if (rc) return fail(rc, "could not resolve the built-in partials buffer on this device (CUDA error %lld)%.0lld", (long long)rc, 0LL);
  B2xReduceArgs b = *a;
  b.scratch = partials;   // every partial is written by the first pass before the second pass reads it: nothing to clear
  return b2x_launch_reduce(prologue, &b, stream);
}
