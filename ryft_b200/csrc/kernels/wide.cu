// StableHLO ops over 64-bit element types (i64, ui64, f64): elementwise, reduce and dot_general
// (crates/ryft-mlir/src/dialects/stable_hlo/operations/arithmetic.rs:190-453, comparison.rs:136-164, casting.rs:123,
// functional.rs:188-219, linear_algebra.rs:561-592; the reference's worked examples of dot_general and all_reduce are
// written with i64 tensors, linear_algebra.rs:671-701 and communication.rs:821-841).
//
// The fused-elementwise machine (vm.h) keeps every value in one 32-bit register, so 64-bit programs take this path
// instead: one launch per op, every operand addressed through per-dimension element strides (0 = broadcast), one thread
// per result element, arithmetic in int64 / uint64 / double.  These kernels are about coverage, not speed: index-heavy
// programs (shapes, offsets, counters) and double-precision reference computations are small.
#include <cstdint>
#include <cuda_fp16.h>

#include "../../../include/b2x_kernels.h"
#include "common.cuh"

namespace b2x {

enum WideClass : int { W_S64 = 0, W_U64 = 1, W_F64 = 2 };

union WideVal {
  int64_t s;
  uint64_t u;
  double f;
};

__device__ __forceinline__ int wide_class(uint8_t elem) {
  switch (elem) {
    case EL_F16: case EL_BF16: case EL_F32: case EL_F64: return W_F64;
    case EL_PRED: case EL_U8: case EL_U16: case EL_U32: case EL_U64: return W_U64;
    default: return W_S64;
  }
}
__host__ __device__ __forceinline__ int wide_elem_size(uint8_t elem) {
  switch (elem) {
    case EL_PRED: case EL_S8: case EL_U8: return 1;
    case EL_S16: case EL_U16: case EL_F16: case EL_BF16: return 2;
    case EL_S32: case EL_U32: case EL_F32: return 4;
    default: return 8;
  }
}
__device__ __forceinline__ float wide_half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return __uint_as_float(sign);
    return (sign ? -1.f : 1.f) * (float)man * 5.9604644775390625e-8f;      // subnormal: man * 2^-24
  }
  if (exp == 31) return __uint_as_float(sign | 0x7f800000u | (man << 13));
  return __uint_as_float(sign | ((exp + 112u) << 23) | (man << 13));
}
// Loads element `off` of a tensor of element type `elem` and widens it to the class of that type.
__device__ __forceinline__ WideVal wide_load(const void* p, uint8_t elem, int64_t off) {
  WideVal v;
  switch (elem) {
    case EL_PRED: v.u = ((const uint8_t*)p)[off] != 0; break;
    case EL_S8: v.s = ((const int8_t*)p)[off]; break;
    case EL_S16: v.s = ((const int16_t*)p)[off]; break;
    case EL_S32: v.s = ((const int32_t*)p)[off]; break;
    case EL_S64: v.s = ((const int64_t*)p)[off]; break;
    case EL_U8: v.u = ((const uint8_t*)p)[off]; break;
    case EL_U16: v.u = ((const uint16_t*)p)[off]; break;
    case EL_U32: v.u = ((const uint32_t*)p)[off]; break;
    case EL_U64: v.u = ((const uint64_t*)p)[off]; break;
    case EL_F16: v.f = (double)wide_half_to_float(((const uint16_t*)p)[off]); break;
    case EL_BF16: v.f = (double)__uint_as_float((uint32_t)((const uint16_t*)p)[off] << 16); break;
    case EL_F32: v.f = (double)((const float*)p)[off]; break;
    default: v.f = ((const double*)p)[off]; break;
  }
  return v;
}
// Converts a value of class `from` to element type `elem` (StableHLO convert: float -> integer truncates toward zero,
// anything -> i1 is "!= 0", float -> narrower float rounds to nearest even) and stores it.
__device__ __forceinline__ void wide_store(void* p, uint8_t elem, int64_t off, WideVal v, int from) {
  const int to = wide_class(elem);
  if (elem == EL_PRED) {
    ((uint8_t*)p)[off] = from == W_F64 ? (v.f != 0.0) : (v.u != 0);
    return;
  }
  if (to == W_F64) {
    const double d = from == W_F64 ? v.f : (from == W_S64 ? (double)v.s : (double)v.u);
    switch (elem) {
      case EL_F64: ((double*)p)[off] = d; break;
      case EL_F32: ((float*)p)[off] = (float)d; break;
      case EL_BF16: {
        // double -> float -> bf16 would round twice; round the double directly: take the float below or equal in
        // magnitude (round toward zero), then decide on the discarded part
        const float f = __double2float_rz(d);
        uint32_t u = __float_as_uint(f);
        if ((u & 0x7f800000u) != 0x7f800000u) {
          const uint32_t lo = u & 0xffffu;
          const bool sticky = (double)f != d;
          u &= 0xffff0000u;
          if (lo > 0x8000u || (lo == 0x8000u && (sticky || (u & 0x10000u)))) u += 0x10000u;
        } else if (u & 0x007fffffu) u |= 0x00400000u;
        ((uint16_t*)p)[off] = (uint16_t)(u >> 16);
        break;
      }
      default: ((uint16_t*)p)[off] = __half_as_ushort(__double2half(d)); break;
    }
    return;
  }
  // integer destinations: wrap to the destination width (two's complement), floats truncate toward zero
  int64_t i;
  if (from == W_F64) i = to == W_U64 ? (int64_t)(uint64_t)__double2ull_rz(v.f) : __double2ll_rz(v.f);
  else i = v.s;
  switch (wide_elem_size(elem)) {
    case 1: ((uint8_t*)p)[off] = (uint8_t)i; break;
    case 2: ((uint16_t*)p)[off] = (uint16_t)i; break;
    case 4: ((uint32_t*)p)[off] = (uint32_t)i; break;
    default: ((uint64_t*)p)[off] = (uint64_t)i; break;
  }
}

__device__ __forceinline__ WideVal wide_binary(int op, int cls, WideVal a, WideVal b) {
  WideVal r;
  r.u = 0;
  if (cls == W_F64) {
    switch (op) {
      case B2X_WIDE_ADD: r.f = a.f + b.f; break;
      case B2X_WIDE_SUB: r.f = a.f - b.f; break;
      case B2X_WIDE_MUL: r.f = a.f * b.f; break;
      case B2X_WIDE_DIV: r.f = a.f / b.f; break;
      case B2X_WIDE_REM: r.f = fmod(a.f, b.f); break;
      case B2X_WIDE_POW: r.f = pow(a.f, b.f); break;
      case B2X_WIDE_MAX: r.f = (a.f != a.f) ? a.f : ((b.f != b.f) ? b.f : fmax(a.f, b.f)); break;
      case B2X_WIDE_MIN: r.f = (a.f != a.f) ? a.f : ((b.f != b.f) ? b.f : fmin(a.f, b.f)); break;
      default: break;
    }
  } else if (cls == W_S64) {
    switch (op) {
      case B2X_WIDE_ADD: r.u = a.u + b.u; break;
      case B2X_WIDE_SUB: r.u = a.u - b.u; break;
      case B2X_WIDE_MUL: r.u = a.u * b.u; break;
      case B2X_WIDE_DIV: r.s = b.s == 0 ? -1 : ((a.s == INT64_MIN && b.s == -1) ? INT64_MIN : a.s / b.s); break;
      case B2X_WIDE_REM: r.s = b.s == 0 ? a.s : ((a.s == INT64_MIN && b.s == -1) ? 0 : a.s % b.s); break;
      case B2X_WIDE_MAX: r.s = a.s > b.s ? a.s : b.s; break;
      case B2X_WIDE_MIN: r.s = a.s < b.s ? a.s : b.s; break;
      case B2X_WIDE_AND: r.u = a.u & b.u; break;
      case B2X_WIDE_OR: r.u = a.u | b.u; break;
      case B2X_WIDE_XOR: r.u = a.u ^ b.u; break;
      case B2X_WIDE_POW: {
        // integer power by squaring; a negative exponent gives 0 except for bases 1 and -1
        if (b.s < 0) { r.s = a.s == 1 ? 1 : (a.s == -1 ? ((b.s & 1) ? -1 : 1) : 0); break; }
        uint64_t base = a.u, acc = 1, e = b.u;
        while (e) { if (e & 1) acc *= base; base *= base; e >>= 1; }
        r.u = acc;
        break;
      }
      default: break;
    }
  } else {
    switch (op) {
      case B2X_WIDE_ADD: r.u = a.u + b.u; break;
      case B2X_WIDE_SUB: r.u = a.u - b.u; break;
      case B2X_WIDE_MUL: r.u = a.u * b.u; break;
      case B2X_WIDE_DIV: r.u = b.u == 0 ? ~0ull : a.u / b.u; break;
      case B2X_WIDE_REM: r.u = b.u == 0 ? a.u : a.u % b.u; break;
      case B2X_WIDE_MAX: r.u = a.u > b.u ? a.u : b.u; break;
      case B2X_WIDE_MIN: r.u = a.u < b.u ? a.u : b.u; break;
      case B2X_WIDE_AND: r.u = a.u & b.u; break;
      case B2X_WIDE_OR: r.u = a.u | b.u; break;
      case B2X_WIDE_XOR: r.u = a.u ^ b.u; break;
      case B2X_WIDE_POW: { uint64_t base = a.u, acc = 1, e = b.u; while (e) { if (e & 1) acc *= base; base *= base; e >>= 1; } r.u = acc; break; }
      default: break;
    }
  }
  return r;
}

__device__ __forceinline__ bool wide_compare(int dir, int cls, WideVal a, WideVal b) {
  switch (dir) {
    case 0: return cls == W_F64 ? a.f == b.f : a.u == b.u;
    case 1: return cls == W_F64 ? a.f != b.f : a.u != b.u;
    case 2: return cls == W_F64 ? a.f >= b.f : (cls == W_S64 ? a.s >= b.s : a.u >= b.u);
    case 3: return cls == W_F64 ? a.f > b.f : (cls == W_S64 ? a.s > b.s : a.u > b.u);
    case 4: return cls == W_F64 ? a.f <= b.f : (cls == W_S64 ? a.s <= b.s : a.u <= b.u);
    default: return cls == W_F64 ? a.f < b.f : (cls == W_S64 ? a.s < b.s : a.u < b.u);
  }
}

__device__ __forceinline__ WideVal wide_unary(int op, int cls, WideVal a) {
  WideVal r;
  r.u = 0;
  if (cls == W_F64) {
    switch (op) {
      case B2X_WIDE_NEG: r.f = -a.f; break;
      case B2X_WIDE_ABS: r.f = fabs(a.f); break;
      case B2X_WIDE_SIGN: r.f = (a.f != a.f) ? a.f : (a.f > 0 ? 1.0 : (a.f < 0 ? -1.0 : a.f)); break;
      case B2X_WIDE_TANH: r.f = tanh(a.f); break;
      case B2X_WIDE_EXP: r.f = exp(a.f); break;
      case B2X_WIDE_LOG: r.f = log(a.f); break;
      case B2X_WIDE_SQRT: r.f = sqrt(a.f); break;
      case B2X_WIDE_RSQRT: r.f = 1.0 / sqrt(a.f); break;
      case B2X_WIDE_LOGISTIC: r.f = 1.0 / (1.0 + exp(-a.f)); break;
      case B2X_WIDE_FLOOR: r.f = floor(a.f); break;
      case B2X_WIDE_CEIL: r.f = ceil(a.f); break;
      case B2X_WIDE_EXPM1: r.f = expm1(a.f); break;
      case B2X_WIDE_LOG1P: r.f = log1p(a.f); break;
      case B2X_WIDE_SIN: r.f = sin(a.f); break;
      case B2X_WIDE_COS: r.f = cos(a.f); break;
      default: r = a; break;
    }
  } else {
    switch (op) {
      case B2X_WIDE_NEG: r.u = 0ull - a.u; break;
      case B2X_WIDE_ABS: r.s = cls == W_S64 ? (a.s < 0 ? -a.s : a.s) : a.s; break;
      case B2X_WIDE_SIGN: r.s = cls == W_S64 ? (a.s > 0) - (a.s < 0) : (a.u != 0); break;
      case B2X_WIDE_NOT: r.u = ~a.u; break;
      default: r = a; break;
    }
  }
  return r;
}

__global__ void __launch_bounds__(256) k_wide_elementwise(const __grid_constant__ B2xWideOp W) {
  const int nd = W.n_dims;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < W.n_elements; i += (int64_t)gridDim.x * 256) {
    int64_t coord[B2X_WIDE_MAX_DIMS];
    int64_t rest = i;
#pragma unroll
    for (int d = B2X_WIDE_MAX_DIMS - 1; d >= 0; d--) {
      coord[d] = 0;
      if (d < nd) { const int64_t n = W.dim[d]; coord[d] = rest % n; rest /= n; }
    }
    WideVal in[3];
    int cls_in[3] = {W_S64, W_S64, W_S64};
#pragma unroll
    for (int k = 0; k < 3; k++) {
      in[k].u = 0;
      if (k < W.n_in) {
        int64_t off = 0;
#pragma unroll
        for (int d = 0; d < B2X_WIDE_MAX_DIMS; d++) if (d < nd) off += coord[d] * W.in_stride[k][d];
        in[k] = wide_load(W.in[k], W.in_elem[k], off);
        cls_in[k] = wide_class(W.in_elem[k]);
      }
    }
    WideVal r;
    int cls = cls_in[0];
    switch (W.op) {
      case B2X_WIDE_COPY: r = in[0]; break;          // also convert, broadcast_in_dim, transpose: the store converts
      case B2X_WIDE_FILL: r.u = W.imm; cls = wide_class(W.out_elem); break;
      case B2X_WIDE_IOTA: r.s = coord[W.aux]; cls = W_S64; break;
      case B2X_WIDE_COMPARE: {
        int c = cls_in[0];
        if (W.aux2 == 1 && c != W_F64) c = W_U64;     // UNSIGNED comparison of integers
        if (W.aux2 == 2 && c == W_U64 && W.in_elem[0] != EL_PRED) c = W_S64;
        r.u = wide_compare(W.aux, c, in[0], in[1]) ? 1 : 0;
        cls = W_U64;
        break;
      }
      case B2X_WIDE_SELECT: r = in[0].u ? in[1] : in[2]; cls = cls_in[1]; break;
      case B2X_WIDE_CLAMP: {                          // min(max(x, lo), hi): operands (lo, x, hi)
        cls = cls_in[1];
        r = wide_binary(B2X_WIDE_MIN, cls, wide_binary(B2X_WIDE_MAX, cls, in[1], in[0]), in[2]);
        break;
      }
      default:
        if (W.n_in >= 2) r = wide_binary(W.op, cls, in[0], in[1]);
        else r = wide_unary(W.op, cls, in[0]);
        break;
    }
    // results of narrow integer types wrap at their own width, as every op of that type does
    wide_store(W.out, W.out_elem, i, r, cls);
  }
}

// Reduction of the middle extent of a contiguous [A, R, B] tensor; one CTA per result element.
__global__ void __launch_bounds__(256) k_wide_reduce(const void* in, uint8_t elem, int64_t A, int64_t R, int64_t B, int monoid, const void* init_ptr,
                                                     uint64_t init_imm, void* out) {
  __shared__ WideVal sm[256];
  const int cls = wide_class(elem);
  int op;
  switch (monoid) {
    case 0: op = B2X_WIDE_ADD; break; case 1: op = B2X_WIDE_MUL; break; case 2: op = B2X_WIDE_MAX; break; case 3: op = B2X_WIDE_MIN; break;
    case 4: op = B2X_WIDE_AND; break; case 5: op = B2X_WIDE_OR; break; default: op = B2X_WIDE_XOR; break;
  }
  for (int64_t o = blockIdx.x; o < A * B; o += gridDim.x) {
    const int64_t a = o / B, b = o % B;
    WideVal acc;
    bool have = false;
    acc.u = 0;
    for (int64_t r = threadIdx.x; r < R; r += 256) {
      const WideVal v = wide_load(in, elem, (a * R + r) * B + b);
      acc = have ? wide_binary(op, cls, acc, v) : v;
      have = true;
    }
    // tree over the threads that saw at least one element (thread t has one iff t < R)
    sm[threadIdx.x] = acc;
    __syncthreads();
    const int64_t live = R < 256 ? R : 256;
    for (int step = 128; step > 0; step >>= 1) {
      if (threadIdx.x < step && threadIdx.x + step < live) sm[threadIdx.x] = wide_binary(op, cls, sm[threadIdx.x], sm[threadIdx.x + step]);
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      WideVal init;
      if (init_ptr) init = wide_load(init_ptr, elem, 0); else init.u = init_imm;
      const WideVal res = live > 0 ? wide_binary(op, cls, init, sm[0]) : init;
      wide_store(out, elem, o, res, cls);
    }
    __syncthreads();
  }
}

// C[b][m][n] = sum_k A[b][m][k] * B[b][k][n] with element strides; one thread per result element.
__global__ void __launch_bounds__(256) k_wide_gemm(const __grid_constant__ B2xGemmArgs G, uint8_t out_elem, void* out) {
  const int cls = wide_class(G.elem);
  const int64_t total = G.batch * G.M * G.N;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t n = i % G.N, m = (i / G.N) % G.M, b = i / (G.N * G.M);
    WideVal acc;
    acc.u = 0;
    if (cls == W_F64) acc.f = 0.0;
    for (int64_t k = 0; k < G.K; k++) {
      const WideVal x = wide_load(G.a, G.elem, b * G.a_batch_stride + m * G.a_row_stride + k * G.a_k_stride);
      const WideVal y = wide_load(G.b, G.elem, b * G.b_batch_stride + n * G.b_row_stride + k * G.b_k_stride);
      if (cls == W_F64) acc.f = fma(x.f, y.f, acc.f); else acc.u += x.u * y.u;
    }
    wide_store(out, out_elem, i, acc, cls);
  }
}

static unsigned wide_grid(int64_t n) {
  int64_t g = (n + 255) / 256;
  const int64_t cap = (int64_t)kNumSms * 16;
  return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace b2x

extern "C" int b2x_launch_wide_elementwise(const B2xWideOp* op, b2x_stream_t stream) {
  using namespace b2x;
  if (op->n_elements <= 0) return 0;
  if (op->n_dims < 0 || op->n_dims > B2X_WIDE_MAX_DIMS || op->n_in < 0 || op->n_in > 3) return (int)cudaErrorInvalidValue;
  k_wide_elementwise<<<wide_grid(op->n_elements), 256, 0, (cudaStream_t)stream>>>(*op);
  count_launch();
  return (int)cudaGetLastError();
}

extern "C" int b2x_launch_wide_reduce(const void* in, uint8_t elem, int64_t A, int64_t R, int64_t B, int monoid, const void* init_ptr, uint64_t init_imm,
                                      void* out, b2x_stream_t stream) {
  using namespace b2x;
  if (A <= 0 || B <= 0) return 0;
  const int64_t outs = A * B;
  const unsigned grid = (unsigned)(outs > (int64_t)kNumSms * 16 ? (int64_t)kNumSms * 16 : outs);
  k_wide_reduce<<<grid, 256, 0, (cudaStream_t)stream>>>(in, elem, A, R, B, monoid, init_ptr, init_imm, out);
  count_launch();
  return (int)cudaGetLastError();
}

extern "C" int b2x_launch_wide_gemm(const B2xGemmArgs* g, uint8_t out_elem, void* out, b2x_stream_t stream) {
  using namespace b2x;
  if (g->batch <= 0 || g->M <= 0 || g->N <= 0) return 0;
  k_wide_gemm<<<wide_grid(g->batch * g->M * g->N), 256, 0, (cudaStream_t)stream>>>(*g, out_elem, out);
  count_launch();
  return (int)cudaGetLastError();
}
