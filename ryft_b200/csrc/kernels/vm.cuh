// Device-side interpreter for B2xVmProgram (format: vm.h).
//
// Every thread runs the program once for V consecutive elements along the innermost root dimension.  All branches
// of the interpreter depend only on the program, never on data, so warps do not diverge; temporaries are named
// register arrays selected by uniform switches (no dynamically indexed local memory).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "vm.h"

namespace b2x {

__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }

__device__ __forceinline__ uint32_t vm_narrow(uint32_t v, uint8_t rnd) {
  switch (rnd) {
    case VM_RN_BF16: return f2u(__bfloat162float(__float2bfloat16_rn(u2f(v))));
    case VM_RN_F16: return f2u(__half2float(__float2half_rn(u2f(v))));
    case VM_RN_S8: return (uint32_t)(int32_t)(int8_t)(v & 0xff);
    case VM_RN_S16: return (uint32_t)(int32_t)(int16_t)(v & 0xffff);
    case VM_RN_U8: return v & 0xffu;
    case VM_RN_U16: return v & 0xffffu;
    case VM_RN_PRED: return v != 0u ? 1u : 0u;
    default: return v;
  }
}

__device__ __forceinline__ int vm_elem_size(uint8_t e) {
  switch (e) {
    case EL_PRED: case EL_S8: case EL_U8: return 1;
    case EL_S16: case EL_U16: case EL_F16: case EL_BF16: return 2;
    case EL_S64: case EL_U64: case EL_F64: return 8;
    default: return 4;
  }
}

// Reads NB bytes at p into raw (NB in {1,2,4,8,16,32}); p must be NB-aligned up to 16 bytes.
template <int NB>
__device__ __forceinline__ void vm_ld_bytes(const void* p, uint32_t* raw) {
  if constexpr (NB == 32) {
    uint4 a = __ldg((const uint4*)p), b = __ldg((const uint4*)p + 1);
    raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w; raw[4] = b.x; raw[5] = b.y; raw[6] = b.z; raw[7] = b.w;
  } else if constexpr (NB == 16) {
    uint4 a = __ldg((const uint4*)p);
    raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w;
  } else if constexpr (NB == 8) {
    uint2 a = __ldg((const uint2*)p);
    raw[0] = a.x; raw[1] = a.y;
  } else if constexpr (NB == 4) {
    raw[0] = __ldg((const uint32_t*)p);
  } else if constexpr (NB == 2) {
    raw[0] = __ldg((const uint16_t*)p);
  } else {
    raw[0] = __ldg((const uint8_t*)p);
  }
}
template <int NB>
__device__ __forceinline__ void vm_st_bytes(void* p, const uint32_t* raw) {
  if constexpr (NB == 32) {
    *((uint4*)p) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
    *((uint4*)p + 1) = make_uint4(raw[4], raw[5], raw[6], raw[7]);
  } else if constexpr (NB == 16) {
    *((uint4*)p) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
  } else if constexpr (NB == 8) {
    *((uint2*)p) = make_uint2(raw[0], raw[1]);
  } else if constexpr (NB == 4) {
    *((uint32_t*)p) = raw[0];
  } else if constexpr (NB == 2) {
    *((uint16_t*)p) = (uint16_t)raw[0];
  } else {
    *((uint8_t*)p) = (uint8_t)raw[0];
  }
}

__device__ __forceinline__ uint32_t vm_decode(uint32_t bits, uint8_t elem) {
  switch (elem) {
    case EL_BF16: return bits << 16;
    case EL_F16: return f2u(__half2float(__ushort_as_half((unsigned short)bits)));
    case EL_S8: return (uint32_t)(int32_t)(int8_t)bits;
    case EL_S16: return (uint32_t)(int32_t)(int16_t)bits;
    default: return bits;  // 32-bit types, unsigned narrow types, pred
  }
}
__device__ __forceinline__ uint32_t vm_encode(uint32_t v, uint8_t elem) {
  switch (elem) {
    case EL_BF16: return __bfloat16_as_ushort(__float2bfloat16_rn(u2f(v)));
    case EL_F16: return __half_as_ushort(__float2half_rn(u2f(v)));
    case EL_PRED: return v != 0u;
    case EL_S8: case EL_U8: return v & 0xffu;
    case EL_S16: case EL_U16: return v & 0xffffu;
    default: return v;
  }
}

// Fetch V elements of tensor T starting at element offset `off`, consecutive elements `istride` apart.
template <int V>
__device__ __forceinline__ void vm_fetch(const B2xVmTensor& T, int64_t off, int64_t istride, uint32_t (&b)[V]) {
  const int es = vm_elem_size(T.elem);
  const char* base = (const char*)T.ptr + off * es;
  if (istride == 0 || V == 1) {
    uint32_t raw;
    if (es == 4) vm_ld_bytes<4>(base, &raw); else if (es == 2) vm_ld_bytes<2>(base, &raw); else vm_ld_bytes<1>(base, &raw);
    raw = vm_decode(raw, T.elem);
#pragma unroll
    for (int j = 0; j < V; j++) b[j] = raw;
    return;
  }
  if (istride == 1) {
    if (es == 4) {
      if (((uintptr_t)base & (V * 4 >= 16 ? 15 : V * 4 - 1)) == 0) {
        uint32_t raw[V];
        vm_ld_bytes<V * 4>(base, raw);
#pragma unroll
        for (int j = 0; j < V; j++) b[j] = raw[j];
        return;
      }
    } else if (es == 2) {
      if (((uintptr_t)base & (V * 2 - 1)) == 0) {
        uint32_t raw[(V + 1) / 2];
        vm_ld_bytes<V * 2>(base, raw);
#pragma unroll
        for (int j = 0; j < V; j++) b[j] = vm_decode((raw[j / 2] >> ((j & 1) * 16)) & 0xffffu, T.elem);
        return;
      }
    } else if (es == 1) {
      if (((uintptr_t)base & (V - 1)) == 0) {
        uint32_t raw[(V + 3) / 4];
        vm_ld_bytes<V>(base, raw);
#pragma unroll
        for (int j = 0; j < V; j++) b[j] = vm_decode((raw[j / 4] >> ((j & 3) * 8)) & 0xffu, T.elem);
        return;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; j++) {
    uint32_t raw;
    const char* p = base + (int64_t)j * istride * es;
    if (es == 4) vm_ld_bytes<4>(p, &raw); else if (es == 2) vm_ld_bytes<2>(p, &raw); else vm_ld_bytes<1>(p, &raw);
    b[j] = vm_decode(raw, T.elem);
  }
}

template <int V>
__device__ __forceinline__ void vm_put(const B2xVmTensor& T, int64_t off, int64_t istride, const uint32_t (&a)[V]) {
  const int es = vm_elem_size(T.elem);
  char* base = (char*)T.ptr + off * es;
  if (istride == 1 && V > 1) {
    if (es == 4 && ((uintptr_t)base & (V * 4 >= 16 ? 15 : V * 4 - 1)) == 0) {
      uint32_t raw[V];
#pragma unroll
      for (int j = 0; j < V; j++) raw[j] = vm_encode(a[j], T.elem);
      vm_st_bytes<V * 4>(base, raw);
      return;
    }
    if (es == 2 && ((uintptr_t)base & (V * 2 - 1)) == 0) {
      uint32_t raw[(V + 1) / 2];
#pragma unroll
      for (int j = 0; j < (V + 1) / 2; j++) raw[j] = 0;
#pragma unroll
      for (int j = 0; j < V; j++) raw[j / 2] |= vm_encode(a[j], T.elem) << ((j & 1) * 16);
      vm_st_bytes<V * 2>(base, raw);
      return;
    }
    if (es == 1 && ((uintptr_t)base & (V - 1)) == 0) {
      uint32_t raw[(V + 3) / 4];
#pragma unroll
      for (int j = 0; j < (V + 3) / 4; j++) raw[j] = 0;
#pragma unroll
      for (int j = 0; j < V; j++) raw[j / 4] |= vm_encode(a[j], T.elem) << ((j & 3) * 8);
      vm_st_bytes<V>(base, raw);
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < V; j++) {
    uint32_t raw = vm_encode(a[j], T.elem);
    char* p = base + (int64_t)j * istride * es;
    if (es == 4) vm_st_bytes<4>(p, &raw); else if (es == 2) vm_st_bytes<2>(p, &raw); else vm_st_bytes<1>(p, &raw);
  }
}

__device__ __forceinline__ float vm_fmax(float x, float y) { return (x != x) ? x : ((y != y) ? y : fmaxf(x, y)); }
__device__ __forceinline__ float vm_fmin(float x, float y) { return (x != x) ? x : ((y != y) ? y : fminf(x, y)); }
__device__ __forceinline__ int vm_sdiv(int x, int y) { return y == 0 ? -1 : ((x == INT_MIN && y == -1) ? INT_MIN : x / y); }
__device__ __forceinline__ int vm_srem(int x, int y) { return y == 0 ? x : ((x == INT_MIN && y == -1) ? 0 : x % y); }
__device__ __forceinline__ uint32_t vm_udiv(uint32_t x, uint32_t y) { return y == 0 ? 0xffffffffu : x / y; }
__device__ __forceinline__ uint32_t vm_urem(uint32_t x, uint32_t y) { return y == 0 ? x : x % y; }
__device__ __forceinline__ int vm_ipow(int x, int y) {
  if (y < 0) return x == 1 ? 1 : (x == -1 ? ((y & 1) ? -1 : 1) : 0);
  int r = 1;
  while (y) { if (y & 1) r *= x; x *= x; y >>= 1; }
  return r;
}
__device__ __forceinline__ float vm_tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ bool vm_cmp(T x, T y, uint8_t dir) {
  switch (dir) {
    case VM_EQ: return x == y;
    case VM_NE: return x != y;
    case VM_GE: return x >= y;
    case VM_GT: return x > y;
    case VM_LE: return x <= y;
    default: return x < y;
  }
}

#define B2X_VM_TEMP_SWITCH(idx, T, stmt)                 \
  switch (idx) {                                          \
    case 0: { auto& T = t0; stmt; } break;                \
    case 1: { auto& T = t1; stmt; } break;                \
    case 2: { auto& T = t2; stmt; } break;                \
    case 3: { auto& T = t3; stmt; } break;                \
    case 4: { auto& T = t4; stmt; } break;                \
    default: { auto& T = t5; stmt; } break;               \
  }

#define B2X_VM_BIN(EF, ES, EU)                                                                              \
  {                                                                                                         \
    if (I.tc == VM_F32) {                                                                                   \
      _Pragma("unroll") for (int j = 0; j < V; j++) { float x = u2f(X[j]), y = u2f(Y[j]); acc[j] = f2u(EF); } \
    } else if (I.tc == VM_S32) {                                                                            \
      _Pragma("unroll") for (int j = 0; j < V; j++) { int x = (int)X[j], y = (int)Y[j]; acc[j] = (uint32_t)(ES); } \
    } else {                                                                                                \
      _Pragma("unroll") for (int j = 0; j < V; j++) { uint32_t x = X[j], y = Y[j]; acc[j] = (uint32_t)(EU); } \
    }                                                                                                       \
  }

#define B2X_VM_UN(EF, ES)                                                                     \
  {                                                                                           \
    if (I.tc == VM_F32) {                                                                     \
      _Pragma("unroll") for (int j = 0; j < V; j++) { float x = u2f(acc[j]); acc[j] = f2u(EF); } \
    } else {                                                                                  \
      _Pragma("unroll") for (int j = 0; j < V; j++) { int x = (int)acc[j]; acc[j] = (uint32_t)(ES); } \
    }                                                                                         \
  }

// Decomposes the linear index of a vector's first element into coordinates of the merged root dims.
__device__ __forceinline__ void vm_coords(const B2xVmProgram& P, uint64_t lin, int64_t (&coord)[B2X_VM_MAX_DIMS]) {
  const int nd = P.n_dims;
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) coord[d] = 0;
  if (nd <= 1) { coord[0] = (int64_t)lin; return; }
  if (lin <= 0xffffffffull) {
    uint32_t l = (uint32_t)lin;
#pragma unroll
    for (int d = B2X_VM_MAX_DIMS - 1; d >= 1; d--) {
      if (d < nd) { uint32_t n = (uint32_t)P.dim[d]; uint32_t q = l / n; coord[d] = (int64_t)(l - q * n); l = q; }
    }
    coord[0] = (int64_t)l;
  } else {
#pragma unroll
    for (int d = B2X_VM_MAX_DIMS - 1; d >= 1; d--) {
      if (d < nd) { uint64_t n = (uint64_t)P.dim[d]; uint64_t q = lin / n; coord[d] = (int64_t)(lin - q * n); lin = q; }
    }
    coord[0] = (int64_t)lin;
  }
}

// Runs the program for the V elements whose first element has linear index `lin` in the root shape.
// `acc0` feeds VM_SRC_ACC0 operands.  On return `acc` holds the final accumulator (used by reductions).
template <int V>
__device__ __forceinline__ void vm_run(const B2xVmProgram& P, uint64_t lin, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  int64_t coord[B2X_VM_MAX_DIMS];
  vm_coords(P, lin, coord);
  const int nd = P.n_dims;
  uint32_t t0[V], t1[V], t2[V], t3[V], t4[V], t5[V];
  uint32_t b[V];
#pragma unroll
  for (int j = 0; j < V; j++) { acc[j] = 0; b[j] = 0; t0[j] = t1[j] = t2[j] = t3[j] = t4[j] = t5[j] = 0; }

#pragma unroll 1
  for (int pc = 0; pc < P.n_instr; pc++) {
    const B2xVmInstr I = P.code[pc];
    // ---- operand fetch ----
    switch (I.src_kind) {
      case VM_SRC_TEMP:
        B2X_VM_TEMP_SWITCH(I.src_idx, T, _Pragma("unroll") for (int j = 0; j < V; j++) b[j] = T[j]);
        break;
      case VM_SRC_TENSOR:
        if (I.op != VM_STORE) {
          const B2xVmTensor& T = P.tensors[I.src_idx];
          int64_t off = 0;
#pragma unroll
          for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d < nd) off += coord[d] * T.stride[d];
          vm_fetch<V>(T, off, T.stride[nd - 1], b);
        }
        break;
      case VM_SRC_IMM:
#pragma unroll
        for (int j = 0; j < V; j++) b[j] = I.imm;
        break;
      case VM_SRC_IOTA: {
        const bool inner = (I.src_idx == nd - 1);
        int32_t c0 = 0;
#pragma unroll
        for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d == I.src_idx) c0 = (int32_t)coord[d];
#pragma unroll
        for (int j = 0; j < V; j++) {
          int32_t c = c0 + (inner ? j : 0);
          b[j] = (I.tc == VM_F32) ? f2u((float)c) : (uint32_t)c;
        }
        break;
      }
      case VM_SRC_ACC0:
#pragma unroll
        for (int j = 0; j < V; j++) b[j] = acc0[j];
        break;
      default: break;
    }
    // ---- execute ----
    switch (I.op) {
      case VM_LOAD:
#pragma unroll
        for (int j = 0; j < V; j++) acc[j] = b[j];
        break;
      case VM_SAVE:
        B2X_VM_TEMP_SWITCH(I.aux, T, _Pragma("unroll") for (int j = 0; j < V; j++) T[j] = acc[j]);
        continue;
      case VM_STORE: {
        const B2xVmTensor& T = P.tensors[I.src_idx];
        int64_t off = 0;
#pragma unroll
        for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d < nd) off += coord[d] * T.stride[d];
        vm_put<V>(T, off, T.stride[nd - 1], acc);
        continue;
      }
#define X acc
#define Y b
      case VM_ADD: B2X_VM_BIN(x + y, x + y, x + y) break;
      case VM_SUB: B2X_VM_BIN(x - y, x - y, x - y) break;
      case VM_MUL: B2X_VM_BIN(x * y, x * y, x * y) break;
      case VM_DIV: B2X_VM_BIN(__fdiv_rn(x, y), vm_sdiv(x, y), vm_udiv(x, y)) break;
      case VM_MAX: B2X_VM_BIN(vm_fmax(x, y), max(x, y), max(x, y)) break;
      case VM_MIN: B2X_VM_BIN(vm_fmin(x, y), min(x, y), min(x, y)) break;
      case VM_POW: B2X_VM_BIN(powf(x, y), vm_ipow(x, y), (uint32_t)vm_ipow((int)x, (int)y)) break;
      case VM_REM: B2X_VM_BIN(fmodf(x, y), vm_srem(x, y), vm_urem(x, y)) break;
      case VM_AND: B2X_VM_BIN(u2f(f2u(x) & f2u(y)), x & y, x & y) break;
      case VM_OR: B2X_VM_BIN(u2f(f2u(x) | f2u(y)), x | y, x | y) break;
      case VM_XOR: B2X_VM_BIN(u2f(f2u(x) ^ f2u(y)), x ^ y, x ^ y) break;
      case VM_CMP: B2X_VM_BIN(u2f(vm_cmp<float>(x, y, I.aux) ? 1u : 0u), vm_cmp<int>(x, y, I.aux) ? 1 : 0, vm_cmp<uint32_t>(x, y, I.aux) ? 1u : 0u) break;
#undef X
#undef Y
#define X b
#define Y acc
      case VM_RSUB: B2X_VM_BIN(x - y, x - y, x - y) break;
      case VM_RDIV: B2X_VM_BIN(__fdiv_rn(x, y), vm_sdiv(x, y), vm_udiv(x, y)) break;
      case VM_RPOW: B2X_VM_BIN(powf(x, y), vm_ipow(x, y), (uint32_t)vm_ipow((int)x, (int)y)) break;
      case VM_RREM: B2X_VM_BIN(fmodf(x, y), vm_srem(x, y), vm_urem(x, y)) break;
      case VM_RCMP: B2X_VM_BIN(u2f(vm_cmp<float>(x, y, I.aux) ? 1u : 0u), vm_cmp<int>(x, y, I.aux) ? 1 : 0, vm_cmp<uint32_t>(x, y, I.aux) ? 1u : 0u) break;
#undef X
#undef Y
      case VM_NEG: B2X_VM_UN(-x, -x) break;
      case VM_ABS: B2X_VM_UN(fabsf(x), (I.tc == VM_S32 ? (x < 0 ? -x : x) : x)) break;
      case VM_TANH: if (I.aux) B2X_VM_UN(vm_tanh_fast(x), x) else B2X_VM_UN(tanhf(x), x) break;
      case VM_EXP: if (I.aux) B2X_VM_UN(__expf(x), x) else B2X_VM_UN(expf(x), x) break;
      case VM_LOG: if (I.aux) B2X_VM_UN(__logf(x), x) else B2X_VM_UN(logf(x), x) break;
      case VM_SQRT: B2X_VM_UN(sqrtf(x), x) break;
      case VM_RSQRT: B2X_VM_UN(__fdiv_rn(1.0f, sqrtf(x)), x) break;
      case VM_LOGISTIC: if (I.aux) B2X_VM_UN(__fdividef(1.0f, 1.0f + __expf(-x)), x) else B2X_VM_UN(__fdiv_rn(1.0f, 1.0f + expf(-x)), x) break;
      case VM_NOT:
#pragma unroll
        for (int j = 0; j < V; j++) acc[j] = (I.rnd == VM_RN_PRED) ? (acc[j] == 0u ? 1u : 0u) : ~acc[j];
        break;
      case VM_SIGN: B2X_VM_UN((x != x) ? x : (x > 0.f ? 1.f : (x < 0.f ? -1.f : x)), (x > 0) - (x < 0)) break;
      case VM_FLOOR: B2X_VM_UN(floorf(x), x) break;
      case VM_CEIL: B2X_VM_UN(ceilf(x), x) break;
      case VM_EXPM1: B2X_VM_UN(expm1f(x), x) break;
      case VM_LOG1P: B2X_VM_UN(log1pf(x), x) break;
      case VM_SIN: B2X_VM_UN(sinf(x), x) break;
      case VM_COS: B2X_VM_UN(cosf(x), x) break;
      case VM_CVT: {
        const uint8_t from = I.aux, to = I.tc;
#pragma unroll
        for (int j = 0; j < V; j++) {
          uint32_t v = acc[j];
          if (I.rnd == VM_RN_PRED) { v = (from == VM_F32) ? (u2f(v) != 0.0f ? 1u : 0u) : (v != 0u ? 1u : 0u); }
          else if (from == VM_F32 && to == VM_S32) v = (uint32_t)__float2int_rz(u2f(v));
          else if (from == VM_F32 && to == VM_U32) v = __float2uint_rz(u2f(v));
          else if (from == VM_S32 && to == VM_F32) v = f2u(__int2float_rn((int)v));
          else if (from == VM_U32 && to == VM_F32) v = f2u(__uint2float_rn(v));
          acc[j] = v;
        }
        break;
      }
      case VM_SELECT:
        B2X_VM_TEMP_SWITCH(I.aux, T, _Pragma("unroll") for (int j = 0; j < V; j++) acc[j] = T[j] ? acc[j] : b[j]);
        break;
      case VM_RSELECT:
        B2X_VM_TEMP_SWITCH(I.aux, T, _Pragma("unroll") for (int j = 0; j < V; j++) acc[j] = T[j] ? b[j] : acc[j]);
        break;
      default: break;
    }
    if (I.rnd != VM_RN_NONE && I.op != VM_CVT) {
#pragma unroll
      for (int j = 0; j < V; j++) acc[j] = vm_narrow(acc[j], I.rnd);
    } else if (I.op == VM_CVT && I.rnd != VM_RN_PRED && I.rnd != VM_RN_NONE) {
#pragma unroll
      for (int j = 0; j < V; j++) acc[j] = vm_narrow(acc[j], I.rnd);
    }
  }
}

}  // namespace b2x
