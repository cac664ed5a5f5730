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
// Stores are streaming (evict-first in L2): results are written once, and a kernel's own operands, which the other
// CTAs are still re-reading out of L2, should not be pushed out by them.
template <int NB>
__device__ __forceinline__ void vm_st_bytes(void* p, const uint32_t* raw) {
  if constexpr (NB == 32) {
    __stcs((uint4*)p, make_uint4(raw[0], raw[1], raw[2], raw[3]));
    __stcs((uint4*)p + 1, make_uint4(raw[4], raw[5], raw[6], raw[7]));
  } else if constexpr (NB == 16) {
    __stcs((uint4*)p, make_uint4(raw[0], raw[1], raw[2], raw[3]));
  } else if constexpr (NB == 8) {
    __stcs((uint2*)p, make_uint2(raw[0], raw[1]));
  } else if constexpr (NB == 4) {
    __stcs((uint32_t*)p, raw[0]);
  } else if constexpr (NB == 2) {
    __stcs((uint16_t*)p, (uint16_t)raw[0]);
  } else {
    __stcs((uint8_t*)p, (uint8_t)raw[0]);
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
__device__ __forceinline__ void vm_fetch(const void* ptr, const uint8_t elem, int64_t off, int64_t istride, uint32_t (&b)[V]) {
  const int es = vm_elem_size(elem);
  const char* base = (const char*)ptr + off * es;
  if (istride == 0 || V == 1) {
    uint32_t raw;
    if (es == 4) vm_ld_bytes<4>(base, &raw); else if (es == 2) vm_ld_bytes<2>(base, &raw); else vm_ld_bytes<1>(base, &raw);
    raw = vm_decode(raw, elem);
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
        for (int j = 0; j < V; j++) b[j] = vm_decode((raw[j / 2] >> ((j & 1) * 16)) & 0xffffu, elem);
        return;
      }
    } else if (es == 1) {
      if (((uintptr_t)base & (V - 1)) == 0) {
        uint32_t raw[(V + 3) / 4];
        vm_ld_bytes<V>(base, raw);
#pragma unroll
        for (int j = 0; j < V; j++) b[j] = vm_decode((raw[j / 4] >> ((j & 3) * 8)) & 0xffu, elem);
        return;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < V; j++) {
    uint32_t raw;
    const char* p = base + (int64_t)j * istride * es;
    if (es == 4) vm_ld_bytes<4>(p, &raw); else if (es == 2) vm_ld_bytes<2>(p, &raw); else vm_ld_bytes<1>(p, &raw);
    b[j] = vm_decode(raw, elem);
  }
}

template <int V>
__device__ __forceinline__ void vm_put(void* ptr, const uint8_t elem, int64_t off, int64_t istride, const uint32_t (&a)[V]) {
  const int es = vm_elem_size(elem);
  char* base = (char*)ptr + off * es;
  if (istride == 1 && V > 1) {
    if (es == 4 && ((uintptr_t)base & (V * 4 >= 16 ? 15 : V * 4 - 1)) == 0) {
      uint32_t raw[V];
#pragma unroll
      for (int j = 0; j < V; j++) raw[j] = vm_encode(a[j], elem);
      vm_st_bytes<V * 4>(base, raw);
      return;
    }
    if (es == 2 && ((uintptr_t)base & (V * 2 - 1)) == 0) {
      uint32_t raw[(V + 1) / 2];
      if (elem == EL_BF16 && V % 2 == 0) {
#pragma unroll
        for (int j = 0; j < V / 2; j++) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(u2f(a[2 * j]), u2f(a[2 * j + 1]));
          raw[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
      } else {
#pragma unroll
        for (int j = 0; j < (V + 1) / 2; j++) raw[j] = 0;
#pragma unroll
        for (int j = 0; j < V; j++) raw[j / 2] |= vm_encode(a[j], elem) << ((j & 1) * 16);
      }
      vm_st_bytes<V * 2>(base, raw);
      return;
    }
    if (es == 1 && ((uintptr_t)base & (V - 1)) == 0) {
      uint32_t raw[(V + 3) / 4];
#pragma unroll
      for (int j = 0; j < (V + 3) / 4; j++) raw[j] = 0;
#pragma unroll
      for (int j = 0; j < V; j++) raw[j / 4] |= vm_encode(a[j], elem) << ((j & 3) * 8);
      vm_st_bytes<V>(base, raw);
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < V; j++) {
    uint32_t raw = vm_encode(a[j], elem);
    char* p = base + (int64_t)j * istride * es;
    if (es == 4) vm_st_bytes<4>(p, &raw); else if (es == 2) vm_st_bytes<2>(p, &raw); else vm_st_bytes<1>(p, &raw);
  }
}

// Row-contiguous variants for the row-wise driver: `p` is the byte address of the vector's first element, already
// checked (once per row) to be 16-byte aligned whenever the tensor is contiguous along the row.
template <int V>
__device__ __forceinline__ void vm_fetch_row(const char* p, const uint8_t elem, const bool contiguous, uint32_t (&b)[V]) {
  const int es = vm_elem_size(elem);
  if (!contiguous) {
    uint32_t raw;
    if (es == 4) vm_ld_bytes<4>(p, &raw); else if (es == 2) vm_ld_bytes<2>(p, &raw); else vm_ld_bytes<1>(p, &raw);
    raw = vm_decode(raw, elem);
#pragma unroll
    for (int j = 0; j < V; j++) b[j] = raw;
  } else if (es == 4) {
    vm_ld_bytes<V * 4>(p, b);
  } else if (es == 2) {
    uint32_t raw[(V + 1) / 2];
    vm_ld_bytes<V * 2>(p, raw);
#pragma unroll
    for (int j = 0; j < V; j++) b[j] = vm_decode((raw[j / 2] >> ((j & 1) * 16)) & 0xffffu, elem);
  } else {
    uint32_t raw[(V + 3) / 4];
    vm_ld_bytes<V>(p, raw);
#pragma unroll
    for (int j = 0; j < V; j++) b[j] = vm_decode((raw[j / 4] >> ((j & 3) * 8)) & 0xffu, elem);
  }
}
template <int V>
__device__ __forceinline__ void vm_put_row(char* p, const uint8_t elem, const uint32_t (&a)[V]) {
  const int es = vm_elem_size(elem);
  if (es == 4) {
    uint32_t raw[V];
#pragma unroll
    for (int j = 0; j < V; j++) raw[j] = vm_encode(a[j], elem);
    vm_st_bytes<V * 4>(p, raw);
  } else if (es == 2) {
    uint32_t raw[(V + 1) / 2];
    if (elem == EL_BF16) {
#pragma unroll
      for (int j = 0; j < V / 2; j++) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(u2f(a[2 * j]), u2f(a[2 * j + 1]));
        raw[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int j = 0; j < (V + 1) / 2; j++) raw[j] = 0;
#pragma unroll
      for (int j = 0; j < V; j++) raw[j / 2] |= vm_encode(a[j], elem) << ((j & 1) * 16);
    }
    vm_st_bytes<V * 2>(p, raw);
  } else {
    uint32_t raw[(V + 3) / 4];
#pragma unroll
    for (int j = 0; j < (V + 3) / 4; j++) raw[j] = 0;
#pragma unroll
    for (int j = 0; j < V; j++) raw[j / 4] |= vm_encode(a[j], elem) << ((j & 3) * 8);
    vm_st_bytes<V>(p, raw);
  }
}

// Per-row addressing state of the row-wise driver's fast path: byte address of each tensor's element (row, column 0)
// and the byte step per column (0 for tensors broadcast along the row).
struct VmRowAddr {
  const char* rp[B2X_VM_MAX_TENSORS];
  int32_t cs[B2X_VM_MAX_TENSORS];
  uint32_t stage[2];   // staged stores only: shared-memory addresses of the vector's first and second 16-byte piece
};
__device__ __forceinline__ void vm_sts16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Staged store of 8 elements (16-bit: one piece, 32-bit: two pieces) for kernels that write their result tile with a
// bulk tensor store from shared memory.
__device__ __forceinline__ void vm_put_stage(const VmRowAddr& RA, const uint8_t elem, const uint32_t (&a)[8]) {
  if (vm_elem_size(elem) == 4) {
    vm_sts16(RA.stage[0], vm_encode(a[0], elem), vm_encode(a[1], elem), vm_encode(a[2], elem), vm_encode(a[3], elem));
    vm_sts16(RA.stage[1], vm_encode(a[4], elem), vm_encode(a[5], elem), vm_encode(a[6], elem), vm_encode(a[7], elem));
  } else {
    uint32_t raw[4];
    if (elem == EL_BF16) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(u2f(a[2 * j]), u2f(a[2 * j + 1]));
        raw[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) raw[j] = vm_encode(a[2 * j], elem) | (vm_encode(a[2 * j + 1], elem) << 16);
    }
    vm_sts16(RA.stage[0], raw[0], raw[1], raw[2], raw[3]);
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

// Fast tanh of a whole vector (used where the planner allows the hardware approximation: a 16-bit float value that is
// only returned).  tanh.approx goes through the 16-lane special-function pipe, which a GEMM epilogue that applies tanh
// to every element saturates long before memory does.  When every element of the vector has |x| <= 1 (pre-activations
// usually do) an odd polynomial on the FMA pipes, two elements per instruction, replaces it: x * P(x^2) with P of degree
// 4 fitted to tanh(x) / x on [0, 1], relative error below 2^-16 (tanh.approx: 2^-11).  Anything else, NaN included,
// takes tanh.approx.
template <int V>
__device__ __forceinline__ void vm_tanh_fast_vec(uint32_t (&a)[V]) {
  if constexpr (V % 2 == 0) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < V; j++) asm("max.NaN.f32 %0, %0, %1;" : "+f"(m) : "f"(fabsf(u2f(a[j]))));   // a NaN element makes m NaN
    if (m <= 1.0f) {
      auto splat = [](float v) { uint64_t r; asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "r"(__float_as_uint(v))); return r; };
      const uint64_t c4 = splat(0.009248304937f), c3 = splat(-0.04529244860f), c2 = splat(0.1307216824f), c1 = splat(-0.3330772912f),
                     one = splat(1.0f);
#pragma unroll
      for (int j = 0; j < V; j += 2) {
        uint64_t x, t, p;
        asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "r"(a[j]), "r"(a[j + 1]));
        asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(t) : "l"(x));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(t), "l"(c4), "l"(c3));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(p), "l"(t), "l"(c2));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(p), "l"(t), "l"(c1));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(p), "l"(t), "l"(one));
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p) : "l"(x), "l"(p));
        asm("mov.b64 {%0, %1}, %2;" : "=r"(a[j]), "=r"(a[j + 1]) : "l"(p));
      }
      return;
    }
  }
#pragma unroll
  for (int j = 0; j < V; j++) a[j] = f2u(vm_tanh_fast(u2f(a[j])));
}

// tanh to within about 2 ulp without divergent branches: odd polynomial for |x| < 0.3, 1 - 2 / (1 + e^{2|x|}) above
// (ex2.approx and rcp.approx are each within 2^-22 relative, the result is >= 0.29 there so the absolute error of the
// quotient stays below one ulp of the result).
__device__ __forceinline__ float vm_tanh(float x) {
  const float ax = fabsf(x);
  const float x2 = x * x;
  float p = fmaf(x2, -0.00886323552f, 0.0218694885f);      // -1382/155925, 62/2835
  p = fmaf(x2, p, -0.0539682540f);                          // -17/315
  p = fmaf(x2, p, 0.133333333f);                            // 2/15
  p = fmaf(x2, p, -0.333333333f);                           // -1/3
  const float small = fmaf(x * x2, p, x);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(ax * 2.88539008f));   // e^{2|x|}
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  const float big = copysignf(fmaf(-2.0f, r, 1.0f), x);
  return ax < 0.3f ? small : big;
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

// ---- out-of-line helpers for rarely used ops: keeps the interpreter's hot code small enough for the instruction cache
static __device__ __noinline__ float vm_rare_f32(uint8_t op, float x, float y) {
  switch (op) {
    case VM_POW: return powf(x, y);
    case VM_REM: return fmodf(x, y);
    case VM_EXPM1: return expm1f(x);
    case VM_LOG1P: return log1pf(x);
    case VM_SIN: return sinf(x);
    case VM_COS: return cosf(x);
    case VM_SIGN: return (x != x) ? x : (x > 0.f ? 1.f : (x < 0.f ? -1.f : x));
    case VM_FLOOR: return floorf(x);
    case VM_CEIL: return ceilf(x);
    case VM_LOG: return logf(x);
    case VM_LOGISTIC: return __fdiv_rn(1.0f, 1.0f + expf(-x));
    case VM_RSQRT: return __fdiv_rn(1.0f, sqrtf(x));
    default: return x;
  }
}
static __device__ __noinline__ uint32_t vm_rare_int(uint8_t op, uint8_t tc, uint32_t x, uint32_t y) {
  const bool s = tc == VM_S32;
  switch (op) {
    case VM_DIV: return s ? (uint32_t)vm_sdiv((int)x, (int)y) : vm_udiv(x, y);
    case VM_REM: return s ? (uint32_t)vm_srem((int)x, (int)y) : vm_urem(x, y);
    case VM_POW: return (uint32_t)vm_ipow((int)x, (int)y);
    case VM_SIGN: return s ? (uint32_t)(((int)x > 0) - ((int)x < 0)) : (x != 0u);
    default: return x;
  }
}

// Register state of one program run: accumulator, operand, temporaries.  Always indexed with compile-time constants
// after inlining, so it lives in registers.
template <int V>
struct VmState {
  uint32_t acc[V], b[V], t0[V], t1[V], t2[V], t3[V], t4[V], t5[V];
};

#define B2X_VM_TEMP_SWITCH(idx, T, stmt)                 \
  switch (idx) {                                          \
    case 0: { auto& T = S.t0; stmt; } break;              \
    case 1: { auto& T = S.t1; stmt; } break;              \
    case 2: { auto& T = S.t2; stmt; } break;              \
    case 3: { auto& T = S.t3; stmt; } break;              \
    case 4: { auto& T = S.t4; stmt; } break;              \
    default: { auto& T = S.t5; stmt; } break;             \
  }

#define B2X_VM_BIN(EF, ES, EU)                                                                                \
  {                                                                                                           \
    if (tc == VM_F32) {                                                                                       \
      _Pragma("unroll") for (int j = 0; j < V; j++) { float x = u2f(X[j]), y = u2f(Y[j]); S.acc[j] = f2u(EF); } \
    } else if (tc == VM_S32) {                                                                                \
      _Pragma("unroll") for (int j = 0; j < V; j++) { int x = (int)X[j], y = (int)Y[j]; S.acc[j] = (uint32_t)(ES); } \
    } else {                                                                                                  \
      _Pragma("unroll") for (int j = 0; j < V; j++) { uint32_t x = X[j], y = Y[j]; S.acc[j] = (uint32_t)(EU); } \
    }                                                                                                         \
  }
#define B2X_VM_BIN_RARE(OPC)                                                                                  \
  {                                                                                                           \
    if (tc == VM_F32) {                                                                                       \
      _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = f2u(vm_rare_f32(OPC, u2f(X[j]), u2f(Y[j])));    \
    } else {                                                                                                  \
      _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = vm_rare_int(OPC, tc, X[j], Y[j]);               \
    }                                                                                                         \
  }
#define B2X_VM_UN_F(EF) { _Pragma("unroll") for (int j = 0; j < V; j++) { float x = u2f(S.acc[j]); S.acc[j] = f2u(EF); } }
#define B2X_VM_UN_RARE(OPC)                                                                                   \
  {                                                                                                           \
    if (tc == VM_F32) {                                                                                       \
      _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = f2u(vm_rare_f32(OPC, u2f(S.acc[j]), 0.f));      \
    } else {                                                                                                  \
      _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = vm_rare_int(OPC, tc, S.acc[j], 0u);             \
    }                                                                                                         \
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

__device__ __forceinline__ int64_t vm_offset(const B2xVmTensor& T, const int64_t (&coord)[B2X_VM_MAX_DIMS], int nd) {
  int64_t off = 0;
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d < nd) off += coord[d] * T.stride[d];
  return off;
}

// One instruction.  Every argument except the state is uniform across the grid; when the caller passes compile-time
// constants (specialised programs) the switches below fold away and only the selected op's code remains.
// `off[t]` is tensor t's element offset for this vector without the part contributed by `col` along the innermost dim
// (callers that have no separate column pass col = 0 and fold everything into off).
template <int V, bool RF = false, bool STG = false, bool AC = false>
__device__ __forceinline__ void vm_exec(const B2xVmProgram& P, const int64_t (&coord)[B2X_VM_MAX_DIMS], const int nd,
                                        const int64_t (&off)[B2X_VM_MAX_TENSORS], const VmRowAddr& RA, const int64_t col, const uint8_t op,
                                        const uint8_t src_kind, const uint8_t src_idx, const uint8_t aux, const uint8_t tc, const uint8_t rnd,
                                        const uint32_t imm, const uint8_t elem, const uint32_t (&acc0)[V], VmState<V>& S) {
  // ---- operand fetch ----
  switch (src_kind) {
    case VM_SRC_TEMP:
      B2X_VM_TEMP_SWITCH(src_idx, T, _Pragma("unroll") for (int j = 0; j < V; j++) S.b[j] = T[j]);
      break;
    case VM_SRC_TENSOR:
      if (op != VM_STORE) {
        if constexpr (RF) {
          const char* rp = nullptr; int32_t cs = 0;
#pragma unroll
          for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) if (t == src_idx) { rp = RA.rp[t]; cs = RA.cs[t]; }
          // AC: the caller has checked that every tensor the program reads is contiguous along the row, so the fetch has
          // no branch and the loads of several vectors can be in flight together
          vm_fetch_row<V>(rp + (int64_t)((int32_t)col * cs), elem, AC ? true : cs != 0, S.b);
        } else {
          const B2xVmTensor& T = P.tensors[src_idx];
          int64_t o = 0;
#pragma unroll
          for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) if (t == src_idx) o = off[t];
          vm_fetch<V>(T.ptr, elem, o + col * T.stride[nd - 1], T.stride[nd - 1], S.b);
        }
      }
      break;
    case VM_SRC_IMM:
#pragma unroll
      for (int j = 0; j < V; j++) S.b[j] = imm;
      break;
    case VM_SRC_IOTA: {
      const bool inner = (src_idx == nd - 1);
      int32_t c0 = 0;
#pragma unroll
      for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d == src_idx) c0 = (int32_t)coord[d];
      if (inner) c0 += (int32_t)col;
#pragma unroll
      for (int j = 0; j < V; j++) {
        int32_t c = c0 + (inner ? j : 0);
        S.b[j] = (tc == VM_F32) ? f2u((float)c) : (uint32_t)c;
      }
      break;
    }
    case VM_SRC_ACC0:
#pragma unroll
      for (int j = 0; j < V; j++) S.b[j] = acc0[j];
      break;
    default: break;
  }
  // ---- execute ----
  bool narrow = true;
  switch (op) {
    case VM_LOAD:
#pragma unroll
      for (int j = 0; j < V; j++) S.acc[j] = S.b[j];
      break;
    case VM_SAVE:
      B2X_VM_TEMP_SWITCH(aux, T, _Pragma("unroll") for (int j = 0; j < V; j++) T[j] = S.acc[j]);
      narrow = false;
      break;
    case VM_STORE: {
      if constexpr (STG) {
        static_assert(V == 8, "staged stores are 8 elements wide");
        vm_put_stage(RA, elem, S.acc);
        narrow = false;
        break;
      } else if constexpr (RF) {
        const char* rp = nullptr; int32_t cs = 0;
#pragma unroll
        for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) if (t == src_idx) { rp = RA.rp[t]; cs = RA.cs[t]; }
        vm_put_row<V>(const_cast<char*>(rp) + (int64_t)((int32_t)col * cs), elem, S.acc);
        narrow = false;
        break;
      }
      const B2xVmTensor& T = P.tensors[src_idx];
      int64_t o = 0;
#pragma unroll
      for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) if (t == src_idx) o = off[t];
      vm_put<V>(T.ptr, elem, o + col * T.stride[nd - 1], T.stride[nd - 1], S.acc);
      narrow = false;
      break;
    }
#define X S.acc
#define Y S.b
    case VM_ADD: B2X_VM_BIN(x + y, x + y, x + y) break;
    case VM_SUB: B2X_VM_BIN(x - y, x - y, x - y) break;
    case VM_MUL: B2X_VM_BIN(x * y, x * y, x * y) break;
    case VM_DIV: if (tc == VM_F32) B2X_VM_BIN(__fdiv_rn(x, y), 0, 0) else B2X_VM_BIN_RARE(VM_DIV) break;
    case VM_MAX: B2X_VM_BIN(vm_fmax(x, y), max(x, y), max(x, y)) break;
    case VM_MIN: B2X_VM_BIN(vm_fmin(x, y), min(x, y), min(x, y)) break;
    case VM_POW: B2X_VM_BIN_RARE(VM_POW) break;
    case VM_REM: B2X_VM_BIN_RARE(VM_REM) break;
    case VM_AND: B2X_VM_BIN(u2f(f2u(x) & f2u(y)), x & y, x & y) break;
    case VM_OR: B2X_VM_BIN(u2f(f2u(x) | f2u(y)), x | y, x | y) break;
    case VM_XOR: B2X_VM_BIN(u2f(f2u(x) ^ f2u(y)), x ^ y, x ^ y) break;
    case VM_CMP: B2X_VM_BIN(u2f(vm_cmp<float>(x, y, aux) ? 1u : 0u), vm_cmp<int>(x, y, aux) ? 1 : 0, vm_cmp<uint32_t>(x, y, aux) ? 1u : 0u) break;
#undef X
#undef Y
#define X S.b
#define Y S.acc
    case VM_RSUB: B2X_VM_BIN(x - y, x - y, x - y) break;
    case VM_RDIV: if (tc == VM_F32) B2X_VM_BIN(__fdiv_rn(x, y), 0, 0) else B2X_VM_BIN_RARE(VM_DIV) break;
    case VM_RPOW: B2X_VM_BIN_RARE(VM_POW) break;
    case VM_RREM: B2X_VM_BIN_RARE(VM_REM) break;
    case VM_RCMP: B2X_VM_BIN(u2f(vm_cmp<float>(x, y, aux) ? 1u : 0u), vm_cmp<int>(x, y, aux) ? 1 : 0, vm_cmp<uint32_t>(x, y, aux) ? 1u : 0u) break;
#undef X
#undef Y
    case VM_NEG:
      if (tc == VM_F32) B2X_VM_UN_F(-x) else { _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = 0u - S.acc[j]; }
      break;
    case VM_ABS:
      if (tc == VM_F32) B2X_VM_UN_F(fabsf(x))
      else if (tc == VM_S32) { _Pragma("unroll") for (int j = 0; j < V; j++) { int x = (int)S.acc[j]; S.acc[j] = (uint32_t)(x < 0 ? -x : x); } }
      break;
    // GEMM epilogues (RF / STG) are bound by instruction issue, not by the special-function pipe: there the one-instruction
    // tanh.approx wins; the standalone elementwise kernel has issue slots to spare and takes the polynomial
    case VM_TANH:
      if (aux) { if constexpr (RF || STG) B2X_VM_UN_F(vm_tanh_fast(x)) else vm_tanh_fast_vec<V>(S.acc); }
      else B2X_VM_UN_F(vm_tanh(x))
      break;
    case VM_EXP: if (aux) B2X_VM_UN_F(__expf(x)) else B2X_VM_UN_F(expf(x)) break;
    case VM_SQRT: B2X_VM_UN_F(sqrtf(x)) break;
    case VM_LOG: if (aux) B2X_VM_UN_F(__logf(x)) else B2X_VM_UN_RARE(VM_LOG) break;
    case VM_LOGISTIC: if (aux) B2X_VM_UN_F(__fdividef(1.0f, 1.0f + __expf(-x))) else B2X_VM_UN_RARE(VM_LOGISTIC) break;
    case VM_RSQRT: B2X_VM_UN_RARE(VM_RSQRT) break;
    case VM_SIGN: B2X_VM_UN_RARE(VM_SIGN) break;
    case VM_FLOOR: B2X_VM_UN_RARE(VM_FLOOR) break;
    case VM_CEIL: B2X_VM_UN_RARE(VM_CEIL) break;
    case VM_EXPM1: B2X_VM_UN_RARE(VM_EXPM1) break;
    case VM_LOG1P: B2X_VM_UN_RARE(VM_LOG1P) break;
    case VM_SIN: B2X_VM_UN_RARE(VM_SIN) break;
    case VM_COS: B2X_VM_UN_RARE(VM_COS) break;
    case VM_NOT:
#pragma unroll
      for (int j = 0; j < V; j++) S.acc[j] = (rnd == VM_RN_PRED) ? (S.acc[j] == 0u ? 1u : 0u) : ~S.acc[j];
      break;
    case VM_CVT: {
      const uint8_t from = aux, to = tc;
#pragma unroll
      for (int j = 0; j < V; j++) {
        uint32_t v = S.acc[j];
        if (rnd == VM_RN_PRED) { v = (from == VM_F32) ? (u2f(v) != 0.0f ? 1u : 0u) : (v != 0u ? 1u : 0u); }
        else if (from == VM_F32 && to == VM_S32) v = (uint32_t)__float2int_rz(u2f(v));
        else if (from == VM_F32 && to == VM_U32) v = __float2uint_rz(u2f(v));
        else if (from == VM_S32 && to == VM_F32) v = f2u(__int2float_rn((int)v));
        else if (from == VM_U32 && to == VM_F32) v = f2u(__uint2float_rn(v));
        S.acc[j] = v;
      }
      break;
    }
    case VM_SELECT:
      B2X_VM_TEMP_SWITCH(aux, T, _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = T[j] ? S.acc[j] : S.b[j]);
      narrow = false;
      break;
    case VM_RSELECT:
      B2X_VM_TEMP_SWITCH(aux, T, _Pragma("unroll") for (int j = 0; j < V; j++) S.acc[j] = T[j] ? S.b[j] : S.acc[j]);
      narrow = false;
      break;
    default: break;
  }
  if (narrow && rnd != VM_RN_NONE && !(op == VM_CVT && rnd == VM_RN_PRED)) {
    if (rnd == VM_RN_BF16 && V % 2 == 0) {
      // pairs through the packed conversion: it issues on the ALU pipes, the scalar one on the 16-lane XU pipe that
      // tanh/exp also need
#pragma unroll
      for (int j = 0; j < V / 2; j++) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(u2f(S.acc[2 * j]), u2f(S.acc[2 * j + 1]));
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(&h);
        S.acc[2 * j] = raw << 16;
        S.acc[2 * j + 1] = raw & 0xffff0000u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < V; j++) S.acc[j] = vm_narrow(S.acc[j], rnd);
    }
  }
}

// ---- specialised programs ---------------------------------------------------------------------------------------------
// VmStatic<ID> describes a program whose structure is known when the library is built (generated table below); ID 0
// is the interpreter.  A specialised run unrolls the program at compile time, so each instruction's opcode, operand
// kind, register class, rounding and tensor element types are constants and the op switches disappear; immediates,
// pointers, strides and dims still come from the B2xVmProgram passed at launch.
struct VmSig { uint8_t op, src_kind, src_idx, aux, tc, rnd; };
template <int ID> struct VmStatic { static constexpr int n = 0; };

}  // namespace b2x
#include "vm_static_table.h"
namespace b2x {

// Number of global stores a specialised program issues per vector.
template <int ID>
__host__ __device__ constexpr int vm_static_stores() {
  int k = 0;
  for (int i = 0; i < VmStatic<ID>::n; i++) if (VmStatic<ID>::at(i).op == VM_STORE) k++;
  return k;
}

template <int V, int ID, bool RF, bool STG, int PC, bool AC = false>
__device__ __forceinline__ void vm_unroll(const B2xVmProgram& P, const int64_t (&coord)[B2X_VM_MAX_DIMS], const int nd,
                                          const int64_t (&off)[B2X_VM_MAX_TENSORS], const VmRowAddr& RA, const int64_t col,
                                          const uint32_t (&acc0)[V], VmState<V>& S) {
  if constexpr (PC < VmStatic<ID>::n) {
    constexpr VmSig G = VmStatic<ID>::at(PC);
    constexpr uint8_t elem = (G.src_kind == VM_SRC_TENSOR) ? VmStatic<ID>::elem(G.src_idx) : (uint8_t)0;
    vm_exec<V, RF, STG, AC>(P, coord, nd, off, RA, col, G.op, G.src_kind, G.src_idx, G.aux, G.tc, G.rnd, P.code[PC].imm, elem, acc0, S);
    vm_unroll<V, ID, RF, STG, PC + 1, AC>(P, coord, nd, off, RA, col, acc0, S);
  }
}

template <int V, int ID, bool RF = false, bool STG = false, bool AC = false>
__device__ __forceinline__ void vm_run_core(const B2xVmProgram& P, const int64_t (&coord)[B2X_VM_MAX_DIMS], const int64_t (&off)[B2X_VM_MAX_TENSORS],
                                            const VmRowAddr& RA, const int64_t col, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  const int nd = P.n_dims;
  VmState<V> S;
#pragma unroll
  for (int j = 0; j < V; j++) { S.acc[j] = 0; S.b[j] = 0; S.t0[j] = S.t1[j] = S.t2[j] = S.t3[j] = S.t4[j] = S.t5[j] = 0; }
  if constexpr (ID == 0) {
#pragma unroll 1
    for (int pc = 0; pc < P.n_instr; pc++) {
      const B2xVmInstr I = P.code[pc];
      const uint8_t elem = (I.src_kind == VM_SRC_TENSOR) ? P.tensors[I.src_idx].elem : (uint8_t)0;
      vm_exec<V, RF>(P, coord, nd, off, RA, col, I.op, I.src_kind, I.src_idx, I.aux, I.tc, I.rnd, I.imm, elem, acc0, S);
    }
  } else {
    vm_unroll<V, ID, RF, STG, 0, AC>(P, coord, nd, off, RA, col, acc0, S);
  }
#pragma unroll
  for (int j = 0; j < V; j++) acc[j] = S.acc[j];
}

// Runs the program for the V elements whose first element has linear index `lin` in the root shape.
// `acc0` feeds VM_SRC_ACC0 operands.  On return `acc` holds the final accumulator (used by reductions).
// Programs whose dims merged down to one or two (the usual case) take a short route to coordinates and offsets: at
// most one division and two multiply-adds per tensor.  A caller that already knows the split of `lin` into
// (c0, c1) over [dim0, dim1] passes it with known = true and saves the division as well.
template <int V, int ID = 0>
__device__ __forceinline__ void vm_run_at(const B2xVmProgram& P, uint64_t lin, bool known, int64_t c0, int64_t c1, const uint32_t (&acc0)[V],
                                          uint32_t (&acc)[V]) {
  int64_t coord[B2X_VM_MAX_DIMS];
  int64_t off[B2X_VM_MAX_TENSORS];
  const int nd = P.n_dims;
  if (nd <= 2) {
    if (nd <= 1) { c0 = (int64_t)lin; c1 = 0; }
    else if (!known) {
      if (lin <= 0xffffffffull) { const uint32_t n = (uint32_t)P.dim[1], l = (uint32_t)lin, q = l / n; c0 = q; c1 = l - q * n; }
      else { const uint64_t n = (uint64_t)P.dim[1], q = lin / n; c0 = (int64_t)q; c1 = (int64_t)(lin - q * n); }
    }
#pragma unroll
    for (int d = 0; d < B2X_VM_MAX_DIMS; d++) coord[d] = 0;
    coord[0] = c0; coord[1] = c1;
#pragma unroll
    for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) {
      off[t] = 0;
      if (t < P.n_tensors) off[t] = c0 * P.tensors[t].stride[0] + (nd == 2 ? c1 * P.tensors[t].stride[1] : 0);
    }
  } else {
    vm_coords(P, lin, coord);
#pragma unroll
    for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) off[t] = (t < P.n_tensors) ? vm_offset(P.tensors[t], coord, nd) : 0;
  }
  VmRowAddr ra;      // unused outside the row-wise fast path
  vm_run_core<V, ID>(P, coord, off, ra, 0, acc0, acc);
}
template <int V, int ID = 0>
__device__ __forceinline__ void vm_run(const B2xVmProgram& P, uint64_t lin, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  vm_run_at<V, ID>(P, lin, false, 0, 0, acc0, acc);
}

// Row-wise driver for kernels that walk a [rows, N] result one row at a time (GEMM epilogues): the coordinate
// decomposition and every tensor's row offset are computed once per row, each vector then only adds its column.
struct VmRow {
  int64_t coord[B2X_VM_MAX_DIMS];
  int64_t off[B2X_VM_MAX_TENSORS];
  VmRowAddr addr;
  bool fast;     // the innermost program dim is a whole number of rows
  bool vec;      // fast, and every tensor is either broadcast along the row or contiguous with a 16-byte aligned row start
  uint64_t row;
  uint32_t N;
};
// What vm_row_begin needs that does not depend on the row: computed once per thread, outside the loop over tiles.
struct VmRowPlan {
  bool fast;      // the innermost program dim is a whole number of rows
  bool small;     // row numbers and all outer dims fit in 32 bits: the row is decomposed with 32-bit divisions
  uint64_t per;   // rows folded into the innermost program dim
  // The usual case (the program's dims merged down to [rows * N] or [rows, N]): every tensor's offset is row * step,
  // so a row needs one multiply-add per tensor instead of a coordinate decomposition.
  bool affine, affine_vec;
  int64_t coord_mul;                           // coord[0] = row * coord_mul
  int64_t rowstep[B2X_VM_MAX_TENSORS];         // elements per row
  int32_t cs[B2X_VM_MAX_TENSORS];              // bytes per column
};
__device__ __forceinline__ VmRowPlan vm_row_plan(const B2xVmProgram& P, uint32_t N) {
  VmRowPlan L;
  const int nd = P.n_dims;
  const uint64_t inner = (uint64_t)P.dim[nd - 1];
  L.fast = (inner % N) == 0;
  L.per = L.fast ? inner / N : 1;
  uint64_t rows = L.per;
  bool small = true;
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS - 1; d++) {
    if (d < nd - 1) { const uint64_t n = (uint64_t)P.dim[d]; small = small && n <= 0x7fffffffull && rows <= 0x7fffffffull; rows *= n; }
  }
  L.small = small && rows <= 0x7fffffffull;
  L.affine = L.fast && (nd == 1 || (nd == 2 && L.per == 1));
  L.coord_mul = nd == 1 ? (int64_t)N : 1;
  bool vec = (uint64_t)N * 8 < 0x7fffffffull;
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) {
    L.rowstep[t] = 0; L.cs[t] = 0;
    if (t < P.n_tensors && L.affine) {
      const int es = vm_elem_size(P.tensors[t].elem);
      const int64_t istride = nd == 1 ? P.tensors[t].stride[0] : P.tensors[t].stride[1];
      L.rowstep[t] = nd == 1 ? (int64_t)N * P.tensors[t].stride[0] : P.tensors[t].stride[0];
      L.cs[t] = (int32_t)istride * es;
      vec = vec && es <= 4 && (istride == 0 || (istride == 1 && ((uintptr_t)P.tensors[t].ptr & 15) == 0 && ((L.rowstep[t] * es) & 15) == 0));
    }
  }
  L.affine_vec = vec;
  return L;
}
__device__ __forceinline__ void vm_row_begin(const B2xVmProgram& P, const VmRowPlan& L, uint64_t row, uint32_t N, VmRow& R) {
  const int nd = P.n_dims;
  R.row = row; R.N = N;
  R.fast = L.fast;
  R.vec = false;
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) R.coord[d] = 0;
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) { R.off[t] = 0; R.addr.rp[t] = nullptr; R.addr.cs[t] = 0; }
  if (!R.fast) return;
  if (L.affine) {
    R.coord[0] = (int64_t)row * L.coord_mul;
#pragma unroll
    for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) {
      if (t < P.n_tensors) {
        R.off[t] = (int64_t)row * L.rowstep[t];
        R.addr.rp[t] = (const char*)P.tensors[t].ptr + R.off[t] * vm_elem_size(P.tensors[t].elem);
        R.addr.cs[t] = L.cs[t];
      }
    }
    R.vec = L.affine_vec;
    return;
  }
  int64_t inner_base;
  if (L.small) {
    const uint32_t per = (uint32_t)L.per, r32 = (uint32_t)row;
    uint32_t outer = r32 / per;
    inner_base = (int64_t)((uint64_t)(r32 - outer * per) * N);
#pragma unroll
    for (int d = B2X_VM_MAX_DIMS - 2; d >= 1; d--) {
      if (d < nd - 1) { const uint32_t n = (uint32_t)P.dim[d]; const uint32_t q = outer / n; R.coord[d] = (int64_t)(outer - q * n); outer = q; }
    }
    if (nd >= 2) R.coord[0] = (int64_t)outer;
  } else {
    const uint64_t per = L.per;
    uint64_t outer = row / per;
    inner_base = (int64_t)((row - outer * per) * N);
#pragma unroll
    for (int d = B2X_VM_MAX_DIMS - 2; d >= 1; d--) {
      if (d < nd - 1) { const uint64_t n = (uint64_t)P.dim[d]; const uint64_t q = outer / n; R.coord[d] = (int64_t)(outer - q * n); outer = q; }
    }
    if (nd >= 2) R.coord[0] = (int64_t)outer;
  }
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d == nd - 1) R.coord[d] = inner_base;
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) if (t < P.n_tensors) R.off[t] = vm_offset(P.tensors[t], R.coord, nd);
  bool vec = true;
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) {
    if (t < P.n_tensors) {
      const int es = vm_elem_size(P.tensors[t].elem);
      const int64_t istride = P.tensors[t].stride[nd - 1];
      const char* rp = (const char*)P.tensors[t].ptr + R.off[t] * es;
      R.addr.rp[t] = rp;
      R.addr.cs[t] = (int32_t)istride * es;
      vec = vec && es <= 4 && (istride == 0 || (istride == 1 && ((uintptr_t)rp & 15) == 0));
    }
  }
  R.vec = vec && (uint64_t)N * 8 < 0x7fffffffull;
}
template <int V, int ID = 0>
__device__ __forceinline__ void vm_run_row(const B2xVmProgram& P, const VmRow& R, uint32_t col, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  if (R.fast) vm_run_core<V, ID>(P, R.coord, R.off, R.addr, (int64_t)col, acc0, acc);
  else vm_run<V, ID>(P, R.row * R.N + col, acc0, acc);
}
// Same, for rows with R.vec set: tensor operands are addressed through R.addr with no per-vector stride or alignment
// decisions.  `col` must be a multiple of 8 elements.
template <int V, int ID = 0>
__device__ __forceinline__ void vm_run_row_vec(const B2xVmProgram& P, const VmRow& R, uint32_t col, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  vm_run_core<V, ID, true>(P, R.coord, R.off, R.addr, (int64_t)col, acc0, acc);
}

// Same again for rows on which every tensor the program reads is contiguous (no operand broadcast along the row): the
// fetches are straight-line loads.
template <int V, int ID>
__device__ __forceinline__ void vm_run_row_contig(const B2xVmProgram& P, const VmRow& R, uint32_t col, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  vm_run_core<V, ID, true, false, true>(P, R.coord, R.off, R.addr, (int64_t)col, acc0, acc);
}
// Whether vm_run_row_contig applies to a row prepared by vm_row_begin.
__device__ __forceinline__ bool vm_row_all_contiguous(const B2xVmProgram& P, const VmRow& R) {
  bool ok = R.vec;
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) if (t < P.n_tensors) ok = ok && R.addr.cs[t] != 0;
  return ok;
}

// Addressing of a block of consecutive result rows whose tensor offsets are affine in the row number (the usual case:
// a 32-row slice of a GEMM tile never straddles an outer program dim unless that dim is tiny).  All fields are the
// same for every thread that passes the same arguments.  Row r of the block (0 <= r < nrows) has tensor t's column 0 at
// base[t] + r * step[t]; its coordinates are `coord` with r * coord_mul added at dim coord_dim.
struct VmRowBlock {
  int64_t coord[B2X_VM_MAX_DIMS];
  const char* base[B2X_VM_MAX_TENSORS];
  int64_t step[B2X_VM_MAX_TENSORS];
  int32_t cs[B2X_VM_MAX_TENSORS];
  int32_t coord_dim;
  int64_t coord_mul;
  bool ok;       // affine, contiguous-or-broadcast along the row, every row start 16-byte aligned
};
__device__ __forceinline__ void vm_row_block(const B2xVmProgram& P, const VmRowPlan& L, uint64_t row0, uint32_t nrows, uint32_t N, VmRowBlock& B) {
  const int nd = P.n_dims;
  VmRow R;
  vm_row_begin(P, L, row0, N, R);
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) B.coord[d] = R.coord[d];
  bool ok = R.vec;
  const bool folded = L.per > 1 || nd < 2;
  B.coord_dim = folded ? nd - 1 : nd - 2;
  B.coord_mul = folded ? (int64_t)N : 1;
  // the block must stay inside one value of every dim outside coord_dim
  int64_t at = 0, extent = 1;
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d == B.coord_dim) { at = R.coord[d]; extent = P.dim[d]; }
  ok = ok && (at + (int64_t)(nrows - 1) * B.coord_mul < extent);
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) {
    B.base[t] = R.addr.rp[t]; B.cs[t] = R.addr.cs[t]; B.step[t] = 0;
    if (t < P.n_tensors) {
      const int es = vm_elem_size(P.tensors[t].elem);
      int64_t st = 0;
#pragma unroll
      for (int d = 0; d < B2X_VM_MAX_DIMS; d++) if (d == B.coord_dim) st = P.tensors[t].stride[d];
      B.step[t] = st * B.coord_mul * es;
      ok = ok && (R.addr.cs[t] == 0 || (B.step[t] & 15) == 0);
    }
  }
  B.ok = ok;
}
// Runs the program for the 8-wide vector at column `col` of row r of the block.
template <int V, int ID>
__device__ __forceinline__ void vm_run_block_row(const B2xVmProgram& P, const VmRowBlock& B, uint32_t r, uint32_t col, const uint32_t (&acc0)[V], uint32_t (&acc)[V]) {
  int64_t coord[B2X_VM_MAX_DIMS];
  int64_t off[B2X_VM_MAX_TENSORS];
  VmRowAddr ra;
#pragma unroll
  for (int d = 0; d < B2X_VM_MAX_DIMS; d++) coord[d] = B.coord[d] + (d == B.coord_dim ? (int64_t)r * B.coord_mul : 0);
#pragma unroll
  for (int t = 0; t < B2X_VM_MAX_TENSORS; t++) { off[t] = 0; ra.rp[t] = B.base[t] + (int64_t)r * B.step[t]; ra.cs[t] = B.cs[t]; }
  vm_run_core<V, ID, true>(P, coord, off, ra, (int64_t)col, acc0, acc);
}

// Index of the tensor a specialised program's (single) store writes, or -1.
template <int ID>
__host__ __device__ constexpr int vm_static_store_tensor() {
  int t = -1;
  for (int i = 0; i < VmStatic<ID>::n; i++) if (VmStatic<ID>::at(i).op == VM_STORE) t = VmStatic<ID>::at(i).src_idx;
  return t;
}
// Row-wise run whose store goes to the staging addresses in `stage` instead of global memory.
template <int ID>
__device__ __forceinline__ void vm_run_row_stage(const B2xVmProgram& P, VmRow& R, uint32_t col, uint32_t stage0, uint32_t stage1,
                                                 const uint32_t (&acc0)[8], uint32_t (&acc)[8]) {
  R.addr.stage[0] = stage0; R.addr.stage[1] = stage1;
  vm_run_core<8, ID, true, true>(P, R.coord, R.off, R.addr, (int64_t)col, acc0, acc);
}

// Signature hash of a program (structure only: ops, operand kinds, classes, rounding, tensor element types).
__host__ inline uint64_t vm_signature_hash(const B2xVmProgram& P) {
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](uint8_t b) { h ^= b; h *= 1099511628211ull; };
  mix((uint8_t)P.n_instr);
  for (int i = 0; i < P.n_instr; i++) {
    const B2xVmInstr& I = P.code[i];
    mix(I.op); mix(I.src_kind); mix(I.src_idx); mix(I.aux); mix(I.tc); mix(I.rnd);
  }
  mix((uint8_t)P.n_tensors);
  for (int t = 0; t < P.n_tensors; t++) mix(P.tensors[t].elem);
  return h;
}

}  // namespace b2x
