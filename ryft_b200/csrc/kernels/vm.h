// Fused-elementwise program format shared by the planner (host) and the kernels (device).
//
// A fusion group of StableHLO elementwise ops (add/multiply/tanh/convert/compare/select/iota/broadcast_in_dim ...;
// semantics: crates/ryft-mlir/src/dialects/stable_hlo/operations/{arithmetic,comparison,trigonometric,exponential,
// casting,control_flow,miscellaneous,manipulation}.rs) is lowered to a short accumulator-machine program.  Each
// thread evaluates the program for V consecutive elements of the group's root shape with every value held in
// registers: one accumulator, a few temporaries, and operands fetched straight from tensors, immediates or index
// generators.  The same program format drives the standalone elementwise kernel, the prologue of the reduce
// kernels and the epilogue of the GEMM kernels, so a chain of ops never round-trips through HBM.
#pragma once
#include <stdint.h>

#define B2X_VM_MAX_INSTR 56
#define B2X_VM_MAX_TENSORS 8
#define B2X_VM_MAX_DIMS 5
#define B2X_VM_TEMPS 6

enum B2xVmOp : uint8_t {
  VM_END = 0,
  VM_LOAD,     // acc = src
  VM_SAVE,     // temp[aux] = acc
  VM_STORE,    // tensor[src_idx][element] = narrow(acc)        (src_kind == VM_SRC_TENSOR)
  // binary, acc = acc OP src; the R* forms compute src OP acc
  VM_ADD, VM_SUB, VM_RSUB, VM_MUL, VM_DIV, VM_RDIV, VM_MAX, VM_MIN, VM_POW, VM_RPOW, VM_REM, VM_RREM,
  VM_AND, VM_OR, VM_XOR,
  VM_CMP,      // acc = (acc CMP src) ? 1 : 0 ; direction in aux (B2xCmp), operand class in tc
  VM_RCMP,     // acc = (src CMP acc) ? 1 : 0
  // unary on acc
  VM_NEG, VM_ABS, VM_TANH, VM_EXP, VM_LOG, VM_SQRT, VM_RSQRT, VM_LOGISTIC, VM_NOT, VM_SIGN, VM_FLOOR, VM_CEIL,
  VM_EXPM1, VM_LOG1P, VM_SIN, VM_COS,
  VM_CVT,      // reinterpret acc from class aux to class tc (value conversion), then narrow per rnd
  // ternary
  VM_SELECT,   // acc = temp[aux] ? acc : src
  VM_RSELECT,  // acc = temp[aux] ? src : acc
};

enum B2xCmp : uint8_t { VM_EQ = 0, VM_NE, VM_GE, VM_GT, VM_LE, VM_LT };

// Register class of a value: all registers are 32 bits wide.
enum B2xVmClass : uint8_t { VM_F32 = 0, VM_S32 = 1, VM_U32 = 2 };

// Narrowing applied after an op so that a value of a narrower element type carries exactly that type's precision
// or range (e.g. a bf16 add rounds to bf16 after every op, as a CPU evaluation in bf16 does).
enum B2xVmRound : uint8_t { VM_RN_NONE = 0, VM_RN_BF16, VM_RN_F16, VM_RN_S8, VM_RN_S16, VM_RN_U8, VM_RN_U16, VM_RN_PRED };

enum B2xVmSrc : uint8_t {
  VM_SRC_NONE = 0,
  VM_SRC_TEMP,    // temp[src_idx]
  VM_SRC_TENSOR,  // tensors[src_idx] at the element's coordinates (strides may be 0 for broadcast dims)
  VM_SRC_IMM,     // imm (raw 32-bit pattern of the class)
  VM_SRC_IOTA,    // coordinate along root dim src_idx (as S32/U32, or converted to F32 when tc == VM_F32)
  VM_SRC_ACC0,    // value handed in by the enclosing kernel (GEMM accumulator); F32
};

// Element types as stored in tensors (numeric values equal b2x::DType).
enum B2xElem : uint8_t {
  EL_PRED = 0, EL_S8, EL_S16, EL_S32, EL_S64, EL_U8, EL_U16, EL_U32, EL_U64, EL_F16, EL_BF16, EL_F32, EL_F64
};

struct B2xVmInstr {
  uint8_t op, src_kind, src_idx, aux, tc, rnd, pad0, pad1;
  uint32_t imm;
};

struct B2xVmTensor {
  void* ptr;                          // patched per launch
  int64_t stride[B2X_VM_MAX_DIMS];    // in elements, per (merged) root dim; 0 = broadcast
  uint8_t elem;                       // B2xElem
  uint8_t pad[7];
};

struct B2xVmProgram {
  int32_t n_instr;
  int32_t n_tensors;
  int32_t n_dims;                     // merged root dims, outermost first; dim[n_dims-1] is the vector dim
  int32_t pad;
  int64_t dim[B2X_VM_MAX_DIMS];
  B2xVmTensor tensors[B2X_VM_MAX_TENSORS];
  B2xVmInstr code[B2X_VM_MAX_INSTR];
};
