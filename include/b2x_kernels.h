/*
 * Kernel-level C ABI of the B200 StableHLO executor: the thin `extern "C"` layer between the launch planner and
 * the hand-written sm_100a kernels.  The PJRT plugin links these entry points statically; `libb2x_kernels.so`
 * exports them for direct use (kernel tests, micro-benchmarks, and a host-side lowering pass written in another
 * language).  Every function enqueues work on `stream` and returns a cudaError_t value (0 = success) without
 * synchronising, unless stated otherwise.  Pointers are device pointers unless named `host_*`.
 *
 * Each entry point names the StableHLO op(s) of the reference whose execution it takes over; the reference itself
 * runs them inside its PJRT plugin (crates/ryft-pjrt/src/programs.rs:923-936, PJRT_LoadedExecutable_Execute).
 */
#ifndef B2X_KERNELS_H_
#define B2X_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#include "../ryft_b200/csrc/kernels/vm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b2x_stream_t; /* cudaStream_t */

#define B2X_API __attribute__((visibility("default")))

/* Fused elementwise group (stablehlo.add/subtract/multiply/divide/maximum/minimum/tanh/exponential/convert/
 * compare/select/iota/broadcast_in_dim/constant ...; crates/ryft-mlir/src/dialects/stable_hlo/operations/
 * arithmetic.rs:190-453, comparison.rs:136-164, control_flow.rs:263, casting.rs:123, miscellaneous.rs:50-129,
 * manipulation.rs:339-359).  `prog` is a host pointer; tensor pointers inside it must be bound.  `vec` in {1,4,8}
 * must divide the innermost program dim. */
B2X_API int b2x_launch_elementwise(const B2xVmProgram* host_prog, int64_t n_elements, int vec, b2x_stream_t stream);

/* stablehlo.reduce over the middle extent of an [A, R, B] view (functional.rs:188-219), with a fused elementwise
 * prologue.  monoid: 0 add, 1 mul, 2 max, 3 min, 4 and, 5 or, 6 xor.  cls: register class of the reduced value
 * (B2xVmClass).  `init_ptr` (device scalar of element type init_elem) is used when non-NULL, else `init_imm`.
 * `scratch` must hold A * b2x_reduce_splits(A,R,B) * B * 4 bytes when that count is > 1.  `host_post` (may be NULL) is a
 * fused consumer: a program over the result's [A * B] elements that receives each finished value (combined with init,
 * rounded to out_elem) as VM_SRC_ACC0 and does all stores itself; `out` is then not written. */
typedef struct {
  int64_t A, R, B;
  uint8_t monoid, cls, out_elem, init_elem;
  uint32_t init_imm;
  const void* init_ptr;
  void* out;
  void* scratch;
  int vec;
  const B2xVmProgram* host_post;
} B2xReduceArgs;
B2X_API int b2x_reduce_splits(int64_t A, int64_t R, int64_t B);
/* Kernels one call of b2x_launch_reduce enqueues for this shape: 1, or 2 for a split column reduction (B > 1). */
B2X_API int b2x_reduce_launches(int64_t A, int64_t R, int64_t B);
B2X_API int b2x_launch_reduce(const B2xVmProgram* host_prologue, const B2xReduceArgs* host_args, b2x_stream_t stream);

/* The same reduction for callers that must not allocate device memory (an embedding runtime that owns the allocator,
 * a serving loop that cannot afford an allocation stall, a process whose free memory is all pooled elsewhere).  This
 * entry point has no counterpart in the reference.  `host_args->scratch` is ignored: partial results go to a fixed
 * array of B2X_REDUCE_NOALLOC_MAX_PARTIALS 32-bit words that is part of the library image (each GPU that loads the
 * library holds those 64 KiB until the process exits).  It calls no cudaMalloc/cudaFree and no allocating routine.
 *   - A reduction that needs more partials (A * b2x_reduce_splits(A,R,B) * B, when the split count is > 1) is refused
 *     with cudaErrorInvalidValue and a message in `err` (may be NULL).
 *   - The first call on each device looks up the array's device address (with that device current); make that call
 *     before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents.  Nothing needs clearing (each call
 *     overwrites every partial it later reads), but two calls whose kernels overlap on the GPU, on any streams, race
 *     on it: order them on one stream or with events. */
#define B2X_REDUCE_NOALLOC_MAX_PARTIALS 16384
B2X_API int b2x_launch_reduce_noalloc(const B2xVmProgram* host_prologue, const B2xReduceArgs* host_args, b2x_stream_t stream, char* err,
                                      size_t err_cap);

/* stablehlo.dot_general (linear_algebra.rs:561-592, 756-797) after normalisation to a strided batched GEMM
 * C[b][m][n] = sum_k A[b][m][k] * B[b][k][n].  Strides are in elements.  The accumulator (f32, or s32 for integer
 * inputs) is handed to `epilogue` as VM_SRC_ACC0; the epilogue's root shape is [batch * M, N] linearised row-major
 * and it performs all stores. */
typedef struct {
  const void* a; const void* b;
  uint8_t elem;              /* B2xElem of both operands */
  int64_t batch, M, N, K;
  int64_t a_batch_stride, a_row_stride, a_k_stride;
  int64_t b_batch_stride, b_row_stride, b_k_stride;
} B2xGemmArgs;
/* CUDA-core kernel: any strides, any supported element type, any size. */
B2X_API int b2x_launch_gemm_simt(const B2xGemmArgs* host_args, const B2xVmProgram* host_epilogue, int vec, b2x_stream_t stream);
/* tcgen05/TMEM kernel for bf16/f16/tf32 operands fed by TMA.  Needs M >= 128, N >= 64, N % 8 == 0, 16-byte aligned
 * bases and strides, and one unit stride per operand.  `status` is a device int32 that receives a non-zero code if a
 * bounded wait inside the kernel expires. */
B2X_API int b2x_launch_gemm_tc(const B2xGemmArgs* host_args, const B2xVmProgram* host_epilogue, int32_t* status, b2x_stream_t stream);
/* Host-only: what b2x_launch_gemm_tc would do for this problem and epilogue program, without touching a device (tests use
 * it to assert that a case runs the same kernel variant as another).  out[0] tile width BN, [1] id of the build-time
 * specialised epilogue (0 = interpreted), [2] epilogue groups (1 or 2), [3] 1 if the multi-store epilogue goes through
 * shared memory (transposed), [4] m-tiles per raster group, [5] m-tiles, [6] n-tiles, [7] k-blocks per tile, [8] stores of
 * the specialised program, [9] CTAs launched, [10] rows of a tile (128, or 256 for the tall tiles of long-K problems),
 * [11] reserved (0). */
B2X_API int b2x_gemm_tc_route(const B2xGemmArgs* host_args, const B2xVmProgram* host_epilogue, int32_t out[12]);
/* Splits f32 operands for the 3xTF32 scheme: writes A' = [hi | hi | lo] and B' = [hi | lo | hi] along K into scratch
 * (K-major rows of 3K elements), so that one TF32 GEMM over K' = 3K yields hi*hi + hi*lo + lo*hi. */
B2X_API int b2x_launch_split_f32(const B2xGemmArgs* host_args, float* a_split, float* b_split, b2x_stream_t stream);

/* Fused causal scaled-dot-product attention forward over [BH, S, D] bf16 (the dot_general -> scale -> iota/compare/
 * select mask -> reduce max -> exponential -> reduce add -> divide -> dot_general chain written with the builders
 * cited above). */
typedef struct {
  const void* q; const void* k; const void* v; void* o;
  int64_t BH, Sq, Sk, D;
  float scale;
  int causal;
} B2xAttentionArgs;
B2X_API int b2x_launch_attention(const B2xAttentionArgs* host_args, int32_t* status, b2x_stream_t stream);

/* Ops over 64-bit element types (i64, ui64, f64; linear_algebra.rs:671-701 and communication.rs:821-841 write the
 * reference's worked examples with i64 tensors).  The fused-elementwise programs above keep values in 32-bit registers,
 * so an op that reads or writes a 64-bit tensor runs as one launch of its own: every operand is addressed through
 * per-dimension element strides (0 = broadcast), one thread per result element, arithmetic in int64 / uint64 / double.
 * The store converts to `out_elem` with StableHLO's convert rules, so B2X_WIDE_COPY also serves convert,
 * broadcast_in_dim and transpose. */
#define B2X_WIDE_MAX_DIMS 6
enum B2xWideOpKind {
  B2X_WIDE_COPY = 0, B2X_WIDE_FILL, B2X_WIDE_IOTA, B2X_WIDE_COMPARE, B2X_WIDE_SELECT, B2X_WIDE_CLAMP,
  B2X_WIDE_ADD, B2X_WIDE_SUB, B2X_WIDE_MUL, B2X_WIDE_DIV, B2X_WIDE_REM, B2X_WIDE_POW, B2X_WIDE_MAX, B2X_WIDE_MIN, B2X_WIDE_AND, B2X_WIDE_OR, B2X_WIDE_XOR,
  B2X_WIDE_NEG, B2X_WIDE_ABS, B2X_WIDE_SIGN, B2X_WIDE_NOT, B2X_WIDE_TANH, B2X_WIDE_EXP, B2X_WIDE_LOG, B2X_WIDE_SQRT, B2X_WIDE_RSQRT, B2X_WIDE_LOGISTIC,
  B2X_WIDE_FLOOR, B2X_WIDE_CEIL, B2X_WIDE_EXPM1, B2X_WIDE_LOG1P, B2X_WIDE_SIN, B2X_WIDE_COS
};
typedef struct {
  int32_t op;                 /* B2xWideOpKind */
  int32_t n_in;               /* operands: 0..3 */
  int32_t n_dims;             /* result dims (row-major result) */
  int32_t aux;                /* IOTA: the dimension; COMPARE: B2xCmp direction */
  int32_t aux2;               /* COMPARE: 0 by operand type, 1 unsigned, 2 signed */
  uint8_t out_elem;           /* B2xElem of the result */
  uint8_t in_elem[3];
  int64_t n_elements;
  int64_t dim[B2X_WIDE_MAX_DIMS];
  int64_t in_stride[3][B2X_WIDE_MAX_DIMS];   /* elements */
  const void* in[3];
  void* out;
  uint64_t imm;               /* FILL: the value's bit pattern in the class of out_elem (int64 / uint64 / double) */
} B2xWideOp;
B2X_API int b2x_launch_wide_elementwise(const B2xWideOp* host_op, b2x_stream_t stream);
/* stablehlo.reduce of the middle extent of a dense [A, R, B] tensor of a 64-bit type (functional.rs:188-219). */
B2X_API int b2x_launch_wide_reduce(const void* in, uint8_t elem, int64_t A, int64_t R, int64_t B, int monoid, const void* init_ptr, uint64_t init_imm,
                                   void* out, b2x_stream_t stream);
/* stablehlo.dot_general over 64-bit operands as a strided batched GEMM (linear_algebra.rs:561-592); `out` is the dense
 * row-major [batch, M, N] result of element type `out_elem`. */
B2X_API int b2x_launch_wide_gemm(const B2xGemmArgs* host_args, uint8_t out_elem, void* out, b2x_stream_t stream);

/* Number of kernels launched through this library since load (all entry points); used by bench reporting. */
B2X_API int64_t b2x_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B2X_KERNELS_H_ */
