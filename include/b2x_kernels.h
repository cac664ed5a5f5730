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
 * the specialised program, [9] CTAs launched. */
B2X_API int b2x_gemm_tc_route(const B2xGemmArgs* host_args, const B2xVmProgram* host_epilogue, int32_t out[10]);
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

/* Number of kernels launched through this library since load (all entry points); used by bench reporting. */
B2X_API int64_t b2x_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B2X_KERNELS_H_ */
