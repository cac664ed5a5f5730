// Launch plan: what Client::compile produces from a StableHLO module and what LoadedExecutable::execute replays.
//
// The plan is a flat list of steps over named buffers.  It is device-independent; per-device state (arena memory,
// uploaded constants, communicators) lives in the runtime.  Reference call sites this stands behind:
// PJRT_Client_Compile (crates/ryft-pjrt/src/programs.rs:1245-1263) builds it, PJRT_LoadedExecutable_Execute
// (crates/ryft-pjrt/src/programs.rs:923-936) runs it.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../frontend/ir.h"
#include "../kernels/vm.h"

namespace b2x {

struct BufRef {
  enum Kind : uint8_t { NONE, ARG, TEMP, OUT, CONST } kind = NONE;
  int32_t index = 0;    // ARG: argument number; OUT: output number
  int64_t offset = 0;   // TEMP: byte offset in the arena; CONST: byte offset in the constant pool; ARG/OUT: byte offset
  bool valid() const { return kind != NONE; }
};

enum class StepKind : uint8_t { ELEMENTWISE, REDUCE, GEMM, ATTENTION, ALL_REDUCE, ALL_GATHER, COPY, WIDE };

struct VmBinding {
  B2xVmProgram prog{};             // tensor pointers are null in the plan; bound at launch
  std::vector<BufRef> bufs;        // one per prog.tensors entry
  int vec = 1;                     // elements per thread-iteration (1, 4 or 8)
  int64_t n_elements = 0;          // size of the root shape
};

struct GemmOperand {
  BufRef buf;
  DType dtype = DType::F32;
  int64_t batch_stride = 0, row_stride = 0, k_stride = 0;  // elements; "row" = M for A, N for B
};

struct Step {
  StepKind kind = StepKind::ELEMENTWISE;
  std::string label;   // for plan dumps and profiling ranges
  VmBinding vm;        // ELEMENTWISE: the whole step; REDUCE: prologue; GEMM: epilogue

  // REDUCE: input viewed as [A, R, B], R reduced
  int64_t rA = 1, rR = 1, rB = 1;
  Monoid monoid = Monoid::ADD;
  uint8_t rcls = VM_F32;           // register class of the reduced value
  DType r_out_dtype = DType::F32;
  BufRef r_out;
  bool r_init_is_imm = true;
  uint32_t r_init_imm = 0;
  BufRef r_init_buf;               // device scalar when !r_init_is_imm
  DType r_init_dtype = DType::F32;
  BufRef scratch;                  // REDUCE partials, GEMM f32-split operands
  int64_t scratch_bytes = 0;
  bool has_post = false;           // REDUCE: consumer groups of the result run inside the reduce kernel on each finished value
  VmBinding post;                  // their program: the result arrives as VM_SRC_ACC0, the program does the stores

  // GEMM: C[b][m][n] = sum_k A[b][m][k] * B[b][k][n]; the epilogue program consumes the accumulator
  int64_t gB = 1, gM = 0, gN = 0, gK = 0;
  GemmOperand ga, gb;
  bool g_tensor_core = false;      // tcgen05 path; otherwise the SIMT kernel
  bool g_split_f32 = false;        // f32 operands run as three TF32 products over hi/lo splits held in scratch
  DType g_acc_dtype = DType::F32;

  // ATTENTION: O = softmax(scale * Q K^T + causal mask) V over [batch, heads, seq, head_dim]
  int64_t aBH = 0, aSq = 0, aSk = 0, aD = 0;
  float a_scale = 1.f;
  bool a_causal = false;
  BufRef aq, ak, av, ao;

  // ALL_REDUCE / ALL_GATHER: per operand src -> dst
  struct Coll { BufRef src, dst; int64_t count; DType dtype; int64_t outer = 1, inner = 1; };
  std::vector<Coll> colls;
  std::vector<std::vector<int64_t>> replica_groups;
  int coll_id = -1;                // index among the plan's collective steps (they run on the communication stream)
  std::vector<int> wait_colls;     // collective ids whose completion this step must wait for before it starts
  bool coll_detached = false;      // no step of the plan waits for it and it touches no arena memory: the compute stream
                                   // does not wait for it either, so it overlaps with the next execution

  // COPY
  BufRef c_src, c_dst;
  int64_t c_bytes = 0;

  // 64-bit element types (i64, ui64, f64) do not fit the 32-bit registers of the fused-elementwise programs: an op that
  // reads or writes such a tensor is a step of its own.  WIDE: one elementwise op (or copy / fill / iota) with strided
  // operands; REDUCE and GEMM steps with `wide` set use the 64-bit kernels and the REDUCE / GEMM fields above.
  bool wide = false;
  int w_op = 0;                    // B2xWideOpKind
  int w_aux = 0, w_aux2 = 0;
  int w_n_in = 0;
  DType w_in_dtype[3] = {DType::S64, DType::S64, DType::S64};
  DType w_out_dtype = DType::S64;
  std::vector<int64_t> w_dims;
  std::vector<int64_t> w_in_strides[3];
  BufRef w_in[3], w_out;
  uint64_t w_imm = 0;

  // bookkeeping for cost analysis
  double flops = 0, bytes = 0;
};

struct OutputInfo { TensorType type; };

struct Plan {
  std::string name;
  std::vector<TensorType> arg_types;
  std::vector<OutputInfo> outputs;
  std::vector<Step> steps;
  int64_t arena_bytes = 0;
  int num_collectives = 0;
  bool has_detached_collectives = false;
  // which arguments a detached collective reads or writes, and which outputs it writes: only those have a reader or
  // writer on the communication stream after the compute stream has finished with the execution
  std::vector<char> arg_in_detached, out_in_detached;
  std::vector<uint8_t> const_pool;
  double total_flops = 0, total_bytes = 0;
  int num_replicas = 1, num_partitions = 1;
  bool uses_replica_id = false;
  std::string dump() const;
};

struct PlanOptions {
  int num_replicas = 1;
  int num_partitions = 1;
  bool allow_tensor_core = true;   // B2X_GEMM=simt turns this off (debugging aid)
  bool allow_fused_attention = true;
  bool allow_epilogue_fusion = true;
  int precision = 0;               // Precision::{Default,High,Highest}
  bool precise_math = false;       // B2X_PRECISE_MATH=1: no hardware-approximate tanh/exp/log anywhere (by default they are used
                                   // only for 16-bit float values that are just returned from the program)
};

// Lowers a verified module to a plan.  `replica` is only used to fold stablehlo.replica_id (plans are otherwise
// identical across replicas; the runtime builds one per replica only if the module reads replica_id).
Plan build_plan(const Module& m, const PlanOptions& opt, int replica);

// Number of partial results per output element the reduce kernel will use for an [A, R, B] reduction; the planner
// sizes scratch with it and the launcher uses the same value.
int reduce_splits(int64_t A, int64_t R, int64_t B);
// Kernel launches of one reduce step of that shape (a split column reduction folds its partials with a second launch).
int reduce_launches(int64_t A, int64_t R, int64_t B);

}  // namespace b2x
