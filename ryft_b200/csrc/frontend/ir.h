// In-memory form of the StableHLO subset the executor accepts.
//
// The input language is what ryft-mlir's builders print (reference:
// crates/ryft-mlir/src/dialects/stable_hlo/operations/*.rs; each op's printed
// form is pinned by a test there).  The module is a single `func.func @main`
// whose arguments are the executable's inputs and whose `return` operands are
// its outputs (reference: crates/ryft-pjrt/src/programs.rs:2492-2498).
#pragma once
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace b2x {

enum class DType : uint8_t { PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, BF16, F32, F64, INVALID };

inline int dtype_size(DType t) {
  switch (t) {
    case DType::PRED: case DType::S8: case DType::U8: return 1;
    case DType::S16: case DType::U16: case DType::F16: case DType::BF16: return 2;
    case DType::S32: case DType::U32: case DType::F32: return 4;
    case DType::S64: case DType::U64: case DType::F64: return 8;
    default: return 0;
  }
}
inline bool dtype_is_float(DType t) { return t == DType::F16 || t == DType::BF16 || t == DType::F32 || t == DType::F64; }
inline bool dtype_is_signed_int(DType t) { return t == DType::S8 || t == DType::S16 || t == DType::S32 || t == DType::S64; }
inline bool dtype_is_unsigned_int(DType t) {
  return t == DType::U8 || t == DType::U16 || t == DType::U32 || t == DType::U64 || t == DType::PRED;
}
const char* dtype_name(DType t);  // MLIR spelling: f32, bf16, i32, ui32, i1 ...

struct TensorType {
  DType dtype = DType::INVALID;
  std::vector<int64_t> dims;
  int rank() const { return (int)dims.size(); }
  int64_t num_elements() const { int64_t n = 1; for (auto d : dims) n *= d; return n; }
  int64_t byte_size() const { return num_elements() * dtype_size(dtype); }
  bool operator==(const TensorType& o) const { return dtype == o.dtype && dims == o.dims; }
  bool operator!=(const TensorType& o) const { return !(*this == o); }
  std::string str() const;
};

enum class OpKind : uint8_t {
  // elementwise, unary
  NEGATE, ABS, TANH, EXP, LOG, SQRT, RSQRT, LOGISTIC, NOT, CONVERT, SIGN, FLOOR, CEIL, EXPM1, LOG1P, SINE, COSINE,
  // elementwise, binary
  ADD, SUBTRACT, MULTIPLY, DIVIDE, MAXIMUM, MINIMUM, POWER, AND, OR, XOR, REMAINDER, COMPARE,
  // elementwise, ternary
  SELECT, CLAMP,
  // sources
  CONSTANT, IOTA, REPLICA_ID, PARTITION_ID,
  // index manipulation
  BROADCAST_IN_DIM, TRANSPOSE, RESHAPE,
  // contraction, reduction, collectives
  DOT_GENERAL, REDUCE, ALL_REDUCE, ALL_GATHER,
  // terminator
  RETURN,
};
const char* op_name(OpKind k);  // "stablehlo.add" ...
bool op_is_elementwise(OpKind k);

enum class CmpDir : uint8_t { EQ, NE, GE, GT, LE, LT };
enum class CmpType : uint8_t { DEFAULT, FLOAT, TOTALORDER, SIGNED, UNSIGNED };
enum class Monoid : uint8_t { ADD, MUL, MAX, MIN, AND, OR, XOR };

struct Op;
struct Value {
  int id = -1;
  TensorType type;
  Op* def = nullptr;  // nullptr for function arguments
  int result_index = 0;
  int arg_index = -1;  // >= 0 for function arguments
  std::string name;    // SSA name as written, for diagnostics
  std::vector<Op*> users;
};

struct Op {
  OpKind kind;
  std::vector<Value*> operands;
  std::vector<Value*> results;
  int line = 0;
  // attributes (only those meaningful for `kind` are set)
  std::vector<int64_t> dims;               // broadcast dims / transpose permutation / reduce dimensions
  int64_t iota_dim = 0;                    // iota; all_gather_dim for ALL_GATHER
  CmpDir cmp_dir = CmpDir::EQ;
  CmpType cmp_type = CmpType::DEFAULT;
  std::vector<int64_t> lhs_batch, rhs_batch, lhs_contract, rhs_contract;  // dot_general
  Monoid monoid = Monoid::ADD;             // reduce / all_reduce body
  std::vector<std::vector<int64_t>> replica_groups;
  bool has_channel = false;
  bool use_global_device_ids = false;
  // constant payload: raw little-endian element bytes; `splat` means one element broadcast to the whole type
  std::vector<uint8_t> const_data;
  bool splat = false;
};

struct Module {
  std::string name = "main";
  std::vector<std::unique_ptr<Value>> values;
  std::vector<std::unique_ptr<Op>> ops;  // topological (program) order; the last one is RETURN
  std::vector<Value*> args;
  std::vector<Value*> outputs;           // operands of RETURN
  std::string source;                    // original text, kept for OptimizedProgram / serialization
  bool has_sharding_attrs = false;       // `sdy.*` / `mhlo.sharding` attributes were seen on the entry function

  Value* new_value(const TensorType& t) {
    values.emplace_back(new Value());
    Value* v = values.back().get();
    v->id = (int)values.size() - 1;
    v->type = t;
    return v;
  }
};

// Thrown by the front end and the planner; `code` is a PJRT_Error_Code value.
struct CompileError : std::runtime_error {
  int code;
  CompileError(int code, const std::string& msg) : std::runtime_error(msg), code(code) {}
};
constexpr int kInvalidArgument = 3;
constexpr int kUnimplemented = 12;
constexpr int kInternal = 13;

// Parses MLIR text (pretty or generic op forms).  Throws CompileError.
std::unique_ptr<Module> parse_module(const std::string& text);

// Exact algebraic rewrites applied before planning (see canonicalize.cc).
void canonicalize(Module& m);

// Shape/dtype verification of every op against StableHLO's rules; fills nothing, throws on violation.
void verify_module(const Module& m);

}  // namespace b2x
