// StableHLO module -> launch plan.
//
// Walks func.func @main in program order and maps every op to a kernel step (reference call site:
// PJRT_Client_Compile, crates/ryft-pjrt/src/programs.rs:1245-1263).  Elementwise ops (and broadcast_in_dim, iota,
// splat constants) are grouped by producer/consumer fusion into accumulator-machine programs (kernels/vm.h); a group
// becomes a standalone elementwise kernel, the prologue of a reduce kernel, or the epilogue of the GEMM that
// produces its input.  transpose/reshape become strided views where the layout allows.  Intermediates live in one
// arena whose offsets are assigned from value lifetimes.
#include "plan.h"

#include "../../../include/b2x_kernels.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>

namespace b2x {
namespace {

[[noreturn]] void unimplemented(const std::string& m) { throw CompileError(kUnimplemented, m); }
[[noreturn]] void internal(const std::string& m) { throw CompileError(kInternal, "planner: " + m); }
// A fusion group that does not fit the accumulator machine (instructions, tensors, temporaries, index dims).  The
// planner answers by cutting the group at an interior value; the message reaches the caller only when no cut exists.
struct GroupTooLarge : CompileError { explicit GroupTooLarge(const std::string& m) : CompileError(kUnimplemented, m) {} };
[[noreturn]] void too_large(const std::string& m) { throw GroupTooLarge(m); }

struct Layout {
  BufRef buf;
  std::vector<int64_t> strides;  // elements per value dim
};
std::vector<int64_t> row_major_strides(const std::vector<int64_t>& dims) {
  std::vector<int64_t> s(dims.size());
  int64_t acc = 1;
  for (int i = (int)dims.size() - 1; i >= 0; i--) { s[i] = acc; acc *= dims[i]; }
  return s;
}
bool is_row_major(const std::vector<int64_t>& dims, const std::vector<int64_t>& strides) {
  int64_t acc = 1;
  for (int i = (int)dims.size() - 1; i >= 0; i--) {
    if (dims[i] != 1 && strides[i] != acc) return false;
    acc *= dims[i];
  }
  return true;
}

struct ClassInfo { uint8_t cls; uint8_t rnd; };
ClassInfo class_of(DType t) {
  switch (t) {
    case DType::F32: return {VM_F32, VM_RN_NONE};
    case DType::BF16: return {VM_F32, VM_RN_BF16};
    case DType::F16: return {VM_F32, VM_RN_F16};
    case DType::S32: return {VM_S32, VM_RN_NONE};
    case DType::S16: return {VM_S32, VM_RN_S16};
    case DType::S8: return {VM_S32, VM_RN_S8};
    case DType::U32: return {VM_U32, VM_RN_NONE};
    case DType::U16: return {VM_U32, VM_RN_U16};
    case DType::U8: return {VM_U32, VM_RN_U8};
    case DType::PRED: return {VM_U32, VM_RN_PRED};
    default:
      unimplemented(std::string("64-bit element type ") + dtype_name(t) + " is not supported in elementwise, reduce or dot_general kernels");
  }
}

float bf16_bits_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
float f16_bits_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else { int e = -1; do { e++; man <<= 1; } while (!(man & 0x400)); u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13); }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f; memcpy(&f, &u, 4); return f;
}
// Converts one stored element to the 32-bit register pattern of its class.
uint32_t element_to_reg(const uint8_t* p, DType t) {
  switch (t) {
    case DType::F32: case DType::S32: case DType::U32: { uint32_t u; memcpy(&u, p, 4); return u; }
    case DType::BF16: { uint16_t h; memcpy(&h, p, 2); return (uint32_t)h << 16; }
    case DType::F16: { uint16_t h; memcpy(&h, p, 2); float f = f16_bits_to_f32(h); uint32_t u; memcpy(&u, &f, 4); return u; }
    case DType::S16: { int16_t h; memcpy(&h, p, 2); return (uint32_t)(int32_t)h; }
    case DType::U16: { uint16_t h; memcpy(&h, p, 2); return h; }
    case DType::S8: return (uint32_t)(int32_t)(int8_t)p[0];
    case DType::U8: return p[0];
    case DType::PRED: return p[0] != 0;
    default: class_of(t); return 0;
  }
}

bool is_wide_type(DType t) { return dtype_size(t) == 8; }
// An op that reads or writes a 64-bit tensor: it runs as a step of its own on the 64-bit kernels.
bool touches_wide(const Op& op) {
  for (auto v : op.operands) if (is_wide_type(v->type.dtype)) return true;
  for (auto v : op.results) if (is_wide_type(v->type.dtype)) return true;
  return false;
}
bool is_fusible_kind(const Op& op) {
  if (touches_wide(op)) return false;
  if (op.kind == OpKind::BROADCAST_IN_DIM) return true;
  if (op.kind == OpKind::CONSTANT) return op.splat;
  if (op.kind == OpKind::RETURN) return false;
  return op_is_elementwise(op.kind);
}
bool is_cheap_kind(OpKind k) {
  return k == OpKind::CONSTANT || k == OpKind::IOTA || k == OpKind::BROADCAST_IN_DIM || k == OpKind::REPLICA_ID ||
         k == OpKind::PARTITION_ID || k == OpKind::COMPARE || k == OpKind::CONVERT;
}

struct ValueState {
  bool fusible = false;      // produced by a fusible op
  bool cheap = false;        // cheap to recompute in every consumer
  bool sink_used = false;    // some consumer needs it in memory
  bool root = false;         // fusible and materialised
  bool dead = false;
  std::set<int> groups;      // consumer groups (ids)
  bool has_layout = false;
  Layout layout;
  int alloc = -1;            // arena allocation id when it owns TEMP memory
  int out_index = -1;        // first module output slot it is written to directly
  bool preassigned = false;  // memory was chosen before its producer ran (in-place collective result)
};

struct Alloc { int64_t bytes; int first, last; int64_t offset = -1; };

struct GNode {
  enum K { OPN, TENSOR, IMM, IOTA, ACC0 } k = OPN;
  const Op* op = nullptr;
  std::vector<int> in;
  DType dtype = DType::F32;
  int tensor = -1;
  uint32_t imm = 0;
  int iota_dim = -1;  // unmerged root dim
  int uses = 0, remaining = 0, temp = -1;
  bool precise = false;
};

class Planner {
 public:
  Planner(const Module& m, const PlanOptions& opt, int replica) : m_(m), opt_(opt), replica_(replica) {}
  Plan run();

 private:
  const Module& m_;
  const PlanOptions& opt_;
  int replica_;
  Plan plan_;
  std::vector<ValueState> vs_;
  std::vector<Alloc> allocs_;
  int n_groups_ = 0;
  std::map<const Op*, int> reduce_group_;           // REDUCE op -> group id
  std::map<const Value*, int> root_group_;          // root value -> group id
  std::vector<const Value*> group_root_;            // group id -> root value (nullptr for reduce groups)
  std::set<int> emitted_groups_;
  std::set<const Op*> skip_ops_;                    // ops swallowed by a fused pattern
  std::map<const Op*, int> op_index_;

  ValueState& st(const Value* v) { return vs_[v->id]; }
  int cur_step() const { return (int)plan_.steps.size(); }

  // ---- arena ------------------------------------------------------------------------------------------------
  BufRef new_temp(int64_t bytes) {
    Alloc a;
    a.bytes = std::max<int64_t>(bytes, 16);
    a.first = a.last = cur_step();
    allocs_.push_back(a);
    BufRef r;
    r.kind = BufRef::TEMP;
    r.index = (int)allocs_.size() - 1;
    return r;
  }
  void touch(const BufRef& b) {
    if (b.kind == BufRef::TEMP) allocs_[b.index].last = std::max(allocs_[b.index].last, cur_step());
  }
  void assign_arena();
  void schedule_collectives();
  void compute_liveness();

  // ---- group building ---------------------------------------------------------------------------------------
  struct TensorUse { BufRef buf; DType dt; std::vector<int64_t> strides; };
  struct GroupBuilder {
    Planner* P;
    std::vector<int64_t> root_dims;
    std::vector<GNode> nodes;
    std::map<std::pair<const Value*, std::vector<int>>, int> memo;
    std::vector<TensorUse> tensors;
    std::set<const Value*> computing;   // values this group computes even though they are materialised
    const Value* acc0_value = nullptr;  // value delivered through VM_SRC_ACC0 (GEMM result)
    struct Out { int node; int tensor; };
    std::vector<Out> outs;
    std::vector<bool> out_terminal;     // per output: the value only leaves the program (no op of the program reads it)
    std::set<int> iota_root_dims;
    std::vector<B2xVmInstr> code;
    std::vector<int> free_temps;
    std::vector<int> dim_to_merged;

    int add_tensor(const BufRef& buf, DType dt, const std::vector<int64_t>& strides) {
      for (size_t i = 0; i < tensors.size(); i++) {
        auto& t = tensors[i];
        if (t.buf.kind == buf.kind && t.buf.index == buf.index && t.buf.offset == buf.offset && t.dt == dt && t.strides == strides) return (int)i;
      }
      tensors.push_back({buf, dt, strides});
      return (int)tensors.size() - 1;
    }
    int node_for(const Value* v, const std::vector<int>& map);
    void add_output(const Value* v, const BufRef& buf);
    VmBinding finish(int final_node);
    void gen(int n);
    void emit(uint8_t op, const GNode* src, int src_node, uint8_t aux, uint8_t tc, uint8_t rnd);
    void emit_src_of(int node, B2xVmInstr* I);
    int alloc_temp();
    void consume(int node);
    bool simple(int n) const { return nodes[n].k != GNode::OPN || nodes[n].temp >= 0; }
  };

  bool load_as_leaf(const Value* v) {
    ValueState& s = st(v);
    if (!s.fusible) return true;
    return s.root && !s.cheap;
  }
  Layout& layout_of(const Value* v) {
    ValueState& s = st(v);
    if (!s.has_layout) internal("value %" + v->name + " has no memory layout where one is needed");
    return s.layout;
  }
  void set_layout(const Value* v, const BufRef& buf, const std::vector<int64_t>& strides) {
    ValueState& s = st(v);
    s.has_layout = true;
    s.layout.buf = buf;
    s.layout.strides = strides;
  }
  // Gives `v` fresh memory: a module output slot when it is returned, arena memory otherwise.
  // When `v` exists only to be all-reduced, the collective runs in place: `v` is produced directly in the buffer of
  // the collective's result (an output buffer when that result is returned).
  const Value* in_place_result(const Value* v) const {
    if (v->users.size() != 1 || v->users[0]->kind != OpKind::ALL_REDUCE) return nullptr;
    for (auto o : m_.outputs) if (o == v) return nullptr;
    const Op* ar = v->users[0];
    int hits = 0;
    const Value* r = nullptr;
    for (size_t i = 0; i < ar->operands.size(); i++) if (ar->operands[i] == v) { hits++; r = ar->results[i]; }
    return hits == 1 ? r : nullptr;
  }
  BufRef materialise(const Value* v) {
    ValueState& s = st(v);
    if (s.has_layout && s.layout.buf.valid() && (s.preassigned || s.alloc >= 0 || s.out_index >= 0)) return s.layout.buf;
    if (const Value* r = in_place_result(v)) {
      BufRef shared = materialise(r);
      st(r).preassigned = true;
      set_layout(v, shared, row_major_strides(v->type.dims));
      return shared;
    }
    BufRef b;
    for (size_t i = 0; i < m_.outputs.size(); i++)
      if (m_.outputs[i] == v) { b.kind = BufRef::OUT; b.index = (int)i; s.out_index = (int)i; break; }
    if (!b.valid()) { b = new_temp(v->type.byte_size()); s.alloc = b.index; }
    set_layout(v, b, row_major_strides(v->type.dims));
    return b;
  }

  void classify();
  struct AttnMatch { const Value* q; const Value* k; const Value* v; float scale; bool causal; };
  std::map<const Op*, AttnMatch> attn_;
  void match_attention();
  void emit_attention(const Op& op, const AttnMatch& m);
  void emit_group_for_root(const Value* v);
  bool collect_consumer_roots(const Op& op, const Value* res, std::vector<const Value*>* fused_roots);
  void force_root(const Value* v);
  const Value* pick_cut(const Value* root);
  void emit_reduce(const Op& op);
  void emit_dot(const Op& op);
  void emit_view_or_copy(const Op& op);
  void emit_wide(const Op& op);
  void emit_wide_copy(const Layout& src, DType src_dt, const std::vector<int64_t>& dims, const BufRef& dst, DType dst_dt, const std::string& label);
  void emit_wide_reduce(const Op& op);
  void emit_collective(const Op& op);
  void emit_outputs();
  BufRef emit_strided_copy(const Layout& src, DType dt, const std::vector<int64_t>& dims, const std::string& label);
  void push_vm_step(VmBinding&& vm, const std::string& label);
  void touch_vm(const VmBinding& vm) { for (auto& b : vm.bufs) touch(b); }
};

// ---- expression DAG -------------------------------------------------------------------------------------------

int Planner::GroupBuilder::node_for(const Value* v, const std::vector<int>& map) {
  auto key = std::make_pair(v, map);
  auto it = memo.find(key);
  if (it != memo.end()) return it->second;
  GNode n;
  n.dtype = v->type.dtype;
  class_of(n.dtype);
  if (v == acc0_value) {
    n.k = GNode::ACC0;
  } else if (!computing.count(v) && P->load_as_leaf(v)) {
    Layout& L = P->layout_of(v);
    std::vector<int64_t> strides(root_dims.size(), 0);
    for (int i = 0; i < v->type.rank(); i++)
      if (map[i] >= 0 && v->type.dims[i] > 1) strides[map[i]] += L.strides[i];
    n.k = GNode::TENSOR;
    n.tensor = add_tensor(L.buf, v->type.dtype, strides);
  } else {
    const Op* op = v->def;
    if (!op) internal("argument reached as a computed node");
    switch (op->kind) {
      case OpKind::CONSTANT:
        n.k = GNode::IMM;
        n.imm = element_to_reg(op->const_data.data(), n.dtype);
        break;
      case OpKind::REPLICA_ID: n.k = GNode::IMM; n.imm = (uint32_t)P->replica_; P->plan_.uses_replica_id = true; break;
      case OpKind::PARTITION_ID: n.k = GNode::IMM; n.imm = 0; break;
      case OpKind::IOTA: {
        int rd = map[op->iota_dim];
        if (rd < 0 || v->type.dims[op->iota_dim] == 1) { n.k = GNode::IMM; n.imm = 0; }
        else { n.k = GNode::IOTA; n.iota_dim = rd; iota_root_dims.insert(rd); }
        break;
      }
      case OpKind::BROADCAST_IN_DIM: {
        const Value* u = op->operands[0];
        std::vector<int> umap(u->type.rank());
        for (int i = 0; i < u->type.rank(); i++) umap[i] = (u->type.dims[i] == 1) ? -1 : map[op->dims[i]];
        int r = node_for(u, umap);
        memo[key] = r;
        return r;
      }
      default: {
        n.k = GNode::OPN;
        n.op = op;
        for (size_t i = 0; i < op->operands.size(); i++) {
          const Value* u = op->operands[i];
          std::vector<int> umap = map;
          if (u->type.rank() == 0 && v->type.rank() != 0) umap.clear();  // scalar pred / clamp bounds
          n.in.push_back(node_for(u, umap));
        }
        break;
      }
    }
  }
  nodes.push_back(n);
  int id = (int)nodes.size() - 1;
  memo[key] = id;
  return id;
}

void Planner::GroupBuilder::add_output(const Value* v, const BufRef& buf) {
  std::vector<int> ident(v->type.rank());
  for (int i = 0; i < v->type.rank(); i++) ident[i] = i;
  int n = node_for(v, ident);
  int t = add_tensor(buf, v->type.dtype, row_major_strides(root_dims));
  outs.push_back({n, t});
  bool terminal = true;
  for (auto u : v->users) if (u->kind != OpKind::RETURN) terminal = false;
  out_terminal.resize(outs.size(), false);
  out_terminal[outs.size() - 1] = terminal;
}

int Planner::GroupBuilder::alloc_temp() {
  if (free_temps.empty()) too_large("an elementwise fusion group needs more than " + std::to_string(B2X_VM_TEMPS) + " live temporaries");
  int t = free_temps.back();
  free_temps.pop_back();
  return t;
}
void Planner::GroupBuilder::consume(int node) {
  GNode& n = nodes[node];
  n.remaining--;
  if (n.remaining <= 0 && n.temp >= 0) { free_temps.push_back(n.temp); n.temp = -1; }
}
void Planner::GroupBuilder::emit_src_of(int node, B2xVmInstr* I) {
  const GNode& n = nodes[node];
  if (n.temp >= 0) { I->src_kind = VM_SRC_TEMP; I->src_idx = (uint8_t)n.temp; return; }
  switch (n.k) {
    case GNode::TENSOR: I->src_kind = VM_SRC_TENSOR; I->src_idx = (uint8_t)n.tensor; break;
    case GNode::IMM: I->src_kind = VM_SRC_IMM; I->imm = n.imm; break;
    case GNode::IOTA: I->src_kind = VM_SRC_IOTA; I->src_idx = (uint8_t)dim_to_merged[n.iota_dim]; break;
    case GNode::ACC0: I->src_kind = VM_SRC_ACC0; break;
    default: internal("operand is not a simple source");
  }
}
void Planner::GroupBuilder::emit(uint8_t op, const GNode*, int src_node, uint8_t aux, uint8_t tc, uint8_t rnd) {
  B2xVmInstr I{};
  I.op = op; I.aux = aux; I.tc = tc; I.rnd = rnd;
  if (src_node >= 0) { emit_src_of(src_node, &I); }
  code.push_back(I);
  if (src_node >= 0) consume(src_node);
}

// Leaves the value of node n in the accumulator.
void Planner::GroupBuilder::gen(int ni) {
  GNode& n = nodes[ni];
  ClassInfo ci = class_of(n.dtype);
  if (simple(ni)) {
    B2xVmInstr I{};
    I.op = VM_LOAD; I.tc = ci.cls;
    emit_src_of(ni, &I);
    // an iota of a narrow float type must carry that type's precision
    if (n.k == GNode::IOTA) I.rnd = ci.rnd;
    code.push_back(I);
    consume(ni);
    return;
  }
  const Op& op = *n.op;
  auto bin = [&](uint8_t fwd, uint8_t rev, uint8_t aux, uint8_t tc, uint8_t rnd) {
    int x = n.in[0], y = n.in[1];
    if (x == y && nodes[x].k == GNode::TENSOR && nodes[x].temp < 0 && !free_temps.empty()) {
      // both operands are the same tensor element (x * x): fetch it once
      gen(x);
      int t = alloc_temp();
      B2xVmInstr S{}; S.op = VM_SAVE; S.aux = (uint8_t)t; code.push_back(S);
      B2xVmInstr I{}; I.op = fwd; I.aux = aux; I.tc = tc; I.rnd = rnd; I.src_kind = VM_SRC_TEMP; I.src_idx = (uint8_t)t;
      code.push_back(I);
      free_temps.push_back(t);
      consume(y);
      return;
    }
    if (simple(y)) { gen(x); emit(fwd, nullptr, y, aux, tc, rnd); }
    else if (simple(x)) { gen(y); emit(rev, nullptr, x, aux, tc, rnd); }
    else {
      gen(y);
      if (nodes[y].temp >= 0) {
        // y was kept for its other uses; hold one more use so that it survives the evaluation of x
        nodes[y].remaining++;
        gen(x);
        emit(fwd, nullptr, y, aux, tc, rnd);
      } else {
        int t = alloc_temp();
        B2xVmInstr S{}; S.op = VM_SAVE; S.aux = (uint8_t)t; code.push_back(S);
        gen(x);
        B2xVmInstr I{}; I.op = fwd; I.aux = aux; I.tc = tc; I.rnd = rnd; I.src_kind = VM_SRC_TEMP; I.src_idx = (uint8_t)t;
        code.push_back(I);
        free_temps.push_back(t);
      }
    }
  };
  auto un = [&](uint8_t vop, uint8_t aux) { gen(n.in[0]); emit(vop, nullptr, -1, aux, ci.cls, ci.rnd); };
  // Hardware-approximate tanh/exp/log (about 2^-11 relative error) only where the value is rounded to a 16-bit float
  // and then only returned from the program: the approximation stays below that type's rounding step and nothing
  // downstream can amplify it.  Everything that another op reads is computed accurately.
  const uint8_t fast = (n.precise || P->opt_.precise_math) ? 0 : 1;
  switch (op.kind) {
    case OpKind::ADD: bin(VM_ADD, VM_ADD, 0, ci.cls, ci.rnd); break;
    case OpKind::MULTIPLY: bin(VM_MUL, VM_MUL, 0, ci.cls, ci.rnd); break;
    case OpKind::MAXIMUM: bin(VM_MAX, VM_MAX, 0, ci.cls, ci.rnd); break;
    case OpKind::MINIMUM: bin(VM_MIN, VM_MIN, 0, ci.cls, ci.rnd); break;
    case OpKind::AND: bin(VM_AND, VM_AND, 0, ci.cls, ci.rnd); break;
    case OpKind::OR: bin(VM_OR, VM_OR, 0, ci.cls, ci.rnd); break;
    case OpKind::XOR: bin(VM_XOR, VM_XOR, 0, ci.cls, ci.rnd); break;
    case OpKind::SUBTRACT: bin(VM_SUB, VM_RSUB, 0, ci.cls, ci.rnd); break;
    case OpKind::DIVIDE: bin(VM_DIV, VM_RDIV, 0, ci.cls, ci.rnd); break;
    case OpKind::POWER: bin(VM_POW, VM_RPOW, 0, ci.cls, ci.rnd); break;
    case OpKind::REMAINDER: bin(VM_REM, VM_RREM, 0, ci.cls, ci.rnd); break;
    case OpKind::COMPARE: {
      DType ot = op.operands[0]->type.dtype;
      uint8_t oc = class_of(ot).cls;
      if (op.cmp_type == CmpType::UNSIGNED) oc = VM_U32;
      if (op.cmp_type == CmpType::SIGNED && oc == VM_U32 && ot != DType::PRED) oc = VM_S32;
      bin(VM_CMP, VM_RCMP, (uint8_t)op.cmp_dir, oc, VM_RN_NONE);
      break;
    }
    case OpKind::NEGATE: un(VM_NEG, 0); break;
    case OpKind::ABS: un(VM_ABS, 0); break;
    case OpKind::TANH: un(VM_TANH, fast); break;
    case OpKind::EXP: un(VM_EXP, fast); break;
    case OpKind::LOG: un(VM_LOG, fast); break;
    case OpKind::SQRT: un(VM_SQRT, 0); break;
    case OpKind::RSQRT: un(VM_RSQRT, 0); break;
    case OpKind::LOGISTIC: un(VM_LOGISTIC, fast); break;
    case OpKind::NOT: un(VM_NOT, 0); break;
    case OpKind::SIGN: un(VM_SIGN, 0); break;
    case OpKind::FLOOR: un(VM_FLOOR, 0); break;
    case OpKind::CEIL: un(VM_CEIL, 0); break;
    case OpKind::EXPM1: un(VM_EXPM1, 0); break;
    case OpKind::LOG1P: un(VM_LOG1P, 0); break;
    case OpKind::SINE: un(VM_SIN, 0); break;
    case OpKind::COSINE: un(VM_COS, 0); break;
    case OpKind::CONVERT: {
      ClassInfo from = class_of(op.operands[0]->type.dtype);
      gen(n.in[0]);
      if (from.cls == ci.cls && (ci.rnd == VM_RN_NONE || ci.rnd == from.rnd) && !(ci.rnd == VM_RN_PRED)) break;  // no-op widening
      emit(VM_CVT, nullptr, -1, from.cls, ci.cls, ci.rnd);
      break;
    }
    case OpKind::SELECT: {
      int p = n.in[0], a = n.in[1], b = n.in[2];
      int tp;
      bool own_tp = false;
      if (nodes[p].temp >= 0) { tp = nodes[p].temp; }
      else { gen(p); tp = alloc_temp(); own_tp = true; B2xVmInstr S{}; S.op = VM_SAVE; S.aux = (uint8_t)tp; code.push_back(S); }
      if (simple(b)) { gen(a); emit(VM_SELECT, nullptr, b, (uint8_t)tp, ci.cls, VM_RN_NONE); }
      else if (simple(a)) { gen(b); emit(VM_RSELECT, nullptr, a, (uint8_t)tp, ci.cls, VM_RN_NONE); }
      else {
        gen(b);
        int tb = alloc_temp();
        B2xVmInstr S{}; S.op = VM_SAVE; S.aux = (uint8_t)tb; code.push_back(S);
        gen(a);
        B2xVmInstr I{}; I.op = VM_SELECT; I.aux = (uint8_t)tp; I.tc = ci.cls; I.src_kind = VM_SRC_TEMP; I.src_idx = (uint8_t)tb;
        code.push_back(I);
        free_temps.push_back(tb);
      }
      if (own_tp) free_temps.push_back(tp); else consume(p);
      break;
    }
    case OpKind::CLAMP: {  // min(max(x, lo), hi)
      int lo = n.in[0], x = n.in[1], hi = n.in[2];
      auto as_src = [&](int node, uint8_t vop) {
        if (simple(node)) { emit(vop, nullptr, node, 0, ci.cls, ci.rnd); return; }
        int t = alloc_temp();
        B2xVmInstr S{}; S.op = VM_SAVE; S.aux = (uint8_t)t; code.push_back(S);   // park x
        gen(node);
        B2xVmInstr I{}; I.op = vop; I.tc = ci.cls; I.rnd = ci.rnd; I.src_kind = VM_SRC_TEMP; I.src_idx = (uint8_t)t;
        code.push_back(I);
        free_temps.push_back(t);
      };
      gen(x);
      as_src(lo, VM_MAX);
      as_src(hi, VM_MIN);
      break;
    }
    default: internal(std::string("no code generation for ") + op_name(op.kind));
  }
  // keep a value with further uses in a temporary
  GNode& n2 = nodes[ni];
  n2.remaining--;
  if (n2.remaining > 0) {
    int t = alloc_temp();
    B2xVmInstr S{}; S.op = VM_SAVE; S.aux = (uint8_t)t; code.push_back(S);
    n2.temp = t;
  }
}

// final_node >= 0: leave that node's value in the accumulator at the end (reduce prologue).
VmBinding Planner::GroupBuilder::finish(int final_node) {
  const int nd = (int)root_dims.size();
  // ---- merge adjacent root dims that every tensor walks as one strided run ----
  std::vector<int64_t> mdims;
  std::vector<std::vector<int64_t>> mstr(tensors.size());
  dim_to_merged.assign(nd, 0);
  bool group_has_iota = false;
  for (int d = 0; d < nd; d++) {
    const int64_t size = root_dims[d];
    if (size == 1) { dim_to_merged[d] = std::max(0, (int)mdims.size() - 1); continue; }  // coordinate is always 0
    const bool iota = iota_root_dims.count(d) != 0;
    bool can = !mdims.empty() && !iota && !group_has_iota;
    for (size_t t = 0; t < tensors.size() && can; t++)
      if (mstr[t].back() != tensors[t].strides[d] * size) can = false;
    if (can) {
      mdims.back() *= size;
      for (size_t t = 0; t < tensors.size(); t++) mstr[t].back() = tensors[t].strides[d];
    } else {
      mdims.push_back(size);
      for (size_t t = 0; t < tensors.size(); t++) mstr[t].push_back(tensors[t].strides[d]);
      group_has_iota = iota;
    }
    dim_to_merged[d] = (int)mdims.size() - 1;
  }
  if (mdims.empty()) { mdims.push_back(1); for (auto& s : mstr) s.push_back(0); }
  if ((int)mdims.size() > B2X_VM_MAX_DIMS)
    too_large("an elementwise fusion group needs more than " + std::to_string(B2X_VM_MAX_DIMS) + " index dimensions after merging");
  if ((int)tensors.size() > B2X_VM_MAX_TENSORS)
    too_large("an elementwise fusion group touches more than " + std::to_string(B2X_VM_MAX_TENSORS) + " tensors");

  // ---- use counts, precision marks ----
  for (auto& n : nodes) for (int i : n.in) nodes[i].uses++;
  for (auto& o : outs) nodes[o.node].uses++;
  if (final_node >= 0) nodes[final_node].uses++;
  for (auto& n : nodes) n.remaining = n.uses;
  for (size_t oi = 0; oi < outs.size(); oi++) {
    DType t = nodes[outs[oi].node].dtype;
    const bool terminal = oi < out_terminal.size() && out_terminal[oi];
    if ((t != DType::BF16 && t != DType::F16) || !terminal) nodes[outs[oi].node].precise = true;
  }
  if (final_node >= 0) nodes[final_node].precise = true;
  for (int i = (int)nodes.size() - 1; i >= 0; i--) {
    GNode& n = nodes[i];
    if (!n.precise || n.k != GNode::OPN) continue;
    for (int j : n.in) nodes[j].precise = true;
  }

  // ---- code ----
  for (int t = B2X_VM_TEMPS - 1; t >= 0; t--) free_temps.push_back(t);
  for (size_t i = 0; i < outs.size(); i++) {
    gen(outs[i].node);
    B2xVmInstr I{};
    I.op = VM_STORE; I.src_kind = VM_SRC_TENSOR; I.src_idx = (uint8_t)outs[i].tensor;
    code.push_back(I);
  }
  if (final_node >= 0) gen(final_node);
  // A store into a 16-bit float tensor rounds to nearest-even itself: the rounding step of the instruction before it is
  // redundant when the accumulator is overwritten right after the store.
  for (size_t i = 1; i < code.size(); i++) {
    if (code[i].op != VM_STORE) continue;
    const bool acc_dead = (i + 1 == code.size() && final_node < 0) || (i + 1 < code.size() && code[i + 1].op == VM_LOAD);
    if (!acc_dead) continue;
    B2xVmInstr& prev = code[i - 1];
    if (prev.op == VM_STORE || prev.op == VM_SAVE || prev.op == VM_SELECT || prev.op == VM_RSELECT) continue;
    const DType elem = tensors[code[i].src_idx].dt;
    if ((elem == DType::BF16 && prev.rnd == VM_RN_BF16) || (elem == DType::F16 && prev.rnd == VM_RN_F16)) prev.rnd = VM_RN_NONE;
  }
  if ((int)code.size() > B2X_VM_MAX_INSTR)
    too_large("an elementwise fusion group compiles to " + std::to_string(code.size()) + " instructions; the limit is " + std::to_string(B2X_VM_MAX_INSTR));

  VmBinding vb;
  B2xVmProgram& pr = vb.prog;
  memset(&pr, 0, sizeof(pr));
  pr.n_instr = (int)code.size();
  pr.n_tensors = (int)tensors.size();
  pr.n_dims = (int)mdims.size();
  vb.n_elements = 1;
  for (size_t d = 0; d < mdims.size(); d++) { pr.dim[d] = mdims[d]; vb.n_elements *= mdims[d]; }
  for (size_t t = 0; t < tensors.size(); t++) {
    pr.tensors[t].elem = (uint8_t)tensors[t].dt;
    for (size_t d = 0; d < mdims.size(); d++) pr.tensors[t].stride[d] = mstr[t][d];
    vb.bufs.push_back(tensors[t].buf);
  }
  for (size_t i = 0; i < code.size(); i++) pr.code[i] = code[i];
  int64_t inner = mdims.back();
  vb.vec = (inner % 8 == 0) ? 8 : (inner % 4 == 0 ? 4 : 1);
  return vb;
}

// ---- fused attention pattern ------------------------------------------------------------------------------------------
// Recognises, ending at the second dot_general:
//   S = dot_general(Q, K) over the last dim, leading dims batched;  [S = S * splat(c)];
//   [S = select(broadcast(compare GE (iota rows, iota cols)), S, splat(-inf))];
//   M = reduce max over the last dim; E = exp(S - broadcast(M)); L = reduce add(E); P = E / broadcast(L); [convert];
//   O = dot_general(P, V) contracting P's last dim with V's key dim.
// Every intermediate must have no user outside the pattern.
void Planner::match_attention() {
  if (!opt_.allow_fused_attention) return;
  auto users_are = [&](const Value* v, std::initializer_list<const Op*> ops) {
    for (auto o : m_.outputs) if (o == v) return false;
    for (auto u : v->users) { bool in = false; for (auto o : ops) if (u == o) in = true; if (!in) return false; }
    return !v->users.empty();
  };
  auto op_of = [&](const Value* v, OpKind k) -> const Op* { return (v->def && v->def->kind == k) ? v->def : nullptr; };
  std::function<bool(const Value*, float*)> splat_f32 = [&](const Value* v, float* out) -> bool {
    if (!v->def) return false;
    if (v->def->kind == OpKind::CONSTANT && v->def->splat && v->type.dtype == DType::F32) { memcpy(out, v->def->const_data.data(), 4); return true; }
    if (v->def->kind == OpKind::BROADCAST_IN_DIM && v->def->operands[0]->type.num_elements() == 1) return splat_f32(v->def->operands[0], out);
    return false;
  };
  auto last_dim_bcast = [&](const Value* v) -> const Value* {   // broadcast of [..., S] to [..., S, T] along all leading dims
    const Op* b = op_of(v, OpKind::BROADCAST_IN_DIM);
    if (!b) return nullptr;
    const Value* u = b->operands[0];
    if (u->type.rank() != v->type.rank() - 1) return nullptr;
    for (int i = 0; i < u->type.rank(); i++) if (b->dims[i] != i || u->type.dims[i] != v->type.dims[i]) return nullptr;
    return u;
  };
  for (auto& up : m_.ops) {
    const Op& d2 = *up;
    if (d2.kind != OpKind::DOT_GENERAL) continue;
    const Value* pv = d2.operands[0];
    const Value* vv = d2.operands[1];
    const int r = pv->type.rank();
    if (r < 2 || vv->type.rank() != r || d2.results[0]->type.dtype != DType::BF16 || vv->type.dtype != DType::BF16) continue;
    std::vector<int64_t> lead;
    for (int i = 0; i < r - 2; i++) lead.push_back(i);
    if (d2.lhs_batch != lead || d2.rhs_batch != lead || d2.lhs_contract != std::vector<int64_t>{r - 1} || d2.rhs_contract != std::vector<int64_t>{r - 2}) continue;
    std::vector<const Op*> chain;
    const Op* cvt = op_of(pv, OpKind::CONVERT);
    const Value* pf = pv;
    if (cvt) { if (!users_are(pv, {&d2}) || pv->type.dtype != DType::BF16) continue; chain.push_back(cvt); pf = cvt->operands[0]; }
    else continue;   // P must reach the second product in bf16
    const Op* div = op_of(pf, OpKind::DIVIDE);
    if (!div || !users_are(pf, {cvt}) || pf->type.dtype != DType::F32) continue;
    const Value* e = div->operands[0];
    const Value* lsrc = last_dim_bcast(div->operands[1]);
    if (!lsrc || !users_are(div->operands[1], {div})) continue;
    const Op* lred = op_of(lsrc, OpKind::REDUCE);
    if (!lred || lred->monoid != Monoid::ADD || lred->operands[0] != e || lred->dims != std::vector<int64_t>{r - 1} || !users_are(lsrc, {div->operands[1]->def})) continue;
    float init = 1.f;
    if (!splat_f32(lred->operands[1], &init) || init != 0.f) continue;
    const Op* ex = op_of(e, OpKind::EXP);
    if (!ex || !users_are(e, {div, lred})) continue;
    const Op* sub = op_of(ex->operands[0], OpKind::SUBTRACT);
    if (!sub || !users_are(ex->operands[0], {ex})) continue;
    const Value* x = sub->operands[0];
    const Value* msrc = last_dim_bcast(sub->operands[1]);
    if (!msrc || !users_are(sub->operands[1], {sub})) continue;
    const Op* mred = op_of(msrc, OpKind::REDUCE);
    if (!mred || mred->monoid != Monoid::MAX || mred->operands[0] != x || mred->dims != std::vector<int64_t>{r - 1} || !users_are(msrc, {sub->operands[1]->def})) continue;
    if (!splat_f32(mred->operands[1], &init) || !(init == -INFINITY)) continue;
    if (!users_are(x, {sub, mred})) continue;
    chain.insert(chain.end(), {div, div->operands[1]->def, lred, ex, sub, sub->operands[1]->def, mred});
    // optional causal mask
    bool causal = false;
    const Value* y = x;
    if (const Op* sel = op_of(x, OpKind::SELECT)) {
      float ninf = 0.f;
      if (!splat_f32(sel->operands[2], &ninf) || !(ninf == -INFINITY)) continue;
      const Op* mb = op_of(sel->operands[0], OpKind::BROADCAST_IN_DIM);
      if (!mb || mb->dims != std::vector<int64_t>{r - 2, r - 1}) continue;
      const Op* cmp = op_of(mb->operands[0], OpKind::COMPARE);
      if (!cmp || cmp->cmp_dir != CmpDir::GE) continue;
      const Op* i0 = op_of(cmp->operands[0], OpKind::IOTA);
      const Op* i1 = op_of(cmp->operands[1], OpKind::IOTA);
      if (!i0 || !i1 || i0->iota_dim != 0 || i1->iota_dim != 1 || !dtype_is_signed_int(i0->results[0]->type.dtype)) continue;
      causal = true;
      y = sel->operands[1];
      chain.push_back(sel);
      if (!users_are(y, {sel})) continue;
    }
    float scale = 1.f;
    const Value* sdot = y;
    if (const Op* mul = op_of(y, OpKind::MULTIPLY)) {
      float c = 0.f;
      if (splat_f32(mul->operands[1], &c)) sdot = mul->operands[0];
      else if (splat_f32(mul->operands[0], &c)) sdot = mul->operands[1];
      else continue;
      if (!(c > 0.f)) continue;
      scale = c;
      chain.push_back(mul);
      if (!users_are(sdot, {mul})) continue;
    }
    const Op* d1 = op_of(sdot, OpKind::DOT_GENERAL);
    if (!d1 || sdot->type.dtype != DType::F32) continue;
    const Value* q = d1->operands[0];
    const Value* k = d1->operands[1];
    if (q->type.rank() != r || k->type.rank() != r || q->type.dtype != DType::BF16 || k->type.dtype != DType::BF16) continue;
    if (d1->lhs_batch != lead || d1->rhs_batch != lead || d1->lhs_contract != std::vector<int64_t>{r - 1} || d1->rhs_contract != std::vector<int64_t>{r - 1}) continue;
    const int64_t D = q->type.dims[r - 1];
    if ((D != 64 && D != 128) || vv->type.dims[r - 1] != D || vv->type.dims[r - 2] != k->type.dims[r - 2]) continue;
    chain.push_back(d1);
    for (auto c : chain) skip_ops_.insert(c);
    attn_[&d2] = AttnMatch{q, k, vv, scale, causal};
  }
}

void Planner::emit_attention(const Op& op, const AttnMatch& m) {
  const Value* res = op.results[0];
  auto contiguous = [&](const Value* v) -> BufRef {
    Layout L = layout_of(v);
    if (!is_row_major(v->type.dims, L.strides)) {
      L.buf = emit_strided_copy(L, v->type.dtype, v->type.dims, "copy:attention_operand");
    }
    return L.buf;
  };
  Step s;
  s.kind = StepKind::ATTENTION;
  s.label = "attention:%" + res->name;
  const int r = m.q->type.rank();
  s.aBH = 1;
  for (int i = 0; i < r - 2; i++) s.aBH *= m.q->type.dims[i];
  s.aSq = m.q->type.dims[r - 2];
  s.aSk = m.k->type.dims[r - 2];
  s.aD = m.q->type.dims[r - 1];
  s.a_scale = m.scale;
  s.a_causal = m.causal;
  s.aq = contiguous(m.q); s.ak = contiguous(m.k); s.av = contiguous(m.v);
  s.ao = materialise(res);
  double pairs = m.causal ? 0.0 : (double)s.aSq * (double)s.aSk;
  if (m.causal) for (int64_t i = 0; i < s.aSq; i++) pairs += (double)std::min<int64_t>(i + 1, s.aSk);
  s.flops = 4.0 * (double)s.aBH * (double)s.aD * pairs;
  s.bytes = (double)m.q->type.byte_size() + (double)m.k->type.byte_size() + (double)m.v->type.byte_size() + (double)res->type.byte_size();
  plan_.steps.push_back(std::move(s));
}

// ---- classification ---------------------------------------------------------------------------------------------

void Planner::classify() {
  vs_.assign(m_.values.size(), ValueState());
  for (size_t i = 0; i < m_.ops.size(); i++) op_index_[m_.ops[i].get()] = (int)i;
  // forward: fusible / cheap
  for (auto& up : m_.ops) {
    const Op& op = *up;
    if (!is_fusible_kind(op)) continue;
    for (auto r : op.results) {
      ValueState& s = st(r);
      s.fusible = true;
      bool cheap = is_cheap_kind(op.kind);
      for (auto u : op.operands) if (st(u).fusible && !st(u).cheap) cheap = false;
      // a cheap op over a materialised tensor of its own size is a real memory pass: keep it single
      if (cheap && (op.kind == OpKind::CONVERT || op.kind == OpKind::COMPARE))
        for (auto u : op.operands) if (!st(u).fusible && u->type.num_elements() > 1) cheap = false;
      s.cheap = cheap;
    }
  }
  auto sink = [&](const Value* v) { if (st(v).fusible) st(v).sink_used = true; };
  // A narrowing convert applied directly to a kernel result (e.g. f32 accumulator -> bf16) is the cheapest place
  // to cut: keep the narrow tensor in memory rather than the wide one.
  for (auto& up : m_.ops) {
    const Op& op = *up;
    if (op.kind != OpKind::CONVERT) continue;
    const Value* u = op.operands[0];
    if (!st(u).fusible && u->def && u->def->kind == OpKind::DOT_GENERAL && dtype_size(op.results[0]->type.dtype) < dtype_size(u->type.dtype) &&
        !op.results[0]->users.empty())
      st(op.results[0]).sink_used = true;
  }
  for (int i = (int)m_.ops.size() - 1; i >= 0; i--) {
    const Op& op = *m_.ops[i];
    if (op.kind == OpKind::RETURN) { for (auto v : op.operands) sink(v); continue; }
    if (is_fusible_kind(op)) {
      const Value* v = op.results[0];
      ValueState& s = st(v);
      if (s.sink_used || (s.groups.size() >= 2 && !s.cheap)) {
        s.root = true;
        int g = n_groups_++;
        group_root_.push_back(v);
        root_group_[v] = g;
        if (!s.cheap) s.groups.clear();
        s.groups.insert(g);
      }
      if (s.groups.empty()) { s.dead = true; continue; }
      for (auto u : op.operands) st(u).groups.insert(s.groups.begin(), s.groups.end());
      continue;
    }
    switch (op.kind) {
      case OpKind::REDUCE: {
        int g = n_groups_++;
        group_root_.push_back(nullptr);
        reduce_group_[&op] = g;
        st(op.operands[0]).groups.insert(g);
        const Value* init = op.operands[1];
        bool imm = init->def && init->def->kind == OpKind::CONSTANT && init->def->splat;
        if (!imm) sink(init);
        break;
      }
      default:
        for (auto v : op.operands) sink(v);
        break;
    }
  }
}

void Planner::push_vm_step(VmBinding&& vm, const std::string& label) {
  Step s;
  s.kind = StepKind::ELEMENTWISE;
  s.label = label;
  s.vm = std::move(vm);
  for (int t = 0; t < s.vm.prog.n_tensors; t++) {
    // a tensor contributes the elements it actually spans: broadcast dims are not re-read from HBM
    double n = 1;
    for (int d = 0; d < s.vm.prog.n_dims; d++) if (s.vm.prog.tensors[t].stride[d] != 0) n *= (double)s.vm.prog.dim[d];
    s.bytes += n * dtype_size((DType)s.vm.prog.tensors[t].elem);
  }
  touch_vm(s.vm);
  plan_.steps.push_back(std::move(s));
}

// Makes an interior value of a group a root of its own, after classification: it is then computed by a group of its
// own and its former group loads it from memory.
void Planner::force_root(const Value* v) {
  ValueState& s = st(v);
  s.root = true;
  const int g = n_groups_++;
  group_root_.push_back(v);
  root_group_[v] = g;
  s.groups.clear();
  s.groups.insert(g);
}

// Where to cut a group that is too large: the interior value (computed by the group, not cheap, so that it becomes a
// leaf once it is a root) whose expression holds closest to half of the group's ops.  nullptr when there is none.
const Value* Planner::pick_cut(const Value* root) {
  std::map<const Value*, int64_t> ops;   // ops evaluated below a value, counted as a tree
  std::function<int64_t(const Value*)> count = [&](const Value* v) -> int64_t {
    if (v != root && load_as_leaf(v)) return 0;
    if (!v->def) return 0;
    auto it = ops.find(v);
    if (it != ops.end()) return it->second;
    int64_t n = 1;
    for (auto u : v->def->operands) n += count(u);
    n = std::min<int64_t>(n, 1 << 20);
    ops[v] = n;
    return n;
  };
  const int64_t total = count(root);
  const Value* best = nullptr;
  int64_t best_dist = 0;
  for (auto& kv : ops) {
    const Value* v = kv.first;
    if (v == root || st(v).cheap || !st(v).fusible || kv.second < 2) continue;
    const int64_t dist = std::llabs(2 * kv.second - total);
    if (!best || dist < best_dist || (dist == best_dist && v->id < best->id)) { best = v; best_dist = dist; }
  }
  return best;
}

void Planner::emit_group_for_root(const Value* v) {
  int g = root_group_[v];
  if (emitted_groups_.count(g)) return;
  emitted_groups_.insert(g);
  BufRef out = materialise(v);
  for (;;) {
    GroupBuilder gb;
    gb.P = this;
    gb.root_dims = v->type.dims;
    gb.computing.insert(v);
    try {
      gb.add_output(v, out);
      VmBinding vb = gb.finish(-1);
      push_vm_step(std::move(vb), std::string("fused:") + op_name(v->def->kind) + ":%" + v->name);
      return;
    } catch (const GroupTooLarge&) {
      const Value* cut = pick_cut(v);
      if (!cut) throw;
      force_root(cut);
      emit_group_for_root(cut);   // may cut again below
    }
  }
}

int reduce_splits_impl(int64_t A, int64_t R, int64_t B) {
  // Enough independent pieces to fill the machine in one wave of four resident CTAs per SM without starving each piece
  // of work.  Must agree with b2x_reduce_splits of the kernel library.
  int64_t outputs = A * std::max<int64_t>(1, (B + 255) / 256);
  if (outputs <= 0 || outputs >= 296 || R < 4096) return 1;   // an empty result has nothing to split
  int64_t s = std::min<int64_t>((592 + outputs - 1) / outputs, R / 2048);
  return (int)std::max<int64_t>(1, std::min<int64_t>(s, 4096));
}

void Planner::emit_reduce(const Op& op) {
  if (is_wide_type(op.operands[0]->type.dtype)) { emit_wide_reduce(op); return; }
  const Value* x = op.operands[0];
  const Value* init = op.operands[1];
  const Value* res = op.results[0];
  ClassInfo ci = class_of(x->type.dtype);
  // maximal runs of adjacent reduced dims, innermost run first
  std::vector<int64_t> rd = op.dims;
  std::sort(rd.begin(), rd.end());
  std::vector<std::pair<int, int>> runs;  // [lo, hi] in the current shape
  std::vector<int64_t> shape = x->type.dims;
  if (rd.empty()) {  // nothing reduced: behaves like a copy combined with init
    runs.push_back({(int)shape.size(), (int)shape.size() - 1});
  } else {
    size_t i = 0;
    while (i < rd.size()) { size_t j = i; while (j + 1 < rd.size() && rd[j + 1] == rd[j] + 1) j++; runs.push_back({(int)rd[i], (int)rd[j]}); i = j + 1; }
    std::reverse(runs.begin(), runs.end());
  }
  bool init_imm = init->def && init->def->kind == OpKind::CONSTANT && init->def->splat;
  static const DType cls_dtype[3] = {DType::F32, DType::S32, DType::U32};

  BufRef cur_buf;                    // input of the current pass when it is an intermediate
  bool first = true;
  for (size_t p = 0; p < runs.size(); p++) {
    bool last = (p + 1 == runs.size());
    int lo = runs[p].first, hi = runs[p].second;
    int64_t A = 1, R = 1, B = 1;
    for (int d = 0; d < (int)shape.size(); d++) { if (d < lo) A *= shape[d]; else if (d <= hi) R *= shape[d]; else B *= shape[d]; }
    Step s;
    s.kind = StepKind::REDUCE;
    s.label = std::string("reduce:%") + res->name + (runs.size() > 1 ? ":pass" + std::to_string(p) : "");
    s.rA = A; s.rR = R; s.rB = B;
    s.monoid = op.monoid;
    s.rcls = ci.cls;
    GroupBuilder gb;
    gb.P = this;
    gb.root_dims = shape;
    int final_node;
    if (first) {
      std::vector<int> ident(x->type.rank());
      for (int i = 0; i < x->type.rank(); i++) ident[i] = i;
      final_node = gb.node_for(x, ident);
    } else {
      GNode n;
      n.k = GNode::TENSOR;
      n.dtype = cls_dtype[ci.cls];
      n.tensor = gb.add_tensor(cur_buf, n.dtype, row_major_strides(shape));
      gb.nodes.push_back(n);
      final_node = 0;
    }
    try {
      s.vm = gb.finish(final_node);
    } catch (const GroupTooLarge&) {
      // the producing chain does not fit into the prologue: compute the reduced tensor (or part of its chain) with
      // groups of its own and read it back
      if (!first || load_as_leaf(x) || st(x).cheap) throw;
      const Value* cut = pick_cut(x);
      if (!cut) { cut = x; }
      force_root(cut);
      emit_group_for_root(cut);
      p--;
      continue;
    }
    // vectors run along R for row reductions and along B otherwise; they must not straddle a row
    {
      int64_t along = (B == 1) ? R : B;
      s.vm.vec = (along % 8 == 0) ? 8 : (along % 4 == 0 ? 4 : 1);
    }
    if (last) {
      s.r_out_dtype = res->type.dtype;
      // Consumer groups of a small result run inside the reduce kernel, on each finished value (e.g. the scaling of a
      // loss): no second launch, no round trip of the result through memory.
      std::vector<const Value*> fused_roots;
      bool res_needs_memory = true;
      if (A * B <= 4096) res_needs_memory = collect_consumer_roots(op, res, &fused_roots);
      while (!fused_roots.empty()) {
        GroupBuilder pb;
        pb.P = this;
        pb.root_dims = res->type.dims;
        pb.acc0_value = res;
        try {
          if (res_needs_memory) pb.add_output(res, materialise(res));
          for (auto r : fused_roots) pb.computing.insert(r);
          for (auto r : fused_roots) pb.add_output(r, materialise(r));
          s.post = pb.finish(-1);
          s.has_post = true;
          break;
        } catch (const GroupTooLarge&) {
          fused_roots.clear();
        }
      }
      if (s.has_post) {
        for (auto r : fused_roots) emitted_groups_.insert(root_group_[r]);
        s.label += "+epilogue(";
        for (auto r : fused_roots) s.label += "%" + r->name + " ";
        s.label += ")";
        touch_vm(s.post);
        if (res_needs_memory) s.r_out = layout_of(res).buf;
      } else {
        s.r_out = materialise(res);
      }
      s.r_init_is_imm = init_imm;
      if (init_imm) s.r_init_imm = element_to_reg(init->def->const_data.data(), init->type.dtype);
      else { s.r_init_buf = layout_of(init).buf; s.r_init_dtype = init->type.dtype; }
    } else {
      s.r_out_dtype = cls_dtype[ci.cls];
      s.r_out = new_temp(A * B * 4);
      s.r_init_is_imm = true;
      // identity of the monoid
      float one = 1.f, ninf = -INFINITY, pinf = INFINITY;
      uint32_t id = 0;
      switch (op.monoid) {
        case Monoid::ADD: case Monoid::OR: case Monoid::XOR: id = 0; break;
        case Monoid::MUL: if (ci.cls == VM_F32) memcpy(&id, &one, 4); else id = 1; break;
        case Monoid::MAX: if (ci.cls == VM_F32) memcpy(&id, &ninf, 4); else id = ci.cls == VM_S32 ? 0x80000000u : 0u; break;
        case Monoid::MIN: if (ci.cls == VM_F32) memcpy(&id, &pinf, 4); else id = ci.cls == VM_S32 ? 0x7fffffffu : 0xffffffffu; break;
        case Monoid::AND: id = 0xffffffffu; break;
      }
      s.r_init_imm = id;
    }
    int S = reduce_splits_impl(A, R, B);
    if (S > 1) { s.scratch_bytes = A * S * B * 4; s.scratch = new_temp(s.scratch_bytes); }
    s.bytes = (double)x->type.byte_size();
    touch_vm(s.vm);
    touch(s.r_out); touch(s.r_init_buf); touch(s.scratch);
    cur_buf = s.r_out;
    plan_.steps.push_back(std::move(s));
    // shape after this pass
    std::vector<int64_t> ns;
    for (int d = 0; d < (int)shape.size(); d++) if (d < lo || d > hi) ns.push_back(shape[d]);
    shape = ns;
    first = false;
  }
}

// Copies a strided view into fresh contiguous arena memory (row-major over `dims`).
BufRef Planner::emit_strided_copy(const Layout& src, DType dt, const std::vector<int64_t>& dims, const std::string& label) {
  int64_t n = 1;
  for (auto d : dims) n *= d;
  BufRef dst = new_temp(n * dtype_size(dt));
  if (dtype_size(dt) == 8) {
    if (!is_row_major(dims, src.strides)) { emit_wide_copy(src, dt, dims, dst, dt, label); return dst; }
    Step s; s.kind = StepKind::COPY; s.label = label; s.c_src = src.buf; s.c_dst = dst; s.c_bytes = n * 8;
    touch(src.buf); touch(dst);
    plan_.steps.push_back(s);
    return dst;
  }
  GroupBuilder gb;
  gb.P = this;
  gb.root_dims = dims;
  GNode nd;
  nd.k = GNode::TENSOR;
  nd.dtype = dt;
  nd.tensor = gb.add_tensor(src.buf, dt, src.strides);
  gb.nodes.push_back(nd);
  int t = gb.add_tensor(dst, dt, row_major_strides(dims));
  gb.outs.push_back({0, t});
  VmBinding vb = gb.finish(-1);
  push_vm_step(std::move(vb), label);
  return dst;
}

// ---- 64-bit element types ----------------------------------------------------------------------------------------------
// Copies (and converts) a strided view into a dense row-major tensor with the 64-bit elementwise kernel.
void Planner::emit_wide_copy(const Layout& src, DType src_dt, const std::vector<int64_t>& dims, const BufRef& dst, DType dst_dt, const std::string& label) {
  if ((int)dims.size() > B2X_WIDE_MAX_DIMS) unimplemented("64-bit tensors of rank above " + std::to_string(B2X_WIDE_MAX_DIMS));
  Step s;
  s.kind = StepKind::WIDE;
  s.label = label;
  s.w_op = B2X_WIDE_COPY;
  s.w_n_in = 1;
  s.w_in_dtype[0] = src_dt; s.w_out_dtype = dst_dt;
  s.w_dims = dims;
  s.w_in_strides[0] = src.strides;
  s.w_in[0] = src.buf; s.w_out = dst;
  int64_t n = 1;
  for (auto d : dims) n *= d;
  s.bytes = (double)n * (dtype_size(src_dt) + dtype_size(dst_dt));
  touch(src.buf); touch(dst);
  plan_.steps.push_back(std::move(s));
}

// One elementwise-class op over 64-bit tensors (or converting to / from one).
void Planner::emit_wide(const Op& op) {
  const Value* res = op.results[0];
  if (res->type.rank() > B2X_WIDE_MAX_DIMS) unimplemented("64-bit tensors of rank above " + std::to_string(B2X_WIDE_MAX_DIMS));
  Step s;
  s.kind = StepKind::WIDE;
  s.label = std::string(op_name(op.kind)) + ":%" + res->name;
  s.w_dims = res->type.dims;
  s.w_out_dtype = res->type.dtype;
  auto operand = [&](int k, const Value* v, const std::vector<int>& map) {
    // map[i] = result dim that operand dim i walks (-1: the operand dim has extent 1)
    Layout& L = layout_of(v);
    std::vector<int64_t> st(res->type.rank(), 0);
    for (int i = 0; i < v->type.rank(); i++) if (map[i] >= 0 && v->type.dims[i] > 1) st[map[i]] += L.strides[i];
    s.w_in[k] = L.buf; s.w_in_dtype[k] = v->type.dtype; s.w_in_strides[k] = st;
    touch(L.buf);
  };
  auto same_shape = [&](const Value* v) {
    std::vector<int> ident(v->type.rank());
    for (int i = 0; i < v->type.rank(); i++) ident[i] = i;
    if (v->type.rank() == 0) ident.clear();
    return ident;
  };
  static const std::map<OpKind, int> simple = {
      {OpKind::ADD, B2X_WIDE_ADD}, {OpKind::SUBTRACT, B2X_WIDE_SUB}, {OpKind::MULTIPLY, B2X_WIDE_MUL}, {OpKind::DIVIDE, B2X_WIDE_DIV},
      {OpKind::REMAINDER, B2X_WIDE_REM}, {OpKind::POWER, B2X_WIDE_POW}, {OpKind::MAXIMUM, B2X_WIDE_MAX}, {OpKind::MINIMUM, B2X_WIDE_MIN},
      {OpKind::AND, B2X_WIDE_AND}, {OpKind::OR, B2X_WIDE_OR}, {OpKind::XOR, B2X_WIDE_XOR}, {OpKind::NEGATE, B2X_WIDE_NEG}, {OpKind::ABS, B2X_WIDE_ABS},
      {OpKind::SIGN, B2X_WIDE_SIGN}, {OpKind::NOT, B2X_WIDE_NOT}, {OpKind::TANH, B2X_WIDE_TANH}, {OpKind::EXP, B2X_WIDE_EXP}, {OpKind::LOG, B2X_WIDE_LOG},
      {OpKind::SQRT, B2X_WIDE_SQRT}, {OpKind::RSQRT, B2X_WIDE_RSQRT}, {OpKind::LOGISTIC, B2X_WIDE_LOGISTIC}, {OpKind::FLOOR, B2X_WIDE_FLOOR},
      {OpKind::CEIL, B2X_WIDE_CEIL}, {OpKind::EXPM1, B2X_WIDE_EXPM1}, {OpKind::LOG1P, B2X_WIDE_LOG1P}, {OpKind::SINE, B2X_WIDE_SIN},
      {OpKind::COSINE, B2X_WIDE_COS}, {OpKind::CONVERT, B2X_WIDE_COPY}, {OpKind::SELECT, B2X_WIDE_SELECT}, {OpKind::CLAMP, B2X_WIDE_CLAMP},
      {OpKind::COMPARE, B2X_WIDE_COMPARE}};
  switch (op.kind) {
    case OpKind::CONSTANT: {   // splat (dense constants live in the constant pool)
      s.w_op = B2X_WIDE_FILL;
      // bit pattern of the value in the class of the result type (int64 / uint64 / double)
      const uint8_t* p = op.const_data.data();
      switch (res->type.dtype) {
        case DType::S64: case DType::U64: case DType::F64: memcpy(&s.w_imm, p, 8); break;
        default: internal("wide fill of a narrow type");
      }
      break;
    }
    case OpKind::IOTA:
      s.w_op = B2X_WIDE_IOTA;
      s.w_aux = (int)op.iota_dim;
      break;
    case OpKind::BROADCAST_IN_DIM: {
      s.w_op = B2X_WIDE_COPY;
      s.w_n_in = 1;
      const Value* u = op.operands[0];
      std::vector<int> map(u->type.rank());
      for (int i = 0; i < u->type.rank(); i++) map[i] = u->type.dims[i] == 1 ? -1 : (int)op.dims[i];
      operand(0, u, map);
      break;
    }
    default: {
      auto it = simple.find(op.kind);
      if (it == simple.end()) unimplemented(std::string(op_name(op.kind)) + " over 64-bit element types");
      s.w_op = it->second;
      s.w_n_in = (int)op.operands.size();
      if (s.w_n_in > 3) internal("wide op with more than three operands");
      for (int k = 0; k < s.w_n_in; k++) {
        const Value* v = op.operands[k];
        // a scalar predicate of select and scalar bounds of clamp apply to every element
        std::vector<int> map = (v->type.rank() == 0 && res->type.rank() != 0) ? std::vector<int>() : same_shape(v);
        operand(k, v, map);
      }
      if (op.kind == OpKind::COMPARE) {
        s.w_aux = (int)op.cmp_dir;
        s.w_aux2 = op.cmp_type == CmpType::UNSIGNED ? 1 : (op.cmp_type == CmpType::SIGNED ? 2 : 0);
      }
      break;
    }
  }
  s.w_out = materialise(res);
  s.bytes = (double)res->type.byte_size();
  for (int k = 0; k < s.w_n_in; k++) s.bytes += (double)op.operands[k]->type.byte_size();
  touch(s.w_out);
  plan_.steps.push_back(std::move(s));
}

// stablehlo.reduce over a 64-bit tensor: one pass per maximal run of adjacent reduced dims, innermost first.
void Planner::emit_wide_reduce(const Op& op) {
  const Value* x = op.operands[0];
  const Value* init = op.operands[1];
  const Value* res = op.results[0];
  const DType dt = x->type.dtype;
  Layout L = layout_of(x);
  BufRef cur = L.buf;
  if (!is_row_major(x->type.dims, L.strides)) cur = emit_strided_copy(L, dt, x->type.dims, "copy:reduce_operand");
  std::vector<int64_t> rd = op.dims;
  std::sort(rd.begin(), rd.end());
  std::vector<std::pair<int, int>> runs;
  std::vector<int64_t> shape = x->type.dims;
  if (rd.empty()) runs.push_back({(int)shape.size(), (int)shape.size() - 1});
  else {
    size_t i = 0;
    while (i < rd.size()) { size_t j = i; while (j + 1 < rd.size() && rd[j + 1] == rd[j] + 1) j++; runs.push_back({(int)rd[i], (int)rd[j]}); i = j + 1; }
    std::reverse(runs.begin(), runs.end());
  }
  const bool init_imm = init->def && init->def->kind == OpKind::CONSTANT && init->def->splat;
  for (size_t p = 0; p < runs.size(); p++) {
    const bool last = p + 1 == runs.size();
    const int lo = runs[p].first, hi = runs[p].second;
    int64_t A = 1, R = 1, B = 1;
    for (int d = 0; d < (int)shape.size(); d++) { if (d < lo) A *= shape[d]; else if (d <= hi) R *= shape[d]; else B *= shape[d]; }
    Step s;
    s.kind = StepKind::REDUCE;
    s.wide = true;
    s.label = std::string("reduce:%") + res->name + (runs.size() > 1 ? ":pass" + std::to_string(p) : "");
    s.rA = A; s.rR = R; s.rB = B;
    s.monoid = op.monoid;
    s.w_in[0] = cur; s.w_in_dtype[0] = dt;
    s.r_out_dtype = dt;
    if (last) {
      s.r_out = materialise(res);
      s.r_init_is_imm = init_imm;
      if (init_imm) memcpy(&s.w_imm, init->def->const_data.data(), 8);
      else { s.r_init_buf = layout_of(init).buf; s.r_init_dtype = dt; }
    } else {
      s.r_out = new_temp(A * B * 8);
      s.r_init_is_imm = true;
      // identity of the monoid in the class of dt
      const bool f = dt == DType::F64, sg = dt == DType::S64;
      double one = 1.0, ninf = -INFINITY, pinf = INFINITY;
      uint64_t id = 0;
      switch (op.monoid) {
        case Monoid::ADD: case Monoid::OR: case Monoid::XOR: id = 0; break;
        case Monoid::MUL: if (f) memcpy(&id, &one, 8); else id = 1; break;
        case Monoid::MAX: if (f) memcpy(&id, &ninf, 8); else id = sg ? 0x8000000000000000ull : 0ull; break;
        case Monoid::MIN: if (f) memcpy(&id, &pinf, 8); else id = sg ? 0x7fffffffffffffffull : ~0ull; break;
        case Monoid::AND: id = ~0ull; break;
      }
      s.w_imm = id;
    }
    s.bytes = (double)A * R * B * 8;
    touch(cur); touch(s.r_out); touch(s.r_init_buf);
    cur = s.r_out;
    plan_.steps.push_back(std::move(s));
    std::vector<int64_t> ns;
    for (int d = 0; d < (int)shape.size(); d++) if (d < lo || d > hi) ns.push_back(shape[d]);
    shape = ns;
  }
}

void Planner::emit_view_or_copy(const Op& op) {
  const Value* x = op.operands[0];
  const Value* r = op.results[0];
  Layout& L = layout_of(x);
  if (op.kind == OpKind::TRANSPOSE) {
    std::vector<int64_t> s(r->type.rank());
    for (int i = 0; i < r->type.rank(); i++) s[i] = L.strides[op.dims[i]];
    set_layout(r, L.buf, s);
  } else {  // RESHAPE
    if (is_row_major(x->type.dims, L.strides)) set_layout(r, L.buf, row_major_strides(r->type.dims));
    else {
      BufRef c = emit_strided_copy(L, x->type.dtype, x->type.dims, "copy:reshape:%" + r->name);
      set_layout(r, c, row_major_strides(r->type.dims));
    }
  }
}

// Collapses the listed dims (outer to inner) of a layout into one (size, stride); false when they do not form a
// single strided run.
bool collapse(const std::vector<int64_t>& dims, const std::vector<int64_t>& strides, const std::vector<int64_t>& which,
              int64_t* size, int64_t* stride) {
  *size = 1;
  *stride = 0;
  int64_t prev = -1;  // stride of the previous (outer) non-unit dim
  for (auto d : which) {
    if (dims[d] == 1) continue;
    if (prev >= 0 && prev != strides[d] * dims[d]) return false;
    prev = strides[d];
    *size *= dims[d];
    *stride = strides[d];
  }
  return true;
}

// The elementwise consumer groups of a kernel result `res` that can run inside the producing kernel (as a GEMM epilogue
// or on the finished values of a reduce): groups rooted at a value of the same shape whose other inputs all exist when
// the kernel runs and that reach `res` with unchanged coordinates.  Returns whether `res` itself must still be stored.
bool Planner::collect_consumer_roots(const Op& op, const Value* res, std::vector<const Value*>* fused_roots) {
  bool res_needs_memory = false;
  for (auto u : res->users) if (!is_fusible_kind(*u) && !(u->kind == OpKind::REDUCE && u->operands[0] == res)) res_needs_memory = true;
  for (auto o : m_.outputs) if (o == res) res_needs_memory = true;
  const int my_index = op_index_[&op];
  for (int g : st(res).groups) {
    const Value* r = group_root_[g];
    bool ok = opt_.allow_epilogue_fusion && r != nullptr && r->type.dims == res->type.dims;
    // every other input of the group must already exist when the kernel runs, and `res` must be reached with
    // unchanged coordinates (not underneath a broadcast)
    std::function<bool(const Value*, bool)> ready = [&](const Value* v, bool under_bcast) -> bool {
      if (v == res) return !under_bcast;
      if (v != r && load_as_leaf(v)) return (v->def == nullptr || op_index_[v->def] < my_index) && st(v).has_layout;
      if (!v->def) return true;
      bool ub = under_bcast || v->def->kind == OpKind::BROADCAST_IN_DIM;
      for (auto o : v->def->operands) if (!ready(o, ub)) return false;
      return true;
    };
    if (ok) ok = ready(r, false);
    if (ok) fused_roots->push_back(r); else res_needs_memory = true;
  }
  std::sort(fused_roots->begin(), fused_roots->end(), [](const Value* a, const Value* b) { return a->id < b->id; });
  return res_needs_memory;
}

void Planner::emit_dot(const Op& op) {
  const Value* lv = op.operands[0];
  const Value* rv = op.operands[1];
  const Value* res = op.results[0];
  DType in_dt = lv->type.dtype;
  if (rv->type.dtype != in_dt) unimplemented("dot_general with operands of different element types");
  const bool wide = is_wide_type(in_dt) || is_wide_type(res->type.dtype);
  bool float_in = (in_dt == DType::F32 || in_dt == DType::BF16 || in_dt == DType::F16 || in_dt == DType::F64);
  bool int_in = (in_dt == DType::S32 || in_dt == DType::S8 || in_dt == DType::S16 || in_dt == DType::U8 || in_dt == DType::U16 || in_dt == DType::U32 ||
                 in_dt == DType::S64 || in_dt == DType::U64);
  if (!float_in && !int_in) unimplemented(std::string("dot_general over ") + dtype_name(in_dt));
  if (!wide) class_of(res->type.dtype);

  auto free_dims = [](int rank, const std::vector<int64_t>& a, const std::vector<int64_t>& b) {
    std::vector<int64_t> f;
    for (int i = 0; i < rank; i++) if (std::find(a.begin(), a.end(), i) == a.end() && std::find(b.begin(), b.end(), i) == b.end()) f.push_back(i);
    return f;
  };
  std::vector<int64_t> lfree = free_dims(lv->type.rank(), op.lhs_batch, op.lhs_contract);
  std::vector<int64_t> rfree = free_dims(rv->type.rank(), op.rhs_batch, op.rhs_contract);

  // contracting pairs ordered by descending lhs stride so that both sides have a chance to collapse
  Layout LL = layout_of(lv), RL = layout_of(rv);
  std::vector<size_t> order(op.lhs_contract.size());
  for (size_t i = 0; i < order.size(); i++) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return LL.strides[op.lhs_contract[a]] > LL.strides[op.lhs_contract[b]]; });
  std::vector<int64_t> lc, rc;
  for (auto i : order) { lc.push_back(op.lhs_contract[i]); rc.push_back(op.rhs_contract[i]); }

  Step s;
  s.kind = StepKind::GEMM;
  s.label = "dot_general:%" + res->name;
  int64_t Bl, Br, M, N, Kl, Kr;
  auto prep = [&](const Value* v, Layout& L, const std::vector<int64_t>& batch, const std::vector<int64_t>& fr,
                  const std::vector<int64_t>& con, GemmOperand* g, int64_t* Bn, int64_t* Fn, int64_t* Kn, const char* side) {
    int64_t bs, fs, ks;
    bool ok = collapse(v->type.dims, L.strides, batch, Bn, &bs) && collapse(v->type.dims, L.strides, fr, Fn, &fs) &&
              collapse(v->type.dims, L.strides, con, Kn, &ks);
    if (!ok) {
      // bring the operand into [batch, free, contract] order once
      std::vector<int64_t> perm = batch;
      perm.insert(perm.end(), fr.begin(), fr.end());
      perm.insert(perm.end(), con.begin(), con.end());
      Layout src;
      src.buf = L.buf;
      std::vector<int64_t> pd;
      for (auto d : perm) { pd.push_back(v->type.dims[d]); src.strides.push_back(L.strides[d]); }
      BufRef c = emit_strided_copy(src, v->type.dtype, pd, std::string("copy:dot_") + side + ":%" + res->name);
      *Bn = 1; *Fn = 1; *Kn = 1;
      for (auto d : batch) *Bn *= v->type.dims[d];
      for (auto d : fr) *Fn *= v->type.dims[d];
      for (auto d : con) *Kn *= v->type.dims[d];
      g->buf = c;
      g->batch_stride = *Fn * *Kn; g->row_stride = *Kn; g->k_stride = 1;
    } else {
      g->buf = L.buf;
      g->batch_stride = bs; g->row_stride = fs; g->k_stride = ks;
    }
    g->dtype = v->type.dtype;
  };
  prep(lv, LL, op.lhs_batch, lfree, lc, &s.ga, &Bl, &M, &Kl, "lhs");
  prep(rv, RL, op.rhs_batch, rfree, rc, &s.gb, &Br, &N, &Kr, "rhs");
  if (Bl != Br || Kl != Kr) internal("dot_general operand factorisation mismatch");
  s.gB = Bl; s.gM = M; s.gN = N; s.gK = Kl;
  s.g_acc_dtype = float_in ? DType::F32 : DType::S32;
  s.flops = 2.0 * (double)s.gB * (double)M * (double)N * (double)Kl;
  if (wide) {
    // 64-bit operands or result: the plain strided kernel, result stored densely, consumers read it from memory
    s.wide = true;
    s.w_out_dtype = res->type.dtype;
    s.w_out = materialise(res);
    s.bytes = (double)lv->type.byte_size() + (double)rv->type.byte_size() + (double)res->type.byte_size();
    touch(s.ga.buf); touch(s.gb.buf); touch(s.w_out);
    plan_.steps.push_back(std::move(s));
    return;
  }

  // ---- tensor-core eligibility ----
  auto tc_operand_ok = [&](const GemmOperand& g, int64_t rows) {
    int es = dtype_size(g.dtype);
    int64_t al = 16 / es;
    bool kmajor = (g.k_stride == 1 || s.gK == 1) && (g.row_stride % al == 0 || rows == 1);
    bool mnmajor = (g.row_stride == 1) && (g.k_stride % al == 0);
    return (kmajor || mnmajor) && (g.batch_stride % al == 0 || s.gB == 1);
  };
  bool tc_dtype = (in_dt == DType::BF16 || in_dt == DType::F16 || in_dt == DType::F32);
  s.g_tensor_core = opt_.allow_tensor_core && tc_dtype && M >= 128 && N >= 64 && N % 8 == 0 && s.gK >= 32 &&
                    tc_operand_ok(s.ga, M) && tc_operand_ok(s.gb, N);
  if (s.g_tensor_core && in_dt == DType::F32) {
    // three TF32 products over hi/lo splits: A' = [Ahi | Ahi | Alo], B' = [Bhi | Blo | Bhi] along K, held in scratch
    s.g_split_f32 = true;
    s.scratch_bytes = (s.gB * M * 3 * s.gK + s.gB * N * 3 * s.gK) * 4 + 2048;
    s.scratch = new_temp(s.scratch_bytes);
  }

  // ---- epilogue: fold in the elementwise consumer groups of the accumulator where possible ----
  std::vector<const Value*> fused_roots;
  bool res_needs_memory = collect_consumer_roots(op, res, &fused_roots);

  for (;;) {
    GroupBuilder gb;
    gb.P = this;
    gb.root_dims = res->type.dims;
    gb.acc0_value = res;
    try {
      if (res_needs_memory || fused_roots.empty()) {
        BufRef out = materialise(res);
        gb.add_output(res, out);
      }
      for (auto r : fused_roots) gb.computing.insert(r);
      for (auto r : fused_roots) { BufRef out = materialise(r); gb.add_output(r, out); }
      s.vm = gb.finish(-1);
      break;
    } catch (const GroupTooLarge&) {
      // the consumer groups do not fit into one epilogue: store the plain result and let them run as kernels of their own
      if (fused_roots.empty()) throw;
      fused_roots.clear();
      res_needs_memory = true;
    }
  }
  for (auto r : fused_roots) emitted_groups_.insert(root_group_[r]);
  if (s.vm.vec != 8) s.g_tensor_core = false, s.g_split_f32 = false;
  // The accumulator arrives as F32 (or S32) registers; a bf16/f16 result type rounds when stored.
  s.bytes = (double)lv->type.byte_size() + (double)rv->type.byte_size();
  for (int t = 0; t < s.vm.prog.n_tensors; t++) s.bytes += (double)s.vm.n_elements * dtype_size((DType)s.vm.prog.tensors[t].elem);
  touch(s.ga.buf); touch(s.gb.buf); touch(s.scratch);
  touch_vm(s.vm);
  if (!fused_roots.empty()) { s.label += "+epilogue("; for (auto r : fused_roots) s.label += "%" + r->name + " "; s.label += ")"; }
  plan_.steps.push_back(std::move(s));
}

void Planner::emit_collective(const Op& op) {
  Step s;
  s.kind = op.kind == OpKind::ALL_REDUCE ? StepKind::ALL_REDUCE : StepKind::ALL_GATHER;
  s.label = std::string(op_name(op.kind));
  s.monoid = op.monoid;
  s.replica_groups = op.replica_groups;
  if (op.use_global_device_ids && opt_.num_partitions > 1) unimplemented("collectives with use_global_device_ids over several partitions");
  // every group must have the same size; an empty list means one group of all replicas
  if (s.replica_groups.empty() || (s.replica_groups.size() == 1 && s.replica_groups[0].empty())) {
    s.replica_groups.assign(1, {});
    for (int i = 0; i < opt_.num_replicas; i++) s.replica_groups[0].push_back(i);
  }
  std::set<int64_t> seen;
  for (auto& g : s.replica_groups) {
    if (g.size() != s.replica_groups[0].size()) unimplemented("replica groups of different sizes");
    for (auto id : g) {
      if (id < 0 || id >= opt_.num_replicas) throw CompileError(kInvalidArgument, std::string(op_name(op.kind)) + ": replica id " + std::to_string(id) + " is outside replica_count = " + std::to_string(opt_.num_replicas));
      if (!seen.insert(id).second) throw CompileError(kInvalidArgument, std::string(op_name(op.kind)) + ": replica id listed twice");
    }
  }
  if ((int)seen.size() != opt_.num_replicas) unimplemented("replica_groups that do not cover every replica");
  struct PendingCopy { Layout src; BufRef dst; DType dt; std::vector<int64_t> dims; };
  std::vector<PendingCopy> pending_copies;
  for (size_t i = 0; i < op.operands.size(); i++) {
    const Value* x = op.operands[i];
    const Value* r = op.results[i];
    Layout L = layout_of(x);
    if (!is_row_major(x->type.dims, L.strides)) {
      L.buf = emit_strided_copy(L, x->type.dtype, x->type.dims, "copy:collective_operand");
      L.strides = row_major_strides(x->type.dims);
    }
    Step::Coll c;
    c.src = L.buf;
    c.dst = materialise(r);
    c.count = x->type.num_elements();
    c.dtype = x->type.dtype;
    if (op.kind == OpKind::ALL_GATHER) {
      for (int d = 0; d < x->type.rank(); d++) { if (d < op.iota_dim) c.outer *= x->type.dims[d]; else c.inner *= x->type.dims[d]; }
      if (c.outer != 1) {
        // NCCL concatenates whole operands (a new outermost group dim); for an inner all_gather_dim the gathered
        // [G, outer, inner] staging buffer is rearranged into [outer, G, inner] by a strided copy afterwards
        const int64_t G = (int64_t)s.replica_groups[0].size();
        BufRef final_dst = c.dst;
        c.dst = new_temp(r->type.byte_size());
        Layout src;
        src.buf = c.dst;
        src.strides = {c.inner, c.outer * c.inner, 1};
        pending_copies.push_back({src, final_dst, x->type.dtype, {c.outer, G, c.inner}});
      }
    } else {
      if (dtype_size(c.dtype) == 8 && c.dtype != DType::F64 && c.dtype != DType::S64 && c.dtype != DType::U64) internal("bad dtype");
    }
    touch(c.src); touch(c.dst);
    s.bytes += (double)x->type.byte_size();
    s.colls.push_back(c);
  }
  plan_.steps.push_back(std::move(s));
  for (auto& pc : pending_copies) {
    if (dtype_size(pc.dt) == 8) { emit_wide_copy(pc.src, pc.dt, pc.dims, pc.dst, pc.dt, "copy:all_gather_interleave"); continue; }
    GroupBuilder gb;
    gb.P = this;
    gb.root_dims = pc.dims;
    GNode nd;
    nd.k = GNode::TENSOR;
    nd.dtype = pc.dt;
    nd.tensor = gb.add_tensor(pc.src.buf, pc.dt, pc.src.strides);
    gb.nodes.push_back(nd);
    int t = gb.add_tensor(pc.dst, pc.dt, row_major_strides(pc.dims));
    gb.outs.push_back({0, t});
    VmBinding vb = gb.finish(-1);
    push_vm_step(std::move(vb), "copy:all_gather_interleave");
  }
}

void Planner::emit_outputs() {
  for (size_t i = 0; i < m_.outputs.size(); i++) {
    const Value* v = m_.outputs[i];
    ValueState& s = st(v);
    plan_.outputs.push_back({v->type});
    Layout& L = layout_of(v);
    bool direct = L.buf.kind == BufRef::OUT && L.buf.index == (int)i && is_row_major(v->type.dims, L.strides);
    if (direct) continue;
    BufRef dst;
    dst.kind = BufRef::OUT;
    dst.index = (int)i;
    if (!is_row_major(v->type.dims, L.strides) && dtype_size(v->type.dtype) == 8) {
      emit_wide_copy(L, v->type.dtype, v->type.dims, dst, v->type.dtype, "copy:output" + std::to_string(i));
    } else if (is_row_major(v->type.dims, L.strides)) {
      Step c;
      c.kind = StepKind::COPY;
      c.label = "copy:output" + std::to_string(i);
      c.c_src = L.buf; c.c_dst = dst; c.c_bytes = v->type.byte_size();
      touch(L.buf);
      c.bytes = 2.0 * (double)c.c_bytes;
      plan_.steps.push_back(c);
    } else {
      GroupBuilder gb;
      gb.P = this;
      gb.root_dims = v->type.dims;
      GNode nd;
      nd.k = GNode::TENSOR;
      nd.dtype = v->type.dtype;
      nd.tensor = gb.add_tensor(L.buf, v->type.dtype, L.strides);
      gb.nodes.push_back(nd);
      int t = gb.add_tensor(dst, v->type.dtype, row_major_strides(v->type.dims));
      gb.outs.push_back({0, t});
      VmBinding vb = gb.finish(-1);
      push_vm_step(std::move(vb), "copy:output" + std::to_string(i));
    }
    (void)s;
  }
}

// ---- read / write sets of a step ------------------------------------------------------------------------------
static bool same_buf(const BufRef& a, const BufRef& b) { return a.kind == b.kind && a.index == b.index && (a.kind != BufRef::CONST || a.offset == b.offset); }
static void step_bufs(const Step& s, std::vector<BufRef>* reads, std::vector<BufRef>* writes) {
  auto vm_sets = [&](const VmBinding& vm) {
    for (int t = 0; t < vm.prog.n_tensors; t++) {
      bool written = false, read = false;
      for (int i = 0; i < vm.prog.n_instr; i++) {
        const B2xVmInstr& I = vm.prog.code[i];
        if (I.src_kind == VM_SRC_TENSOR && I.src_idx == t) { if (I.op == VM_STORE) written = true; else read = true; }
      }
      if (written) writes->push_back(vm.bufs[t]);
      if (read) reads->push_back(vm.bufs[t]);
    }
  };
  switch (s.kind) {
    case StepKind::ELEMENTWISE: vm_sets(s.vm); break;
    case StepKind::WIDE:
      for (int k = 0; k < s.w_n_in; k++) reads->push_back(s.w_in[k]);
      writes->push_back(s.w_out);
      break;
    case StepKind::REDUCE:
      if (s.wide) {
        reads->push_back(s.w_in[0]);
        writes->push_back(s.r_out);
        if (s.r_init_buf.valid()) reads->push_back(s.r_init_buf);
        break;
      }
      vm_sets(s.vm);
      if (s.has_post) vm_sets(s.post);
      if (s.r_out.valid()) writes->push_back(s.r_out);
      if (s.r_init_buf.valid()) reads->push_back(s.r_init_buf);
      if (s.scratch.valid()) writes->push_back(s.scratch);
      break;
    case StepKind::GEMM:
      reads->push_back(s.ga.buf); reads->push_back(s.gb.buf);
      if (s.wide) { writes->push_back(s.w_out); break; }
      vm_sets(s.vm);
      if (s.scratch.valid()) writes->push_back(s.scratch);
      break;
    case StepKind::ATTENTION:
      reads->push_back(s.aq); reads->push_back(s.ak); reads->push_back(s.av); writes->push_back(s.ao);
      if (s.scratch.valid()) writes->push_back(s.scratch);
      break;
    case StepKind::ALL_REDUCE: case StepKind::ALL_GATHER:
      for (auto& c : s.colls) { reads->push_back(c.src); writes->push_back(c.dst); }
      break;
    case StepKind::COPY: reads->push_back(s.c_src); writes->push_back(s.c_dst); break;
  }
}

// Collectives run on a communication stream beside the compute stream.  Each one is split per operand, moved up to
// directly behind the step that produces its operand, and the first later step that touches its result is told to
// wait for it; so a gradient all-reduce overlaps with the GEMMs that follow its producer.
void Planner::schedule_collectives() {
  std::vector<Step> split;
  for (auto& s : plan_.steps) {
    if ((s.kind == StepKind::ALL_REDUCE || s.kind == StepKind::ALL_GATHER) && s.colls.size() > 1) {
      // operands whose producer runs earlier go first, so that each can start as soon as its data exists
      std::vector<std::pair<int, size_t>> order;
      for (size_t k = 0; k < s.colls.size(); k++) {
        int producer = -1;
        for (int j = 0; j < (int)split.size(); j++) {
          std::vector<BufRef> r, w;
          step_bufs(split[j], &r, &w);
          for (auto& b : w) if (same_buf(b, s.colls[k].src)) producer = j;
        }
        order.push_back({producer, k});
      }
      std::stable_sort(order.begin(), order.end());
      for (auto& o : order) {
        const Step::Coll& c = s.colls[o.second];
        Step t = s; t.colls.assign(1, c); t.bytes = (double)c.count * dtype_size(c.dtype); split.push_back(std::move(t));
      }
    } else split.push_back(std::move(s));
  }
  // hoist
  std::vector<Step> out;
  int last_coll_pos = -1;
  for (auto& s : split) {
    if (s.kind != StepKind::ALL_REDUCE && s.kind != StepKind::ALL_GATHER) { out.push_back(std::move(s)); continue; }
    int pos = (int)out.size();
    while (pos - 1 > last_coll_pos) {
      std::vector<BufRef> r, w;
      step_bufs(out[pos - 1], &r, &w);
      bool conflict = false;
      for (auto& c : s.colls) {
        for (auto& b : w) if (same_buf(b, c.src) || same_buf(b, c.dst)) conflict = true;
        for (auto& b : r) if (same_buf(b, c.dst)) conflict = true;
      }
      if (conflict) break;
      pos--;
    }
    out.insert(out.begin() + pos, std::move(s));
    last_coll_pos = pos;
  }
  // ids and waits
  int n = 0;
  for (auto& s : out) if (s.kind == StepKind::ALL_REDUCE || s.kind == StepKind::ALL_GATHER) s.coll_id = n++;
  plan_.num_collectives = n;
  for (size_t i = 0; i < out.size(); i++) {
    if (out[i].coll_id < 0) continue;
    bool waited = false;
    for (size_t j = i + 1; j < out.size(); j++) {
      std::vector<BufRef> r, w;
      step_bufs(out[j], &r, &w);
      bool dep = false;
      for (auto& c : out[i].colls) {
        for (auto& b : r) if (same_buf(b, c.dst)) dep = true;
        for (auto& b : w) if (same_buf(b, c.dst) || same_buf(b, c.src)) dep = true;
      }
      if (dep) { out[j].wait_colls.push_back(out[i].coll_id); waited = true; break; }
    }
    if (!waited) {
      bool arena = false;
      for (auto& c : out[i].colls) if (c.src.kind == BufRef::TEMP || c.dst.kind == BufRef::TEMP) arena = true;
      if (!arena) { out[i].coll_detached = true; plan_.has_detached_collectives = true; }
    }
  }
  plan_.arg_in_detached.assign(plan_.arg_types.size(), 0);
  plan_.out_in_detached.assign(plan_.outputs.size(), 0);
  for (auto& s : out) {
    if (!s.coll_detached) continue;
    for (auto& c : s.colls)
      for (const BufRef* b : {&c.src, &c.dst}) {
        if (b->kind == BufRef::ARG && (size_t)b->index < plan_.arg_in_detached.size()) plan_.arg_in_detached[b->index] = 1;
        if (b->kind == BufRef::OUT && (size_t)b->index < plan_.out_in_detached.size()) plan_.out_in_detached[b->index] = 1;
      }
  }
  plan_.steps = std::move(out);
}

void Planner::compute_liveness() {
  for (auto& a : allocs_) { a.first = 1 << 30; a.last = -1; }
  auto use = [&](const BufRef& b, int i) {
    if (b.kind != BufRef::TEMP) return;
    allocs_[b.index].first = std::min(allocs_[b.index].first, i);
    allocs_[b.index].last = std::max(allocs_[b.index].last, i);
  };
  const int n = (int)plan_.steps.size();
  for (int i = 0; i < n; i++) {
    std::vector<BufRef> r, w;
    step_bufs(plan_.steps[i], &r, &w);
    for (auto& b : r) use(b, i);
    for (auto& b : w) use(b, i);
  }
  // a collective keeps reading/writing until the step that waits for it (or the end of the plan)
  for (int i = 0; i < n; i++) {
    const Step& s = plan_.steps[i];
    if (s.coll_id < 0) continue;
    int until = n - 1;
    for (int j = i + 1; j < n; j++)
      if (std::find(plan_.steps[j].wait_colls.begin(), plan_.steps[j].wait_colls.end(), s.coll_id) != plan_.steps[j].wait_colls.end()) { until = j; break; }
    for (auto& c : s.colls) { use(c.src, until); use(c.dst, until); }
  }
  for (auto& a : allocs_) if (a.last < 0) { a.first = 0; a.last = 0; }
}

void Planner::assign_arena() {
  // first-fit over lifetimes, larger buffers first so that they pack without holes
  std::vector<int> order(allocs_.size());
  for (size_t i = 0; i < order.size(); i++) order[i] = (int)i;
  std::sort(order.begin(), order.end(), [&](int a, int b) { return allocs_[a].bytes > allocs_[b].bytes; });
  const int64_t align = 1024;
  int64_t top = 0;
  std::vector<int> placed;
  for (int id : order) {
    Alloc& a = allocs_[id];
    int64_t size = (a.bytes + align - 1) / align * align;
    std::vector<std::pair<int64_t, int64_t>> busy;
    for (int p : placed) {
      Alloc& q = allocs_[p];
      if (q.last < a.first || q.first > a.last) continue;
      busy.push_back({q.offset, q.offset + (q.bytes + align - 1) / align * align});
    }
    std::sort(busy.begin(), busy.end());
    int64_t off = 0;
    for (auto& b : busy) { if (off + size <= b.first) break; off = std::max(off, b.second); }
    a.offset = off;
    top = std::max(top, off + size);
    placed.push_back(id);
  }
  plan_.arena_bytes = top;
  auto fix = [&](BufRef& b) { if (b.kind == BufRef::TEMP) { b.offset = allocs_[b.index].offset; } };
  for (auto& s : plan_.steps) {
    for (auto& b : s.vm.bufs) fix(b);
    for (auto& b : s.post.bufs) fix(b);
    fix(s.r_out); fix(s.r_init_buf); fix(s.scratch); fix(s.ga.buf); fix(s.gb.buf);
    fix(s.aq); fix(s.ak); fix(s.av); fix(s.ao); fix(s.c_src); fix(s.c_dst);
    for (int k = 0; k < 3; k++) fix(s.w_in[k]);
    fix(s.w_out);
    for (auto& c : s.colls) { fix(c.src); fix(c.dst); }
  }
}

Plan Planner::run() {
  plan_.name = m_.name;
  plan_.num_replicas = opt_.num_replicas;
  plan_.num_partitions = opt_.num_partitions;
  if (m_.has_sharding_attrs && opt_.num_partitions > 1)
    unimplemented("automatic SPMD partitioning (sharding attributes with partition_count > 1) is not supported; write the collectives explicitly");
  if (opt_.num_partitions > 1) unimplemented("partition_count > 1 is not supported; use replica_count for data parallelism");
  for (auto a : m_.args) {
    plan_.arg_types.push_back(a->type);
  }
  match_attention();
  classify();
  for (auto a : m_.args) {
    BufRef b;
    b.kind = BufRef::ARG;
    b.index = a->arg_index;
    set_layout(a, b, row_major_strides(a->type.dims));
  }
  for (auto& up : m_.ops) {
    const Op& op = *up;
    if (skip_ops_.count(&op)) continue;
    switch (op.kind) {
      case OpKind::RETURN: break;
      case OpKind::CONSTANT:
        if (!op.splat) {
          const Value* r = op.results[0];
          int64_t off = ((int64_t)plan_.const_pool.size() + 255) / 256 * 256;
          plan_.const_pool.resize(off);
          plan_.const_pool.insert(plan_.const_pool.end(), op.const_data.begin(), op.const_data.end());
          BufRef b;
          b.kind = BufRef::CONST;
          b.offset = off;
          set_layout(r, b, row_major_strides(r->type.dims));
          break;
        }
        // fallthrough: splat constants are fusible
      default:
        if (is_fusible_kind(op)) {
          const Value* r = op.results[0];
          if (st(r).root && !st(r).dead) emit_group_for_root(r);
          break;
        }
        if (touches_wide(op) && (op_is_elementwise(op.kind) || op.kind == OpKind::CONSTANT || op.kind == OpKind::IOTA ||
                                 op.kind == OpKind::BROADCAST_IN_DIM)) {
          emit_wide(op);
          break;
        }
        switch (op.kind) {
          case OpKind::REDUCE: emit_reduce(op); break;
          case OpKind::DOT_GENERAL: {
            auto it = attn_.find(&op);
            if (it != attn_.end()) emit_attention(op, it->second); else emit_dot(op);
            break;
          }
          case OpKind::TRANSPOSE: case OpKind::RESHAPE: emit_view_or_copy(op); break;
          case OpKind::ALL_REDUCE: case OpKind::ALL_GATHER: emit_collective(op); break;
          default: unimplemented(std::string(op_name(op.kind)) + " has no lowering");
        }
    }
  }
  emit_outputs();
  schedule_collectives();
  compute_liveness();
  assign_arena();
  for (auto& s : plan_.steps) { plan_.total_flops += s.flops; plan_.total_bytes += s.bytes; }
  return std::move(plan_);
}

const char* vm_op_name(uint8_t op) {
  static const char* n[] = {"end", "load", "save", "store", "add", "sub", "rsub", "mul", "div", "rdiv", "max", "min", "pow", "rpow",
                            "rem", "rrem", "and", "or", "xor", "cmp", "rcmp", "neg", "abs", "tanh", "exp", "log", "sqrt", "rsqrt",
                            "logistic", "not", "sign", "floor", "ceil", "expm1", "log1p", "sin", "cos", "cvt", "select", "rselect"};
  return op < sizeof(n) / sizeof(n[0]) ? n[op] : "?";
}
std::string buf_str(const BufRef& b) {
  switch (b.kind) {
    case BufRef::ARG: return "arg" + std::to_string(b.index);
    case BufRef::OUT: return "out" + std::to_string(b.index);
    case BufRef::TEMP: return "tmp@" + std::to_string(b.offset);
    case BufRef::CONST: return "const@" + std::to_string(b.offset);
    default: return "-";
  }
}
std::string vm_str(const VmBinding& vm) {
  std::ostringstream o;
  o << "    vm: dims=[";
  for (int d = 0; d < vm.prog.n_dims; d++) o << (d ? "," : "") << vm.prog.dim[d];
  o << "] vec=" << vm.vec << " tensors=[";
  for (int t = 0; t < vm.prog.n_tensors; t++) {
    o << (t ? ", " : "") << buf_str(vm.bufs[t]) << ":" << dtype_name((DType)vm.prog.tensors[t].elem) << "(";
    for (int d = 0; d < vm.prog.n_dims; d++) o << (d ? "," : "") << vm.prog.tensors[t].stride[d];
    o << ")";
  }
  o << "]\n    code:";
  for (int i = 0; i < vm.prog.n_instr; i++) {
    const B2xVmInstr& I = vm.prog.code[i];
    o << " " << vm_op_name(I.op);
    switch (I.src_kind) {
      case VM_SRC_TEMP: o << " t" << (int)I.src_idx; break;
      case VM_SRC_TENSOR: o << " T" << (int)I.src_idx; break;
      case VM_SRC_IMM: o << " #0x" << std::hex << I.imm << std::dec; break;
      case VM_SRC_IOTA: o << " iota" << (int)I.src_idx; break;
      case VM_SRC_ACC0: o << " acc0"; break;
      default: break;
    }
    if (I.op == VM_SAVE || I.op == VM_SELECT || I.op == VM_RSELECT) o << " [t" << (int)I.aux << "]";
    else if (I.aux) o << " aux=" << (int)I.aux;
    if (I.rnd) o << " rn" << (int)I.rnd;
    o << ";";
  }
  o << "\n";
  return o.str();
}

}  // namespace

int reduce_splits(int64_t A, int64_t R, int64_t B) { return reduce_splits_impl(A, R, B); }
int reduce_launches(int64_t A, int64_t R, int64_t B) {
  if (A <= 0 || B <= 0) return 0;
  return (reduce_splits_impl(A, R, B) > 1 && R > 0 && B != 1) ? 2 : 1;
}

std::string Plan::dump() const {
  std::ostringstream o;
  o << "plan " << name << ": " << steps.size() << " steps, arena " << arena_bytes << " B, consts " << const_pool.size() << " B, replicas "
    << num_replicas << "\n";
  int i = 0;
  for (auto& s : steps) {
    o << "  [" << i++ << "] ";
    for (int w : s.wait_colls) o << "(wait #" << w << ") ";
    switch (s.kind) {
      case StepKind::ELEMENTWISE: o << "elementwise " << s.label << "\n" << vm_str(s.vm); break;
      case StepKind::REDUCE:
        if (s.wide) {
          o << "reduce " << s.label << " [A=" << s.rA << ",R=" << s.rR << ",B=" << s.rB << "] monoid=" << (int)s.monoid << " 64-bit " << buf_str(s.w_in[0]) << " -> "
            << buf_str(s.r_out) << ":" << dtype_name(s.r_out_dtype) << "\n";
          break;
        }
        o << "reduce " << s.label << " [A=" << s.rA << ",R=" << s.rR << ",B=" << s.rB << "] monoid=" << (int)s.monoid << " -> " << buf_str(s.r_out)
          << ":" << dtype_name(s.r_out_dtype) << "\n" << vm_str(s.vm);
        if (s.has_post) o << "    on each result:\n" << vm_str(s.post);
        break;
      case StepKind::GEMM:
        o << "gemm " << s.label << " B=" << s.gB << " M=" << s.gM << " N=" << s.gN << " K=" << s.gK << (s.wide ? " 64-bit" : (s.g_tensor_core ? " tcgen05" : " simt"))
          << (s.g_split_f32 ? " 3xtf32" : "") << " A=" << buf_str(s.ga.buf) << "(" << s.ga.batch_stride << "," << s.ga.row_stride << ","
          << s.ga.k_stride << ") B=" << buf_str(s.gb.buf) << "(" << s.gb.batch_stride << "," << s.gb.row_stride << "," << s.gb.k_stride << ")\n"
          << vm_str(s.vm);
        break;
      case StepKind::ATTENTION:
        o << "attention " << s.label << " BH=" << s.aBH << " Sq=" << s.aSq << " Sk=" << s.aSk << " D=" << s.aD << " scale=" << s.a_scale
          << (s.a_causal ? " causal" : "") << "\n";
        break;
      case StepKind::ALL_REDUCE: case StepKind::ALL_GATHER:
        o << (s.kind == StepKind::ALL_REDUCE ? "all_reduce" : "all_gather") << " #" << s.coll_id << " " << buf_str(s.colls[0].src) << " -> " << buf_str(s.colls[0].dst)
          << " count=" << s.colls[0].count << " groups=" << s.replica_groups.size() << (s.coll_detached ? " detached" : "") << "\n";
        break;
      case StepKind::WIDE:
        o << "wide " << s.label << " op=" << s.w_op << " dims=[";
        for (size_t d = 0; d < s.w_dims.size(); d++) o << (d ? "," : "") << s.w_dims[d];
        o << "]";
        for (int k = 0; k < s.w_n_in; k++) o << " " << buf_str(s.w_in[k]) << ":" << dtype_name(s.w_in_dtype[k]);
        o << " -> " << buf_str(s.w_out) << ":" << dtype_name(s.w_out_dtype) << "\n";
        break;
      case StepKind::COPY: o << "copy " << s.label << " " << buf_str(s.c_src) << " -> " << buf_str(s.c_dst) << " " << s.c_bytes << " B\n"; break;
    }
  }
  return o.str();
}

Plan build_plan(const Module& m, const PlanOptions& opt, int replica) {
  Planner p(m, opt, replica);
  return p.run();
}

}  // namespace b2x
