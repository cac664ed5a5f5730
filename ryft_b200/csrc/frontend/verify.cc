// Shape and element-type checks for the accepted StableHLO subset.  The rules restate the constraints the
// reference documents next to each builder (e.g. dot_general: crates/ryft-mlir/src/dialects/stable_hlo/
// operations/linear_algebra.rs:561-592; broadcast_in_dim: manipulation.rs:271-285; reduce: functional.rs:109-118).
#include <algorithm>
#include <set>

#include "ir.h"

namespace b2x {
namespace {
[[noreturn]] void bad(const Op& op, const std::string& msg) {
  throw CompileError(kInvalidArgument, std::string(op_name(op.kind)) + " (line " + std::to_string(op.line) + "): " + msg);
}
void need(const Op& op, bool cond, const std::string& msg) { if (!cond) bad(op, msg); }
bool unique_in_range(const std::vector<int64_t>& v, int64_t n) {
  std::set<int64_t> s;
  for (auto d : v) { if (d < 0 || d >= n || !s.insert(d).second) return false; }
  return true;
}
}  // namespace

void verify_module(const Module& m) {
  for (auto& up : m.ops) {
    const Op& op = *up;
    auto& in = op.operands;
    auto& out = op.results;
    switch (op.kind) {
      case OpKind::RETURN: break;
      case OpKind::CONSTANT: need(op, out.size() == 1, "needs one result"); break;
      case OpKind::IOTA:
        need(op, out.size() == 1 && op.iota_dim >= 0 && op.iota_dim < out[0]->type.rank(), "iota dimension out of range");
        need(op, out[0]->type.dtype != DType::PRED, "iota of i1 is not defined");
        break;
      case OpKind::REPLICA_ID: case OpKind::PARTITION_ID:
        need(op, out.size() == 1 && out[0]->type.rank() == 0 && out[0]->type.dtype == DType::U32, "result must be tensor<ui32>");
        break;
      case OpKind::BROADCAST_IN_DIM: {
        need(op, in.size() == 1 && out.size() == 1, "needs one operand and one result");
        auto& a = in[0]->type; auto& r = out[0]->type;
        need(op, a.dtype == r.dtype, "element types differ");
        need(op, (int)op.dims.size() == a.rank(), "dims must have one entry per operand dimension");
        need(op, unique_in_range(op.dims, r.rank()), "dims must be unique and within the result rank");
        for (int i = 0; i < a.rank(); i++)
          need(op, a.dims[i] == 1 || a.dims[i] == r.dims[op.dims[i]], "operand dimension " + std::to_string(i) + " is neither 1 nor the matching result dimension");
        break;
      }
      case OpKind::TRANSPOSE: {
        need(op, in.size() == 1 && out.size() == 1, "needs one operand and one result");
        auto& a = in[0]->type; auto& r = out[0]->type;
        need(op, a.dtype == r.dtype && a.rank() == r.rank() && (int)op.dims.size() == a.rank() && unique_in_range(op.dims, a.rank()), "bad permutation");
        for (int i = 0; i < r.rank(); i++) need(op, r.dims[i] == a.dims[op.dims[i]], "result shape is not the permuted operand shape");
        break;
      }
      case OpKind::RESHAPE:
        need(op, in.size() == 1 && out.size() == 1 && in[0]->type.dtype == out[0]->type.dtype &&
                     in[0]->type.num_elements() == out[0]->type.num_elements(), "element counts differ");
        break;
      case OpKind::DOT_GENERAL: {
        need(op, in.size() == 2 && out.size() == 1, "needs two operands and one result");
        auto& a = in[0]->type; auto& b = in[1]->type; auto& r = out[0]->type;
        need(op, op.lhs_batch.size() == op.rhs_batch.size() && op.lhs_contract.size() == op.rhs_contract.size(), "dimension-number lists differ in length");
        std::vector<int64_t> la = op.lhs_batch, lb = op.rhs_batch;
        la.insert(la.end(), op.lhs_contract.begin(), op.lhs_contract.end());
        lb.insert(lb.end(), op.rhs_contract.begin(), op.rhs_contract.end());
        need(op, unique_in_range(la, a.rank()) && unique_in_range(lb, b.rank()), "batching/contracting dimensions must be unique and in range");
        std::vector<int64_t> expect;
        for (size_t i = 0; i < op.lhs_batch.size(); i++) {
          need(op, a.dims[op.lhs_batch[i]] == b.dims[op.rhs_batch[i]], "batch dimension sizes differ");
          expect.push_back(a.dims[op.lhs_batch[i]]);
        }
        for (size_t i = 0; i < op.lhs_contract.size(); i++)
          need(op, a.dims[op.lhs_contract[i]] == b.dims[op.rhs_contract[i]], "contracting dimension sizes differ");
        for (int i = 0; i < a.rank(); i++) if (std::find(la.begin(), la.end(), i) == la.end()) expect.push_back(a.dims[i]);
        for (int i = 0; i < b.rank(); i++) if (std::find(lb.begin(), lb.end(), i) == lb.end()) expect.push_back(b.dims[i]);
        need(op, r.dims == expect, "result shape must be batch dims, then lhs free dims, then rhs free dims; got " + r.str());
        break;
      }
      case OpKind::REDUCE: {
        need(op, in.size() == 2 && out.size() == 1, "only single-input reductions are supported");
        auto& a = in[0]->type; auto& r = out[0]->type;
        need(op, in[1]->type.rank() == 0 && in[1]->type.dtype == a.dtype && r.dtype == a.dtype, "init value must be a scalar of the input element type");
        need(op, unique_in_range(op.dims, a.rank()), "reduction dimensions must be unique and in range");
        std::vector<int64_t> expect;
        for (int i = 0; i < a.rank(); i++) if (std::find(op.dims.begin(), op.dims.end(), i) == op.dims.end()) expect.push_back(a.dims[i]);
        need(op, r.dims == expect, "result shape must be the input shape without the reduced dimensions");
        break;
      }
      case OpKind::ALL_REDUCE:
        need(op, in.size() == out.size() && !in.empty(), "needs as many results as operands");
        for (size_t i = 0; i < in.size(); i++) need(op, in[i]->type == out[i]->type, "result types must equal operand types");
        break;
      case OpKind::ALL_GATHER: {
        need(op, in.size() == out.size() && !in.empty(), "needs as many results as operands");
        need(op, !op.replica_groups.empty(), "needs replica_groups");
        int64_t g = (int64_t)op.replica_groups[0].size();
        for (size_t i = 0; i < in.size(); i++) {
          auto& a = in[i]->type; auto& r = out[i]->type;
          need(op, a.dtype == r.dtype && a.rank() == r.rank() && op.iota_dim >= 0 && op.iota_dim < a.rank(), "bad all_gather_dim");
          for (int d = 0; d < a.rank(); d++)
            need(op, r.dims[d] == (d == op.iota_dim ? a.dims[d] * g : a.dims[d]), "result shape must be the operand shape scaled by the group size along all_gather_dim");
        }
        break;
      }
      case OpKind::CONVERT:
        need(op, in.size() == 1 && out.size() == 1 && in[0]->type.dims == out[0]->type.dims, "shapes differ");
        break;
      case OpKind::COMPARE:
        need(op, in.size() == 2 && out.size() == 1 && in[0]->type == in[1]->type, "operands must have the same type");
        need(op, out[0]->type.dtype == DType::PRED && out[0]->type.dims == in[0]->type.dims, "result must be an i1 tensor of the operand shape");
        break;
      case OpKind::SELECT:
        need(op, in.size() == 3 && out.size() == 1 && in[1]->type == in[2]->type && out[0]->type == in[1]->type, "on_true, on_false and the result must have the same type");
        need(op, in[0]->type.dtype == DType::PRED && (in[0]->type.rank() == 0 || in[0]->type.dims == in[1]->type.dims), "predicate must be i1 and scalar or of the result shape");
        break;
      case OpKind::CLAMP:
        need(op, in.size() == 3 && out.size() == 1 && out[0]->type == in[1]->type, "result must have the operand type");
        for (int i : {0, 2})
          need(op, in[i]->type.dtype == in[1]->type.dtype && (in[i]->type.rank() == 0 || in[i]->type.dims == in[1]->type.dims), "min/max must be scalars or of the operand shape");
        break;
      default: {  // same-type elementwise
        need(op, out.size() == 1 && !in.empty(), "needs operands and one result");
        for (auto v : in) need(op, v->type == out[0]->type, "operand type " + v->type.str() + " differs from result type " + out[0]->type.str());
        break;
      }
    }
    for (auto r : out) need(op, r->type.dtype != DType::INVALID, "invalid result type");
  }
  (void)m;
}

}  // namespace b2x
