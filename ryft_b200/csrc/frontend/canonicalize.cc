// Exact algebraic rewrites applied to a parsed module before planning.
//
//   multiply(all_reduce_sum(x), splat(2^k))  ->  all_reduce_sum(multiply(x, splat(2^k)))
//
// The data-parallel gradient step divides the reduced gradients by the replica count.  Scaling by a power of two
// commutes exactly with floating-point addition (barring underflow), so the scale can move in front of the collective,
// where it fuses into the epilogue of the GEMM that produces the gradient; the collective then runs in place on the
// output buffer and no separate scaling pass over the gradients remains.  Other constants are left alone.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "ir.h"

namespace b2x {
namespace {

bool splat_value(const Value* v, float* out) {
  if (!v->def) return false;
  const Op* d = v->def;
  if (d->kind == OpKind::BROADCAST_IN_DIM && d->operands[0]->type.num_elements() == 1) return splat_value(d->operands[0], out);
  if (d->kind != OpKind::CONSTANT || !d->splat) return false;
  if (v->type.dtype == DType::F32) { memcpy(out, d->const_data.data(), 4); return true; }
  if (v->type.dtype == DType::BF16) { uint16_t h; memcpy(&h, d->const_data.data(), 2); uint32_t u = (uint32_t)h << 16; memcpy(out, &u, 4); return true; }
  return false;
}
bool is_power_of_two(float c) {
  if (!(c > 0.f) || !std::isfinite(c)) return false;
  int e;
  return std::frexp(c, &e) == 0.5f;
}
void remove_user(Value* v, Op* op) {
  auto it = std::find(v->users.begin(), v->users.end(), op);
  if (it != v->users.end()) v->users.erase(it);
}

}  // namespace

void canonicalize(Module& m) {
  for (size_t idx = 0; idx < m.ops.size(); idx++) {
    Op* ar = m.ops[idx].get();
    if (ar->kind != OpKind::ALL_REDUCE || ar->monoid != Monoid::ADD) continue;
    for (size_t i = 0; i < ar->results.size(); i++) {
      Value* r = ar->results[i];
      Value* x = ar->operands[i];
      if (r->users.size() != 1 || (x->type.dtype != DType::F32 && x->type.dtype != DType::BF16)) continue;
      Op* mul = r->users[0];
      if (mul->kind != OpKind::MULTIPLY || mul->operands[0] == mul->operands[1]) continue;
      Value* other = mul->operands[0] == r ? mul->operands[1] : mul->operands[0];
      float c = 0.f;
      if (!splat_value(other, &c) || !is_power_of_two(c)) continue;
      // constant and multiply in front of the collective
      std::unique_ptr<Op> k(new Op());
      k->kind = OpKind::CONSTANT;
      k->line = ar->line;
      k->splat = true;
      if (x->type.dtype == DType::F32) { k->const_data.resize(4); memcpy(k->const_data.data(), &c, 4); }
      else { uint32_t u; memcpy(&u, &c, 4); uint16_t h = (uint16_t)(u >> 16); k->const_data.resize(2); memcpy(k->const_data.data(), &h, 2); }
      Value* kv = m.new_value(x->type);
      kv->def = k.get();
      kv->name = r->name + "_scale";
      k->results.push_back(kv);
      std::unique_ptr<Op> y(new Op());
      y->kind = OpKind::MULTIPLY;
      y->line = ar->line;
      y->operands = {x, kv};
      Value* yv = m.new_value(x->type);
      yv->def = y.get();
      yv->name = r->name + "_scaled";
      y->results.push_back(yv);
      kv->users.push_back(y.get());
      remove_user(x, ar);
      x->users.push_back(y.get());
      yv->users.push_back(ar);
      ar->operands[i] = yv;
      // uses of the old product now read the collective's result
      Value* prod = mul->results[0];
      r->users.clear();
      for (Op* u : prod->users) {
        for (auto& o : u->operands) if (o == prod) o = r;
        r->users.push_back(u);
      }
      for (auto& o : m.outputs) if (o == prod) o = r;
      prod->users.clear();
      remove_user(other, mul);
      auto mit = std::find_if(m.ops.begin(), m.ops.end(), [&](const std::unique_ptr<Op>& p) { return p.get() == mul; });
      if (mit != m.ops.end()) m.ops.erase(mit);   // the multiply sits behind the collective: indices up to idx are unaffected
      m.ops.insert(m.ops.begin() + idx, std::move(y));
      m.ops.insert(m.ops.begin() + idx, std::move(k));
      idx += 2;
    }
  }
}

}  // namespace b2x
