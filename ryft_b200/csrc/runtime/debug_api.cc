// Host-only helpers exported from libb2x_kernels.so: compile a module and return the launch plan as text.  Needs
// no GPU, so the front end and the planner can be checked anywhere.
#include <cstring>
#include <string>

#include "plan.h"

extern "C" __attribute__((visibility("default"))) int b2x_plan_dump(const char* mlir, size_t mlir_size, int num_replicas, char* out, size_t out_cap,
                                                                     size_t* out_size) {
  std::string text;
  int code = 0;
  try {
    auto m = b2x::parse_module(std::string(mlir, mlir_size));
    b2x::PlanOptions o;
    o.num_replicas = num_replicas > 0 ? num_replicas : 1;
    text = b2x::build_plan(*m, o, 0).dump();
  } catch (const b2x::CompileError& e) {
    code = e.code;
    text = e.what();
  } catch (const std::exception& e) {
    code = 13;
    text = e.what();
  }
  if (out_size) *out_size = text.size();
  if (out && out_cap) {
    size_t n = text.size() < out_cap - 1 ? text.size() : out_cap - 1;
    memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return code;
}
