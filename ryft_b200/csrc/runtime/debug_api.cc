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

#include "objects.h"

// Parses a serialized CompileOptionsProto the way PJRT_Client_Compile does and reports the fields the executor
// honours: out[0] = replica_count, out[1] = partition_count, out[2] = device_ordinal, out[3] = precision,
// out[4] = number of device-assignment entries, out[5..] = the assignment (replica -> device id), up to cap entries.
extern "C" __attribute__((visibility("default"))) int b2x_debug_parse_compile_options(const char* data, size_t size, int64_t* out, size_t cap) {
  b2x::CompileOptions co;
  std::string err;
  if (!b2x::parse_compile_options(data, size, &co, &err)) return 3;
  if (cap < 5) return 3;
  out[0] = co.num_replicas; out[1] = co.num_partitions; out[2] = co.device_ordinal; out[3] = co.precision;
  size_t n = 0;
  if (co.has_device_assignment && !co.da_devices.empty())
    for (auto d : co.da_devices[0]) { if (5 + n < cap) out[5 + n] = d; n++; }
  out[4] = (int64_t)n;
  return 0;
}
