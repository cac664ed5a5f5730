// Host-only helpers exported from libb2x_kernels.so: compile a module and return the launch plan as text.  Needs
// no GPU, so the front end and the planner can be checked anywhere.
#include <cstdlib>
#include <cstring>
#include <string>

#include "plan.h"

// The switches the plugin reads at compile time, so that the host-only helpers below show the plan that would run.
static b2x::PlanOptions options_from_environment(int num_replicas) {
  b2x::PlanOptions o;
  o.num_replicas = num_replicas > 0 ? num_replicas : 1;
  if (const char* f = getenv("B2X_FUSED_ATTENTION")) o.allow_fused_attention = strcmp(f, "0") != 0;
  if (const char* f = getenv("B2X_EPILOGUE_FUSION")) o.allow_epilogue_fusion = strcmp(f, "0") != 0;
  if (const char* g = getenv("B2X_GEMM")) o.allow_tensor_core = strcmp(g, "simt") != 0;
  if (const char* f = getenv("B2X_PRECISE_MATH")) o.precise_math = strcmp(f, "0") != 0;
  return o;
}

extern "C" __attribute__((visibility("default"))) int b2x_plan_dump(const char* mlir, size_t mlir_size, int num_replicas, char* out, size_t out_cap,
                                                                     size_t* out_size) {
  std::string text;
  int code = 0;
  try {
    auto m = b2x::parse_module(std::string(mlir, mlir_size));
    b2x::PlanOptions o = options_from_environment(num_replicas);
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

// Lists the fused-elementwise programs of a module's launch plan, one per line:
//   role|BN|vec|hash|n_instr|op.src_kind.src_idx.aux.tc.rnd,...|elem,elem,...|label
// role is elementwise, reduce or gemm_tc.  Input of gen_vm_static.py, which builds the table of specialised programs.
extern "C" __attribute__((visibility("default"))) int b2x_plan_signatures(const char* mlir, size_t mlir_size, int num_replicas, char* out, size_t out_cap,
                                                                           size_t* out_size) {
  std::string text;
  int code = 0;
  try {
    auto m = b2x::parse_module(std::string(mlir, mlir_size));
    b2x::PlanOptions o;
    o.num_replicas = num_replicas > 0 ? num_replicas : 1;
    b2x::Plan plan = b2x::build_plan(*m, o, 0);
    for (auto& s : plan.steps) {
      const char* role = nullptr;
      int bn = 0;
      if (s.kind == b2x::StepKind::ELEMENTWISE) role = "elementwise";
      else if (s.kind == b2x::StepKind::REDUCE) role = "reduce";
      else if (s.kind == b2x::StepKind::GEMM && s.g_tensor_core && !s.g_split_f32) { role = "gemm_tc"; bn = s.gN >= 256 ? 256 : (s.gN >= 128 ? 128 : 64); }
      if (!role) continue;
      const B2xVmProgram& P = s.vm.prog;
      uint64_t h = 1469598103934665603ull;
      auto mix = [&](uint8_t b) { h ^= b; h *= 1099511628211ull; };
      mix((uint8_t)P.n_instr);
      std::string code_s, elems;
      for (int i = 0; i < P.n_instr; i++) {
        const B2xVmInstr& I = P.code[i];
        mix(I.op); mix(I.src_kind); mix(I.src_idx); mix(I.aux); mix(I.tc); mix(I.rnd);
        if (i) code_s += ",";
        code_s += std::to_string(I.op) + "." + std::to_string(I.src_kind) + "." + std::to_string(I.src_idx) + "." + std::to_string(I.aux) + "." +
                  std::to_string(I.tc) + "." + std::to_string(I.rnd);
      }
      mix((uint8_t)P.n_tensors);
      for (int t = 0; t < P.n_tensors; t++) { mix(P.tensors[t].elem); if (t) elems += ","; elems += std::to_string(P.tensors[t].elem); }
      text += std::string(role) + "|" + std::to_string(bn) + "|" + std::to_string(s.vm.vec) + "|" + std::to_string(h) + "|" + std::to_string(P.n_instr) + "|" + code_s +
              "|" + elems + "|" + s.label + "\n";
    }
  } catch (const b2x::CompileError& e) {
    code = e.code;
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

#include "../../../include/b2x_kernels.h"

// Lists, one line per tensor-core GEMM step of the module's plan, the kernel variant the launcher will pick:
//   label|M|N|K|batch|BN|static id|epilogue groups|transposed|group_m|m tiles|n tiles|k blocks|stores|ctas
extern "C" __attribute__((visibility("default"))) int b2x_plan_routes(const char* mlir, size_t mlir_size, int num_replicas, char* out, size_t out_cap,
                                                                       size_t* out_size) {
  std::string text;
  int code = 0;
  try {
    auto m = b2x::parse_module(std::string(mlir, mlir_size));
    b2x::PlanOptions o = options_from_environment(num_replicas);
    b2x::Plan plan = b2x::build_plan(*m, o, 0);
    for (auto& s : plan.steps) {
      if (s.kind != b2x::StepKind::GEMM || !s.g_tensor_core) continue;
      B2xGemmArgs ga{};
      ga.elem = (uint8_t)s.ga.dtype;
      ga.batch = s.gB; ga.M = s.gM; ga.N = s.gN; ga.K = s.gK;
      ga.a_batch_stride = s.ga.batch_stride; ga.a_row_stride = s.ga.row_stride; ga.a_k_stride = s.ga.k_stride;
      ga.b_batch_stride = s.gb.batch_stride; ga.b_row_stride = s.gb.row_stride; ga.b_k_stride = s.gb.k_stride;
      if (s.g_split_f32) {
        ga.K = 3 * s.gK;
        ga.a_k_stride = 1; ga.a_row_stride = ga.K; ga.a_batch_stride = s.gM * ga.K;
        ga.b_k_stride = 1; ga.b_row_stride = ga.K; ga.b_batch_stride = s.gN * ga.K;
      }
      int32_t r[12] = {};
      int rc = b2x_gemm_tc_route(&ga, &s.vm.prog, r);
      text += s.label + "|" + std::to_string(s.gM) + "|" + std::to_string(s.gN) + "|" + std::to_string(ga.K) + "|" + std::to_string(s.gB);
      for (int i = 0; i < 11; i++) text += "|" + std::to_string(rc ? -1 : r[i]);
      text += "\n";
    }
  } catch (const b2x::CompileError& e) {
    code = e.code;
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
