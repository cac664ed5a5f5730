// Replays a launch plan on one device: binds buffer references to device pointers and enqueues each step's kernel on
// the device's compute stream; collectives go to the communication stream, bracketed by events, so that they overlap
// with later compute steps (reference call site: PJRT_LoadedExecutable_Execute,
// crates/ryft-pjrt/src/programs.rs:923-936).  Nothing here synchronises with the host.
#include "../../../include/b2x_kernels.h"
#include "nccl_dyn.h"
#include "objects.h"

namespace b2x {
namespace {

struct Binder {
  const std::vector<void*>& args;
  const std::vector<void*>& outs;
  char* arena;
  char* consts;
  void* operator()(const BufRef& b) const {
    switch (b.kind) {
      case BufRef::ARG: return (char*)args[b.index] + b.offset;
      case BufRef::OUT: return (char*)outs[b.index] + b.offset;
      case BufRef::TEMP: return arena + b.offset;
      case BufRef::CONST: return consts + b.offset;
      default: return nullptr;
    }
  }
};

void bind_program(const VmBinding& vm, const Binder& bind, B2xVmProgram* out) {
  *out = vm.prog;
  for (int t = 0; t < out->n_tensors; t++) out->tensors[t].ptr = bind(vm.bufs[t]);
}

PJRT_Error* kernel_error(int rc, const Step& s) {
  return make_error(PJRT_Error_Code_INTERNAL, "launching '" + s.label + "' failed: " + cudaGetErrorString((cudaError_t)rc));
}

}  // namespace

PJRT_Error* run_plan(PJRT_LoadedExecutable* le, int local_index, int replica, const std::vector<void*>& args,
                     const std::vector<void*>& outs) {
  PJRT_Device* dev = le->addressable[local_index];
  PJRT_LoadedExecutable::PerDevice& pd = le->per_device[local_index];
  const Plan& plan = le->core->plan_for(replica);
  B2X_CUDA(cudaSetDevice(dev->cuda_ordinal));
  Binder bind{args, outs, (char*)pd.arena, (char*)pd.consts};
  cudaStream_t cs = dev->compute;
  B2xVmProgram prog;
  std::vector<int> outstanding;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>>* timed = nullptr;
  if (pd.timing) { pd.timed.emplace_back(); timed = &pd.timed.back(); pd.last_args = args; pd.last_outs = outs; }
  for (const Step& s : plan.steps) {
    for (int w : s.wait_colls) B2X_CUDA(cudaStreamWaitEvent(cs, pd.coll_done[w], 0));
    const bool on_comm = s.kind == StepKind::ALL_REDUCE || s.kind == StepKind::ALL_GATHER;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    if (timed && !on_comm) { B2X_CUDA(cudaEventCreate(&t0)); B2X_CUDA(cudaEventCreate(&t1)); B2X_CUDA(cudaEventRecord(t0, cs)); }
    switch (s.kind) {
      case StepKind::ELEMENTWISE: {
        bind_program(s.vm, bind, &prog);
        int rc = b2x_launch_elementwise(&prog, s.vm.n_elements, s.vm.vec, cs);
        if (rc) return kernel_error(rc, s);
        break;
      }
      case StepKind::WIDE: {
        B2xWideOp w{};
        w.op = s.w_op; w.n_in = s.w_n_in; w.n_dims = (int)s.w_dims.size(); w.aux = s.w_aux; w.aux2 = s.w_aux2;
        w.out_elem = (uint8_t)s.w_out_dtype;
        w.n_elements = 1;
        for (size_t d = 0; d < s.w_dims.size(); d++) { w.dim[d] = s.w_dims[d]; w.n_elements *= s.w_dims[d]; }
        for (int k = 0; k < s.w_n_in; k++) {
          w.in_elem[k] = (uint8_t)s.w_in_dtype[k];
          w.in[k] = bind(s.w_in[k]);
          for (size_t d = 0; d < s.w_in_strides[k].size() && d < (size_t)B2X_WIDE_MAX_DIMS; d++) w.in_stride[k][d] = s.w_in_strides[k][d];
        }
        w.out = bind(s.w_out);
        w.imm = s.w_imm;
        int rc = b2x_launch_wide_elementwise(&w, cs);
        if (rc) return kernel_error(rc, s);
        break;
      }
      case StepKind::REDUCE: {
        if (s.wide) {
          int rc = b2x_launch_wide_reduce(bind(s.w_in[0]), (uint8_t)s.w_in_dtype[0], s.rA, s.rR, s.rB, (int)s.monoid,
                                          s.r_init_is_imm ? nullptr : bind(s.r_init_buf), s.w_imm, bind(s.r_out), cs);
          if (rc) return kernel_error(rc, s);
          break;
        }
        bind_program(s.vm, bind, &prog);
        B2xReduceArgs ra{};
        ra.A = s.rA; ra.R = s.rR; ra.B = s.rB;
        ra.monoid = (uint8_t)s.monoid; ra.cls = s.rcls;
        ra.out_elem = (uint8_t)s.r_out_dtype; ra.init_elem = (uint8_t)s.r_init_dtype;
        ra.init_imm = s.r_init_imm;
        ra.init_ptr = s.r_init_is_imm ? nullptr : bind(s.r_init_buf);
        ra.out = s.r_out.valid() ? bind(s.r_out) : nullptr;
        ra.scratch = s.scratch.valid() ? bind(s.scratch) : nullptr;
        ra.vec = s.vm.vec;
        B2xVmProgram post;
        if (s.has_post) { bind_program(s.post, bind, &post); ra.host_post = &post; }
        int rc = b2x_launch_reduce(&prog, &ra, cs);
        if (rc) return kernel_error(rc, s);
        break;
      }
      case StepKind::GEMM: {
        bind_program(s.vm, bind, &prog);
        B2xGemmArgs ga{};
        ga.a = bind(s.ga.buf); ga.b = bind(s.gb.buf);
        ga.elem = (uint8_t)s.ga.dtype;
        ga.batch = s.gB; ga.M = s.gM; ga.N = s.gN; ga.K = s.gK;
        ga.a_batch_stride = s.ga.batch_stride; ga.a_row_stride = s.ga.row_stride; ga.a_k_stride = s.ga.k_stride;
        ga.b_batch_stride = s.gb.batch_stride; ga.b_row_stride = s.gb.row_stride; ga.b_k_stride = s.gb.k_stride;
        int rc;
        if (s.wide) {
          rc = b2x_launch_wide_gemm(&ga, (uint8_t)s.w_out_dtype, bind(s.w_out), cs);
        } else if (s.g_tensor_core) {
          if (s.g_split_f32) {
            // A' = [hi | hi | lo], B' = [hi | lo | hi]: K-major rows of 3K floats in scratch
            float* a_split = (float*)bind(s.scratch);
            size_t a_elems = (size_t)(s.gB * s.gM * 3 * s.gK);
            float* b_split = a_split + ((a_elems + 255) / 256) * 256;
            rc = b2x_launch_split_f32(&ga, a_split, b_split, cs);
            if (rc) return kernel_error(rc, s);
            ga.a = a_split; ga.b = b_split;
            ga.K = 3 * s.gK;
            ga.a_k_stride = 1; ga.a_row_stride = ga.K; ga.a_batch_stride = s.gM * ga.K;
            ga.b_k_stride = 1; ga.b_row_stride = ga.K; ga.b_batch_stride = s.gN * ga.K;
          }
          rc = b2x_launch_gemm_tc(&ga, &prog, dev->status_dev, cs);
        } else {
          rc = b2x_launch_gemm_simt(&ga, &prog, s.vm.vec, cs);
        }
        if (rc) return kernel_error(rc, s);
        break;
      }
      case StepKind::ATTENTION: {
        B2xAttentionArgs aa{};
        aa.q = bind(s.aq); aa.k = bind(s.ak); aa.v = bind(s.av); aa.o = bind(s.ao);
        aa.BH = s.aBH; aa.Sq = s.aSq; aa.Sk = s.aSk; aa.D = s.aD;
        aa.scale = s.a_scale; aa.causal = s.a_causal ? 1 : 0;
        int rc = b2x_launch_attention(&aa, dev->status_dev, cs);
        if (rc) return kernel_error(rc, s);
        break;
      }
      case StepKind::ALL_REDUCE: case StepKind::ALL_GATHER: {
        // the group this replica belongs to, as global device ids in rank order
        std::vector<int> group;
        for (auto& g : s.replica_groups) {
          bool mine = false;
          for (auto r : g) if ((int)r == replica) mine = true;
          if (!mine) continue;
          for (auto r : g) group.push_back(le->core->device_assignment[(size_t)r]);
        }
        if (group.empty()) return make_error(PJRT_Error_Code_INTERNAL, "replica is in no replica group");
        B2X_CUDA(cudaEventRecord(pd.fork, cs));
        B2X_CUDA(cudaStreamWaitEvent(dev->comm, pd.fork, 0));
        if (timed) { B2X_CUDA(cudaEventCreate(&t0)); B2X_CUDA(cudaEventCreate(&t1)); B2X_CUDA(cudaEventRecord(t0, dev->comm)); }
        for (auto& c : s.colls) {
          void* src = bind(c.src);
          void* dst = bind(c.dst);
          if (group.size() == 1) {
            if (src != dst) B2X_CUDA(cudaMemcpyAsync(dst, src, (size_t)c.count * dtype_size(c.dtype), cudaMemcpyDeviceToDevice, dev->comm));
            continue;
          }
          void* comm = le->client->nccl ? le->client->nccl->comm_for(group, dev->desc.id) : nullptr;
          if (!comm) return make_error(PJRT_Error_Code_INTERNAL, "no communicator for this replica group");
          PJRT_Error* e = s.kind == StepKind::ALL_REDUCE
                              ? le->client->nccl->all_reduce(comm, src, dst, (size_t)c.count, (int)c.dtype, (int)s.monoid, dev->comm)
                              : le->client->nccl->all_gather(comm, src, dst, (size_t)c.count, (int)c.dtype, dev->comm);
          if (e) return e;
        }
        if (timed) B2X_CUDA(cudaEventRecord(t1, dev->comm));
        B2X_CUDA(cudaEventRecord(pd.coll_done[s.coll_id], dev->comm));
        if (!s.coll_detached) outstanding.push_back(s.coll_id);
        break;
      }
      case StepKind::COPY:
        B2X_CUDA(cudaMemcpyAsync(bind(s.c_dst), bind(s.c_src), (size_t)s.c_bytes, cudaMemcpyDeviceToDevice, cs));
        break;
    }
    if (timed) {
      if (!on_comm) B2X_CUDA(cudaEventRecord(t1, cs));
      timed->push_back({t0, t1});
    }
  }
  for (int id : outstanding) B2X_CUDA(cudaStreamWaitEvent(cs, pd.coll_done[id], 0));
  return nullptr;
}

}  // namespace b2x
