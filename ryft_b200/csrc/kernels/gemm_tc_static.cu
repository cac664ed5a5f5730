// Build-time specialised epilogues of the tcgen05 GEMM: one kernel per (program, tile width) pair listed in
// vm_static_table.h.  Kept in its own translation unit so that it compiles in parallel with the interpreter variant.
#include "gemm_tc.cuh"

namespace b2x {

template <int BN> struct TcStages { static constexpr int value = BN == 256 ? 4 : (BN == 128 ? 6 : 8); };

int launch_tc_static(int id, int BN, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, const B2xVmProgram& epi, int32_t* status,
                     cudaStream_t stream) {
#define X(I, W) if (id == I && BN == W) return launch_tc<W, TcStages<W>::value, false, I>(tmA, tmB, p, epi, status, stream);
  B2X_VM_STATIC_GEMM(X)
#undef X
  (void)id; (void)BN; (void)tmA; (void)tmB; (void)p; (void)epi; (void)status; (void)stream;
  return -1;
}

// f32 operands (3xTF32): only the program that stores the accumulator as f32 is specialised, so that the plain
// `dot_general` on f32 tensors leaves through the bulk-store epilogue instead of the interpreter.
template <int ID>
constexpr bool tc_plain_f32_store() {
  if (VmStatic<ID>::n != 2) return false;
  const VmSig a = VmStatic<ID>::at(0), b = VmStatic<ID>::at(1);
  return a.op == VM_LOAD && a.src_kind == VM_SRC_ACC0 && b.op == VM_STORE && b.src_kind == VM_SRC_TENSOR && VmStatic<ID>::elem(b.src_idx) == EL_F32;
}
template <int ID, int W>
static int launch_tf32_if_plain(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, const B2xVmProgram& epi, int32_t* status,
                                cudaStream_t stream) {
  if constexpr (tc_plain_f32_store<ID>()) return launch_tc<W, TcStages<W>::value, true, ID>(tmA, tmB, p, epi, status, stream);
  else return -1;
}
int launch_tc_static_tf32(int id, int BN, const CUtensorMap& tmA, const CUtensorMap& tmB, const TcParams& p, const B2xVmProgram& epi, int32_t* status,
                          cudaStream_t stream) {
#define X(I, W) if (id == I && BN == W) return launch_tf32_if_plain<I, W>(tmA, tmB, p, epi, status, stream);
  B2X_VM_STATIC_GEMM(X)
#undef X
  (void)id; (void)BN; (void)tmA; (void)tmB; (void)p; (void)epi; (void)status; (void)stream;
  return -1;
}

bool tc_static_has(int id, int BN) {
#define X(I, W) if (id == I && BN == W) return true;
  B2X_VM_STATIC_GEMM(X)
#undef X
  (void)id; (void)BN;
  return false;
}
bool tc_static_has_tf32(int id, int BN) {
#define X(I, W) if (id == I && BN == W) return tc_plain_f32_store<I>();
  B2X_VM_STATIC_GEMM(X)
#undef X
  (void)id; (void)BN;
  return false;
}
int tc_static_stores(int id) {
#define X(I, W) if (id == I) return vm_static_stores<I>();
  B2X_VM_STATIC_GEMM(X)
#undef X
  (void)id;
  return 0;
}

}  // namespace b2x
