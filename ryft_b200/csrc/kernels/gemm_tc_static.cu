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

}  // namespace b2x
