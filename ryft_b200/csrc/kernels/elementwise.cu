// Standalone fused elementwise kernel: one pass over HBM for a whole group of StableHLO elementwise ops.
//
// HBM-bound by design: every operand is read once with 128-bit (or 2 x 128-bit) coalesced vector accesses, all
// intermediate values stay in registers (vm.cuh), and every output is written once.  Algorithmic bytes per element
// = sum of operand and result element sizes.  The grid is a whole number of waves over the 148 SMs and threads walk
// the tensor with a grid stride so that consecutive warps touch consecutive 512-byte or 1-KiB spans.
#include "../../../include/b2x_kernels.h"
#include "common.cuh"
#include "vm.cuh"

namespace b2x {
std::atomic<int64_t> g_launch_count{0};

template <int V, int ID>
__global__ void __launch_bounds__(256) k_elementwise(const __grid_constant__ B2xVmProgram P, uint64_t n_vec) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  uint32_t zero[V];
#pragma unroll
  for (int j = 0; j < V; j++) zero[j] = 0;
  for (uint64_t v = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += stride) {
    uint32_t acc[V];
    vm_run<V, ID>(P, v * V, zero, acc);
  }
}
}  // namespace b2x

extern "C" int b2x_launch_elementwise(const B2xVmProgram* prog, int64_t n_elements, int vec, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_elements <= 0) return 0;
  if (vec != 1 && vec != 4 && vec != 8) return (int)cudaErrorInvalidValue;
  if (n_elements % vec != 0) return (int)cudaErrorInvalidValue;
  uint64_t n_vec = (uint64_t)n_elements / vec;
  // 8 resident CTAs of 256 threads per SM; cap the grid at 4 waves and let the grid-stride loop do the rest
  uint64_t blocks = (n_vec + 255) / 256;
  uint64_t cap = (uint64_t)kNumSms * 8 * 4;
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks), block(256);
  if (vec == 8) {
    // a program whose structure was known at build time runs as straight-line code, anything else is interpreted
    switch (vm_static_enabled() ? vm_static_lookup(vm_signature_hash(*prog)) : 0) {
#define X(I) case I: k_elementwise<8, I><<<grid, block, 0, stream>>>(*prog, n_vec); break;
      B2X_VM_STATIC_ELEMENTWISE(X)
#undef X
      default: k_elementwise<8, 0><<<grid, block, 0, stream>>>(*prog, n_vec); break;
    }
  } else if (vec == 4) k_elementwise<4, 0><<<grid, block, 0, stream>>>(*prog, n_vec);
  else k_elementwise<1, 0><<<grid, block, 0, stream>>>(*prog, n_vec);
  count_launch();
  return (int)cudaGetLastError();
}

extern "C" int64_t b2x_kernel_launch_count(void) { return b2x::g_launch_count.load(); }
