// CUDA-core strided batched GEMM with the fused-elementwise epilogue.
//
// This is the general path of stablehlo.dot_general: any element type the executor supports (f32/bf16/f16 with f32
// accumulation, 8/16/32-bit integers with 32-bit accumulation), any strides, any sizes (down to the 2x3x2 example
// in the reference's README).  Large aligned bf16/f16/f32 problems go to the tcgen05 kernel instead.
// 64x64 output tile per CTA, 16-deep k-slabs staged in shared memory, 4x4 register tile per thread.
#include "../../../include/b2x_kernels.h"
#include "common.cuh"
#include "vm.cuh"

namespace b2x {

struct GemmK {
  const char* a; const char* b;
  int elem, es;
  int64_t batch, M, N, K;
  int64_t sab, sam, sak, sbb, sbn, sbk;
};

__device__ __forceinline__ uint32_t ld_elem(const char* base, int64_t idx, int elem, int es) {
  uint32_t raw;
  const char* p = base + idx * es;
  if (es == 4) raw = __ldg((const uint32_t*)p); else if (es == 2) raw = __ldg((const uint16_t*)p); else raw = __ldg((const uint8_t*)p);
  return vm_decode(raw, (uint8_t)elem);
}

template <bool INT, int V>
__global__ void __launch_bounds__(256) k_gemm_simt(const __grid_constant__ GemmK G, const __grid_constant__ B2xVmProgram P) {
  __shared__ uint32_t As[16][64 + 4];
  __shared__ uint32_t Bs[16][64 + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  for (int64_t bi = blockIdx.z; bi < G.batch; bi += gridDim.z) {
    float cf[4][4];
    int ci[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) { cf[i][j] = 0.f; ci[i][j] = 0; }
    for (int64_t k0 = 0; k0 < G.K; k0 += 16) {
      // stage A[64 x 16] and B[16 x 64]; the thread->element map follows whichever stride is unit for coalescing
#pragma unroll
      for (int e = 0; e < 4; e++) {
        int idx = threadIdx.x + e * 256;
        int mm, kk;
        if (G.sak == 1) { kk = idx & 15; mm = idx >> 4; } else { mm = idx & 63; kk = idx >> 6; }
        int64_t m = m0 + mm, k = k0 + kk;
        uint32_t v = 0;
        if (m < G.M && k < G.K) v = ld_elem(G.a, bi * G.sab + m * G.sam + k * G.sak, G.elem, G.es);
        As[kk][mm] = v;
      }
#pragma unroll
      for (int e = 0; e < 4; e++) {
        int idx = threadIdx.x + e * 256;
        int nn, kk;
        if (G.sbk == 1) { kk = idx & 15; nn = idx >> 4; } else { nn = idx & 63; kk = idx >> 6; }
        int64_t n = n0 + nn, k = k0 + kk;
        uint32_t v = 0;
        if (n < G.N && k < G.K) v = ld_elem(G.b, bi * G.sbb + n * G.sbn + k * G.sbk, G.elem, G.es);
        Bs[kk][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < 16; kk++) {
        uint32_t av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) {
            if (INT) ci[i][j] += (int)av[i] * (int)bv[j];
            else cf[i][j] = fmaf(u2f(av[i]), u2f(bv[j]), cf[i][j]);
          }
      }
      __syncthreads();
    }
    // epilogue: the fused elementwise program consumes the accumulator and performs the stores
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t m = m0 + ty * 4 + i;
      if (m >= G.M) continue;
      const int64_t n = n0 + tx * 4;
      if (V == 4) {
        if (n < G.N) {
          uint32_t a0[4], acc[4];
#pragma unroll
          for (int j = 0; j < 4; j++) a0[j] = INT ? (uint32_t)ci[i][j] : f2u(cf[i][j]);
          vm_run<4>(P, (uint64_t)((bi * G.M + m) * G.N + n), a0, acc);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if (n + j < G.N) {
            uint32_t a0[1], acc[1];
            a0[0] = INT ? (uint32_t)ci[i][j] : f2u(cf[i][j]);
            vm_run<1>(P, (uint64_t)((bi * G.M + m) * G.N + n + j), a0, acc);
          }
        }
      }
    }
  }
}

}  // namespace b2x

extern "C" int b2x_launch_gemm_simt(const B2xGemmArgs* a, const B2xVmProgram* epilogue, int vec, b2x_stream_t stream_) {
  using namespace b2x;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->batch <= 0 || a->M <= 0 || a->N <= 0) return 0;
  GemmK G{};
  G.a = (const char*)a->a; G.b = (const char*)a->b;
  G.elem = a->elem;
  switch (a->elem) {
    case EL_F32: case EL_S32: case EL_U32: G.es = 4; break;
    case EL_BF16: case EL_F16: case EL_S16: case EL_U16: G.es = 2; break;
    case EL_S8: case EL_U8: case EL_PRED: G.es = 1; break;
    default: return (int)cudaErrorInvalidValue;
  }
  const bool is_int = !(a->elem == EL_F32 || a->elem == EL_BF16 || a->elem == EL_F16);
  G.batch = a->batch; G.M = a->M; G.N = a->N; G.K = a->K;
  G.sab = a->a_batch_stride; G.sam = a->a_row_stride; G.sak = a->a_k_stride;
  G.sbb = a->b_batch_stride; G.sbn = a->b_row_stride; G.sbk = a->b_k_stride;
  int64_t gy = (a->M + 63) / 64;
  if (gy > 65535) return (int)cudaErrorInvalidValue;
  dim3 grid((unsigned)((a->N + 63) / 64), (unsigned)gy, (unsigned)(a->batch > 1024 ? 1024 : a->batch)), block(256);
  const bool v4 = (vec >= 4) && (a->N % 4 == 0);
  if (is_int) { if (v4) k_gemm_simt<true, 4><<<grid, block, 0, stream>>>(G, *epilogue); else k_gemm_simt<true, 1><<<grid, block, 0, stream>>>(G, *epilogue); }
  else { if (v4) k_gemm_simt<false, 4><<<grid, block, 0, stream>>>(G, *epilogue); else k_gemm_simt<false, 1><<<grid, block, 0, stream>>>(G, *epilogue); }
  count_launch();
  return (int)cudaGetLastError();
}
