// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// fp32 accumulators in TMEM -> epilogue from TMEM.
//
//   C[M,N] = opA * opB      A: [M,K] (K-major) or [K,M] (MN-major), bf16
//                            B: [N,K] (K-major) or [K,N] (MN-major), bf16
//                            C: bf16 or fp32, row-major
//
// One CTA per SM (grid = min(#tiles, #SMs)); the CTA body lives in gemm_core.cuh.  All four
// operand-major combinations run on the tensor cores directly (MN-major operands use the MN-major
// shared-memory descriptor), so dgrad / wgrad need no transposed copies.
//
// This is the kernel behind aten.mm / apb200::mm_nd / mm_wgrad / gemm; the reference reaches
// cuBLAS for the same nodes (autoparallel/graph_passes/graph_utils.py:320-412).
#include "gemm_core.cuh"

namespace apb {

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  FuseParams f{};
  gemm_cta<A_MN, B_MN, FUSE_NONE>(tmA, tmB, p, f, blockIdx.x, gridDim.x, smem_raw);
}

}  // namespace apb

using namespace apb;

// Returns 0 on success; >0 = argument / driver error (nothing launched).
extern "C" int apb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                             long long ldc, int a_mn_major, int b_mn_major, int out_fp32, uint32_t* status,
                             int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(C) & 15) return 3;
  CUtensorMap tmA, tmB;
  const int e = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_mn_major, b_mn_major);
  if (e) return e;  // TMA needs 16-byte aligned bases and row strides
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + BN - 1) / BN;
  p.status = status;
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < num_sms ? tiles : num_sms;
  auto launch = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
    kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(tmA, tmB, p);
  };
  if (!a_mn_major && !b_mn_major) launch(gemm_bf16_kernel<false, false>);
  else if (!a_mn_major && b_mn_major) launch(gemm_bf16_kernel<false, true>);
  else if (a_mn_major && !b_mn_major) launch(gemm_bf16_kernel<true, false>);
  else launch(gemm_bf16_kernel<true, true>);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
