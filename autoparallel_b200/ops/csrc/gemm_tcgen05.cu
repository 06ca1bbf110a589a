// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// fp32 accumulators in TMEM -> epilogue from TMEM.
//
//   C[M,N] = opA * opB      A: [M,K] (K-major) or [K,M] (MN-major), bf16
//                            B: [N,K] (K-major) or [K,N] (MN-major), bf16
//                            C: bf16 or fp32, row-major
//
// Two kernels from one body (gemm_core.cuh): one CTA per SM on 128 x 256 tiles, and CTA pairs on
// 256 x 256 tiles with tcgen05 cta_group::2, which halves the B traffic into each SM's shared
// memory; ``apb_gemm_set_pair_mode`` selects between them.  All four
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

template <bool A_MN, bool B_MN, int ST = 0, bool DYN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  FuseParams f{};
  gemm_cta<A_MN, B_MN, FUSE_NONE, true, false, ST, DYN>(tmA, tmB, p, f, blockIdx.x, gridDim.x, smem_raw);
}

// Grouped GEMM: G problems of one shape (the expert projections of a capacity-based MoE layer).
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  FuseParams f{};
  gemm_cta<A_MN, B_MN, FUSE_NONE, false, true>(tmA, tmB, p, f, blockIdx.x, gridDim.x, smem_raw);
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_grouped_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  FuseParams f{};
  gemm_cta<A_MN, B_MN, FUSE_NONE, true, true>(tmA, tmB, p, f, blockIdx.x, gridDim.x, smem_raw);
}

static int g_pair_mode = 1;  // 0: one CTA per tile, 1: CTA pairs where the shape allows (default)

}  // namespace apb

// Number of CTA pairs that can be resident at once (an SM without a free partner in its GPC stays
// idle); cached after the first query.
extern "C" int apb_gemm_resident_pairs(int num_sms) {
  static int cached = 0;
  if (cached > 0) return cached;
  auto kern = apb::gemm_bf16_pair_kernel<false, false>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, apb::GEMM_SMEM_BYTES);
  using namespace apb;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(num_sms & ~1));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = num_sms / 2;
  }
  cached = n;
  return n;
}

using namespace apb;

// SMs that the GEMM kernels leave idle so that communication kernels launched on other streams (NCCL)
// find a free SM right away: a persistent GEMM CTA owns its SM's shared memory for the whole kernel.
// TMA stages of the CTA-pair GEMM: 6 fill the SM's shared memory; 5 or 4 leave 32 / 64 KB more for a
// communication kernel's CTA to become resident beside a GEMM CTA.
static int g_pair_stages = 6;
extern "C" void apb_gemm_set_pair_stages(int n) { g_pair_stages = n <= 4 ? 4 : (n == 5 ? 5 : 6); }
extern "C" int apb_gemm_get_pair_stages() { return g_pair_stages; }
// Dynamic tile scheduling of the CTA-pair GEMM (see gemm_core.cuh): off = every pair owns a fixed share.
static int g_dynamic_tiles = 0;
extern "C" void apb_gemm_set_dynamic_tiles(int on) { g_dynamic_tiles = on ? 1 : 0; }
extern "C" int apb_gemm_get_dynamic_tiles() { return g_dynamic_tiles; }

// {next tile, pairs that left, SM-pair requests, pairs that gave up their SMs} per device; the last pair of a
// launch zeroes all but the requests.
static int* tile_counters() {
  static int* per_device[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (per_device[dev] == nullptr) {
    int* ptr = nullptr;
    if (cudaMalloc(&ptr, 4 * sizeof(int)) != cudaSuccess || cudaMemset(ptr, 0, 4 * sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    per_device[dev] = ptr;
  }
  return per_device[dev];
}

// Asks the GEMM kernels that follow on this device to give up ``pairs`` SM pairs (see gemm_core.cuh).  Runs as a
// one-warp kernel in stream order, so the request appears exactly when the stream reaches this point; such
// a kernel fits beside a resident GEMM CTA.  Outstanding requests are capped.
__global__ void yield_request_kernel(int* counters, int pairs, int cap) {
  if (threadIdx.x == 0) {
    const int cur = *reinterpret_cast<volatile int*>(counters + 2);
    if (cur < cap) atomicAdd(counters + 2, pairs < cap - cur ? pairs : cap - cur);
  }
}
extern "C" int apb_gemm_yield_request(int pairs, cudaStream_t stream) {
  int* counters = tile_counters();
  if (counters == nullptr || pairs <= 0) return 0;
  yield_request_kernel<<<1, 32, 0, stream>>>(counters, pairs, 32);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
// Outstanding requests (synchronises the device; for tests).
extern "C" int apb_gemm_yield_outstanding() {
  int* counters = tile_counters();
  if (counters == nullptr) return -1;
  int host[4] = {0, 0, 0, 0};
  cudaDeviceSynchronize();
  cudaMemcpy(host, counters, sizeof(host), cudaMemcpyDeviceToHost);
  return host[0] != 0 || host[1] != 0 || host[3] != 0 ? -2 : host[2];
}

static int g_reserved_sms = 0;
extern "C" void apb_gemm_set_reserved_sms(int n) { g_reserved_sms = n < 0 ? 0 : (n & ~1); }
extern "C" int apb_gemm_get_reserved_sms() { return g_reserved_sms; }
extern "C" void apb_gemm_set_pair_mode(int on) { g_pair_mode = on ? 1 : 0; }
extern "C" int apb_gemm_get_pair_mode() { return g_pair_mode; }

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
  if (g_pair_mode && M >= 2 * BM && N >= BN) {
    // CTA pairs: B is loaded in boxes of 128 rows (each CTA stages half of the 256 tile columns)
    int e2 = 0;
    if (!b_mn_major) e2 = make_map(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BN / 2);
    if (e2) return e2;
    const int tiles2 = ((M + 2 * BM - 1) / (2 * BM)) * p.num_n_tiles;
    int resident = apb_gemm_resident_pairs(num_sms) - g_reserved_sms / 2;
    if (resident < 1) resident = 1;
    const int pairs = tiles2 < resident ? tiles2 : resident;
    const int smem2 = g_pair_stages * (A_STAGE_BYTES + B_STAGE_BYTES / 2) + 1024 + 256;
    auto launch2 = [&](auto kern) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2);
      kern<<<2 * pairs, GEMM_THREADS, smem2, stream>>>(tmA, tmB, p);
    };
#define APB_LAUNCH_PAIR(ST)                                                              \
  do {                                                                                   \
    if (!a_mn_major && !b_mn_major) launch2(gemm_bf16_pair_kernel<false, false, ST>);    \
    else if (!a_mn_major && b_mn_major) launch2(gemm_bf16_pair_kernel<false, true, ST>); \
    else if (a_mn_major && !b_mn_major) launch2(gemm_bf16_pair_kernel<true, false, ST>); \
    else launch2(gemm_bf16_pair_kernel<true, true, ST>);                                 \
  } while (0)
    int* counters = (g_dynamic_tiles && g_pair_stages == 6) ? tile_counters() : nullptr;
    if (counters != nullptr) {
      p.tile_counter = counters;
      if (!a_mn_major && !b_mn_major) launch2(gemm_bf16_pair_kernel<false, false, 0, true>);
      else if (!a_mn_major && b_mn_major) launch2(gemm_bf16_pair_kernel<false, true, 0, true>);
      else if (a_mn_major && !b_mn_major) launch2(gemm_bf16_pair_kernel<true, false, 0, true>);
      else launch2(gemm_bf16_pair_kernel<true, true, 0, true>);
    } else if (g_pair_stages == 4) APB_LAUNCH_PAIR(4);
    else if (g_pair_stages == 5) APB_LAUNCH_PAIR(5);
    else APB_LAUNCH_PAIR(0);
    return cudaGetLastError() == cudaSuccess ? 0 : 4;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int usable = num_sms - g_reserved_sms > 0 ? num_sms - g_reserved_sms : 1;
  const int grid = tiles < usable ? tiles : usable;
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

// C[g] = opA[g] * opB[g] for g < G; every operand is a dense stack [G, rows, cols] of bf16 matrices
// (K-major [rows=M or N, cols=K], or MN-major [rows=K, cols=M or N]); C is [G, M, N] bf16 or fp32.
extern "C" int apb_gemm_grouped_bf16(const void* A, const void* B, void* C, int G, int M, int N, int K, int a_mn_major,
                                     int b_mn_major, int out_fp32, uint32_t* status, int num_sms, cudaStream_t stream) {
  if (G <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  const int a_inner = a_mn_major ? M : K, b_inner = b_mn_major ? N : K;
  if ((a_inner & 7) || (b_inner & 7) || (N & 7)) return 3;  // 16-byte rows for TMA and for the vector stores
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15)) return 3;
  const bool pair = g_pair_mode && M >= 2 * BM && N >= BN;
  CUtensorMap tmA, tmB;
  int e = !a_mn_major ? make_map_3d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)G, (uint64_t)K, BM)
                      : make_map_3d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)G, (uint64_t)M, BK);
  if (e) return e;
  e = !b_mn_major ? make_map_3d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)G, (uint64_t)K, pair ? BN / 2 : BN)
                  : make_map_3d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)G, (uint64_t)N, BK);
  if (e) return e;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = N; p.out_fp32 = out_fp32;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + BN - 1) / BN;
  p.status = status;
  p.groups = G;
  auto launch = [&](auto kern, int grid) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
    kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(tmA, tmB, p);
  };
  if (pair) {
    const long long tiles2 = (long long)G * ((M + 2 * BM - 1) / (2 * BM)) * p.num_n_tiles;
    int resident = apb_gemm_resident_pairs(num_sms) - g_reserved_sms / 2;
    if (resident < 1) resident = 1;
    const int grid = 2 * (int)(tiles2 < resident ? tiles2 : resident);
    if (!a_mn_major && !b_mn_major) launch(gemm_grouped_pair_kernel<false, false>, grid);
    else if (!a_mn_major && b_mn_major) launch(gemm_grouped_pair_kernel<false, true>, grid);
    else if (a_mn_major && !b_mn_major) launch(gemm_grouped_pair_kernel<true, false>, grid);
    else launch(gemm_grouped_pair_kernel<true, true>, grid);
  } else {
    const long long tiles = (long long)G * p.num_m_tiles * p.num_n_tiles;
    const int usable = num_sms - g_reserved_sms > 0 ? num_sms - g_reserved_sms : 1;
    const int grid = (int)(tiles < usable ? tiles : usable);
    if (!a_mn_major && !b_mn_major) launch(gemm_grouped_kernel<false, false>, grid);
    else if (!a_mn_major && b_mn_major) launch(gemm_grouped_kernel<false, true>, grid);
    else if (a_mn_major && !b_mn_major) launch(gemm_grouped_kernel<true, false>, grid);
    else launch(gemm_grouped_kernel<true, true>, grid);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
