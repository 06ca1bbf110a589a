// GEMM fused with its neighbouring collective, one kernel per rank, over NVLink peer memory.
//
//   all-gather -> GEMM   (FUSE_GATHER_A / FUSE_GATHER_B): a seventh warp in every GEMM CTA drives
//       the copy engine: it publishes the CTA's share of this rank's shard, pulls the same share of
//       every peer's shard ONCE into a local full-size operand buffer (bulk copies through a ring of
//       bounce buffers in shared memory) and bumps a per-shard "landed" counter; the GEMM warps
//       (one CTA per SM, same persistent tcgen05 main loop as the plain GEMM) start on the local
//       shard and wait on the counter only when they reach a tile of a shard that has not landed
//       yet.  No SM is taken from the GEMM.  Covers the FSDP parameter gather in forward
//       (weights [N/n, K] gathered along N) and in backward (the same weights consumed as a
//       [K', N'] operand, i.e. gathered along the contraction dim) and the tensor-parallel
//       activation gather (A rows).
//   GEMM -> reduce-scatter (FUSE_REDUCE_SCATTER): the epilogue stores each fp32 accumulator tile into
//       this rank's slot of the OWNING rank's staging area with 16-byte stores over NVLink; once
//       every rank has signalled that its tiles are complete, the owner's communication CTAs sum
//       the n slots, scale / cast, and write the output shard.  Covers the gradient reduce-scatter (weight
//       gradient GEMM) and the row-parallel projection followed by a sequence-sharded output.
//
// No NCCL: remote data moves with plain (unicast) bulk loads and 16-byte peer stores issued from
// the kernel, so transfer and tensor-core work overlap tile by tile.  Waits are bounded; a timeout is
// reported through the status word.  Reference counterparts (host-driven pipelines of cuBLAS calls
// and P2P copies): autoparallel/graph_passes/async_tp/asynctp_ops.py:396-531, 1104-1186.
#include "gemm_core.cuh"

namespace apb {

struct CommParams {
  int comm_ctas;  // reduce-scatter only: CTAs that wait for the peers and publish "slots free"
  long long acc_elems;  // fp32 elements of this rank's accumulation buffer (rows_per_rank * N)
  void* out;
  int out_fp32;
  float scale;
  // arrival-counter targets (running totals kept by the host)
  uint32_t t_phase0, t_phase1, t_gemm;
};

// Final phase of GEMM -> reduce-scatter, executed by the GEMM CTAs once their tiles are done: wait
// until every rank has signalled that its tiles are stored, then sum the n slots of this rank's
// staging area into the output shard.  (All GEMM CTAs are resident at that point: one per SM.)
__device__ __forceinline__ void rs_final_reduce(const GemmParams& p, const FuseParams& f, const CommParams& c, int cta, int ncta) {
  using namespace apbs;
  uint8_t* my_ws = f.peers.base[f.rank];
  const float* slots = reinterpret_cast<const float*>(my_ws + HEADER_BYTES);  // [n][rows_per_rank * N]
  __shared__ uint32_t ok_r;
  if (threadIdx.x == 0) ok_r = 1u;
  __syncthreads();
  if (threadIdx.x < f.n)
    if (!wait_ge<true>(flag_ptr(my_ws, OFF_CONTRIB, threadIdx.x), f.epoch, p.status)) ok_r = 0u;
  __syncthreads();
  if (!ok_r) return;
  // One CTA per SM with 192 threads: 16 independent 16-byte loads per thread (48 KB per SM) are
  // needed to keep HBM busy; fewer left this pass latency-bound.
  constexpr int U = 16;
  const long long stride = (long long)ncta * blockDim.x;
  if (f.slot_bf16) {
    // bf16 slots, bf16 result: 8 elements per 16-byte vector, summed in fp32
    const __nv_bfloat16* slots16 = reinterpret_cast<const __nv_bfloat16*>(my_ws + HEADER_BYTES);
    const long long nvec8 = c.acc_elems >> 3;
    for (long long i0 = (long long)cta * blockDim.x + threadIdx.x; i0 < nvec8; i0 += U * stride) {
      float acc[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      for (int k = 0; k < f.n; ++k) {
        const uint4* sl = reinterpret_cast<const uint4*>(slots16 + (long long)k * c.acc_elems);
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * stride < nvec8) x[u] = sl[i0 + u * stride];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * stride >= nvec8) continue;
          const uint32_t w[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[u][2 * e] += __uint_as_float(w[e] << 16);
            acc[u][2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec8) continue;
        uint4 o;
        o.x = pack_bf16(acc[u][0] * c.scale, acc[u][1] * c.scale);
        o.y = pack_bf16(acc[u][2] * c.scale, acc[u][3] * c.scale);
        o.z = pack_bf16(acc[u][4] * c.scale, acc[u][5] * c.scale);
        o.w = pack_bf16(acc[u][6] * c.scale, acc[u][7] * c.scale);
        reinterpret_cast<uint4*>(c.out)[i] = o;
      }
    }
    return;
  }
  const long long nvec = c.acc_elems >> 2;
  for (long long i0 = (long long)cta * blockDim.x + threadIdx.x; i0 < nvec; i0 += U * stride) {
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < f.n; ++k) {
      const float4* sl = reinterpret_cast<const float4*>(slots + (long long)k * c.acc_elems);
      float4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < nvec) x[u] = sl[i0 + u * stride];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < nvec) { acc[u].x += x[u].x; acc[u].y += x[u].y; acc[u].z += x[u].z; acc[u].w += x[u].w; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      float4 v = acc[u];
      v.x *= c.scale; v.y *= c.scale; v.z *= c.scale; v.w *= c.scale;
      reinterpret_cast<float4*>(c.out)[i] = v;
    }
  }
}

__device__ __forceinline__ void comm_reduce_scatter(const GemmParams& p, const FuseParams& f, const CommParams& c, int cta) {
  using namespace apbs;
  uint8_t* my_ws = f.peers.base[f.rank];
  __shared__ uint32_t ok_s;
  if (threadIdx.x == 0) ok_s = 1u;
  __syncthreads();
  // my staging area is free once every peer has finished the previous collective
  if (threadIdx.x < f.n && threadIdx.x != f.rank)
    if (!wait_ge<true>(flag_ptr(my_ws, OFF_DONE, threadIdx.x), f.epoch - 1, p.status)) ok_s = 0u;
  __syncthreads();
  if (!ok_s) return;
  if (arrive_is_last(flag_ptr(my_ws, OFF_COUNTERS, 2), c.t_phase0)) {
    if (threadIdx.x < f.n) st_release_sys(flag_ptr(f.peers.base[threadIdx.x], OFF_READY, f.rank), f.epoch);
  }
  // Return at once: every CTA of the launch requests the GEMM's shared memory, so only one CTA
  // fits per SM and a communication CTA that lingered would keep a GEMM CTA off its SM.
}

template <bool A_MN, bool B_MN, int FUSE, bool PAIR>
__device__ __forceinline__ void fused_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const FuseParams& f,
                                           const CommParams& c, uint8_t* smem_raw) {
  if (FUSE == FUSE_REDUCE_SCATTER && (int)blockIdx.x < c.comm_ctas) {
    comm_reduce_scatter(p, f, c, blockIdx.x);
    return;
  }
  gemm_cta<A_MN, B_MN, FUSE, PAIR>(tmA, tmB, p, f, blockIdx.x - c.comm_ctas, gridDim.x - c.comm_ctas, smem_raw);
  if (FUSE == FUSE_REDUCE_SCATTER) {
    using namespace apbs;
    uint8_t* my_ws = f.peers.base[f.rank];
    if (arrive_is_last(flag_ptr(my_ws, OFF_COUNTERS, 4), c.t_gemm)) {
      if (threadIdx.x < f.n) {
        st_release_sys(flag_ptr(f.peers.base[threadIdx.x], OFF_CONTRIB, f.rank), f.epoch);
        if (threadIdx.x != f.rank) st_release_sys(flag_ptr(f.peers.base[threadIdx.x], OFF_DONE, f.rank), f.epoch);
      }
    }
    rs_final_reduce(p, f, c, blockIdx.x - c.comm_ctas, gridDim.x - c.comm_ctas);
  }
}

template <bool A_MN, bool B_MN, int FUSE>
__global__ void __launch_bounds__(FUSE == FUSE_REDUCE_SCATTER ? GEMM_THREADS : GEMM_AG_THREADS, 1)
gemm_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p,
                  FuseParams f, CommParams c) {
  extern __shared__ uint8_t smem_raw[];
  fused_body<A_MN, B_MN, FUSE, false>(tmA, tmB, p, f, c, smem_raw);
}

// Same on CTA pairs (clusters of two, 256 x 256 tiles).  With a reduce-scatter the communication
// CTAs come first in the grid and their number is even, so GEMM CTAs 2i and 2i+1 share a cluster.
template <bool A_MN, bool B_MN, int FUSE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FUSE == FUSE_REDUCE_SCATTER ? GEMM_THREADS : GEMM_AG_THREADS, 1)
gemm_fused_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p,
                       FuseParams f, CommParams c) {
  extern __shared__ uint8_t smem_raw[];
  fused_body<A_MN, B_MN, FUSE, true>(tmA, tmB, p, f, c, smem_raw);
}

}  // namespace apb

using namespace apb;

extern "C" int apb_gemm_get_pair_mode();
extern "C" int apb_gemm_resident_pairs(int num_sms);
extern "C" int apb_gemm_get_reserved_sms();

static bool fused_uses_pairs(int M, int N, int comm_ctas) {
  return apb_gemm_get_pair_mode() && M >= 2 * BM && N >= BN && (comm_ctas & 1) == 0;
}

// Number of GEMM CTAs a fused launch of this shape runs (the host keeps running totals of their arrivals).
extern "C" int apb_gemm_fused_ctas(int fuse, int M, int N, int comm_ctas, int num_sms) {
  const int cc = fuse == FUSE_REDUCE_SCATTER ? comm_ctas : 0;
  if (fused_uses_pairs(M, N, cc)) {
    const int tiles2 = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    int resident = apb_gemm_resident_pairs(num_sms) - cc / 2 - apb_gemm_get_reserved_sms() / 2;
    if (resident < 1) resident = 1;
    return 2 * (tiles2 < resident ? tiles2 : resident);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int usable = num_sms - apb_gemm_get_reserved_sms() > 0 ? num_sms - apb_gemm_get_reserved_sms() : 1;
  return tiles < usable ? tiles : usable;
}

// fuse: 1 gather A, 2 gather B, 3 reduce-scatter.  ``targets``: {phase0, phase1, gemm} arrival totals
// (gathers: one arrival per GEMM CTA in phases 0 and 1; reduce-scatter: comm_ctas in phase 0, GEMM CTAs in 'gemm').
// For gathers the tensor map of the gathered operand is built over ``gbuf`` (the local full-size
// buffer); the caller passes that pointer as A or B.  Returns 0 or an error code.
extern "C" int apb_gemm_fused(int fuse, const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                              long long ldb, long long ldc, int a_mn_major, int b_mn_major, int out_fp32,
                              const unsigned long long* peer_ptrs, int rank, int n, unsigned epoch, int rows_per_shard,
                              const void* shard_src, void* gbuf, long long shard_bytes, uint32_t* landed,
                              unsigned landed_target, int rows_per_rank, float scale, long long stage_capacity,
                              const unsigned* targets, int comm_ctas, uint32_t* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (n > apbs::MAX_RANKS || n < 1 || comm_ctas < 1) return 3;
  const bool pair = fused_uses_pairs(M, N, fuse == FUSE_REDUCE_SCATTER ? comm_ctas : 0);
  CUtensorMap tmA, tmB;
  const int e = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_mn_major, b_mn_major, pair);
  if (e) return e;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + BN - 1) / BN;
  p.status = status;
  FuseParams f{};
  for (int i = 0; i < n; ++i) f.peers.base[i] = reinterpret_cast<uint8_t*>(peer_ptrs[i]);
  f.rank = rank; f.n = n; f.epoch = epoch;
  f.rows_per_shard = rows_per_shard; f.landed = landed; f.landed_target = landed_target; f.rows_per_rank = rows_per_rank;
  CommParams c{};
  c.comm_ctas = comm_ctas;
  f.shard_src = static_cast<const uint8_t*>(shard_src); f.gbuf = static_cast<uint8_t*>(gbuf); f.shard_bytes = shard_bytes;
  f.t_publish = targets[0]; f.t_pulled = targets[1];
  c.out = C; c.out_fp32 = out_fp32; c.scale = scale;
  c.t_phase0 = targets[0]; c.t_phase1 = targets[1]; c.t_gemm = targets[2];
  if (fuse == FUSE_REDUCE_SCATTER) {
    if (rows_per_rank <= 0 || (rows_per_rank % BM) != 0 || (long long)rows_per_rank * n != M || (N & 7)) return 3;
    c.acc_elems = (long long)rows_per_rank * N;
    f.slot_bf16 = out_fp32 ? 0 : 1;  // partial sums travel in the precision of the result
    if (c.acc_elems * (out_fp32 ? 4 : 2) * n > stage_capacity) return 7;  // one slot per source rank
  } else {
    if ((shard_bytes & 15) || shard_bytes > stage_capacity || rows_per_shard <= 0) return shard_bytes > stage_capacity ? 7 : 3;
    if ((reinterpret_cast<uintptr_t>(shard_src) & 15) || (reinterpret_cast<uintptr_t>(gbuf) & 15)) return 3;  // bulk copies
    c.comm_ctas = 0;
  }
  const int gemm_ctas = apb_gemm_fused_ctas(fuse, M, N, comm_ctas, num_sms);
  const int grid = gemm_ctas + c.comm_ctas;
  const int smem_bytes = fuse == FUSE_REDUCE_SCATTER ? GEMM_FUSED_RS_SMEM_BYTES : GEMM_FUSED_AG_SMEM_BYTES;
  const int threads = fuse == FUSE_REDUCE_SCATTER ? GEMM_THREADS : GEMM_AG_THREADS;
  auto launch = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    kern<<<grid, threads, smem_bytes, stream>>>(tmA, tmB, p, f, c);
  };
#define APB_LAUNCH_FUSED(FUSE)                                                               \
  do {                                                                                       \
    if (pair) {                                                                              \
      if (!a_mn_major && !b_mn_major) launch(gemm_fused_pair_kernel<false, false, FUSE>);    \
      else if (!a_mn_major && b_mn_major) launch(gemm_fused_pair_kernel<false, true, FUSE>); \
      else if (a_mn_major && !b_mn_major) launch(gemm_fused_pair_kernel<true, false, FUSE>); \
      else launch(gemm_fused_pair_kernel<true, true, FUSE>);                                 \
    } else {                                                                                 \
      if (!a_mn_major && !b_mn_major) launch(gemm_fused_kernel<false, false, FUSE>);         \
      else if (!a_mn_major && b_mn_major) launch(gemm_fused_kernel<false, true, FUSE>);      \
      else if (a_mn_major && !b_mn_major) launch(gemm_fused_kernel<true, false, FUSE>);      \
      else launch(gemm_fused_kernel<true, true, FUSE>);                                      \
    }                                                                                        \
  } while (0)
  if (fuse == FUSE_GATHER_A) APB_LAUNCH_FUSED(FUSE_GATHER_A);
  else if (fuse == FUSE_GATHER_B) APB_LAUNCH_FUSED(FUSE_GATHER_B);
  else if (fuse == FUSE_REDUCE_SCATTER) APB_LAUNCH_FUSED(FUSE_REDUCE_SCATTER);
  else return 3;
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
