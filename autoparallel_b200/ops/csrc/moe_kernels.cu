// Index kernels of the mixture-of-experts dispatch (capacity based, block local; semantics in ops/moe_ops.py):
//
//   moe_slots     arrival rank of every (token, choice) inside its expert, per token block, in token-major order
//                 -> row of the block's [E * C] buffer, or E * C for an assignment beyond the capacity
//   moe_scatter   buf[e, blk, c, :] = w[t, j] * src[t, :]            (buffer [E, nb, C, d], zero-filled by the caller)
//   moe_gather    out[t, :] = sum_j w[t, j] * buf[slot[t, j], :]     (dropped assignments contribute nothing)
//   moe_gate_grad dw[t, j] = < buf[slot[t, j], :], g[t, :] >
//
// The counterpart in the reference is its one hand-written device kernel, the Triton permutation-index kernel of its
// DeepSeek-V3 test model (autoparallel/_testing/models/dsv3.py:62-91), which turns rank-major token order into expert-major
// order with per-expert padding; here the same job is a counting pass over static-capacity buffers.
//
// All four are bandwidth / latency trivial next to the expert GEMMs; they exist so that the dispatch is four launches
// instead of a few dozen index kernels, and so that no intermediate [T * k, d] tensor is materialised.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace apb {

// One CTA per token block.  Shared memory: base[E] (assignments of each expert seen in earlier rounds) and
// wcnt[warps][E] (assignments of each expert held by each warp in this round).
__global__ void moe_slots_kernel(const long long* __restrict__ gate_idx, long long* __restrict__ slot, int per_block, int E,
                                 int C) {
  extern __shared__ int smem_i[];
  int* base = smem_i;
  int* wcnt = smem_i + E;
  const int nwarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long* in = gate_idx + (long long)blockIdx.x * per_block;
  long long* out = slot + (long long)blockIdx.x * per_block;
  for (int i = threadIdx.x; i < E * (nwarps + 1); i += blockDim.x) smem_i[i] = 0;
  __syncthreads();
  for (int start = 0; start < per_block; start += blockDim.x) {
    const int i = start + threadIdx.x;
    const bool valid = i < per_block;
    const int e = valid ? (int)in[i] : -1;
    const bool ok = valid && e >= 0 && e < E;
    const unsigned active = __ballot_sync(0xffffffffu, ok);
    int lane_rank = 0;
    if (ok) {
      const unsigned same = __match_any_sync(active, e);
      lane_rank = __popc(same & ((1u << lane) - 1u));
      if (lane_rank == 0) wcnt[warp * E + e] = __popc(same);
    }
    __syncthreads();
    if (ok) {
      int pos = base[e] + lane_rank;
      for (int w = 0; w < warp; ++w) pos += wcnt[w * E + e];
      out[i] = pos < C ? (long long)e * C + pos : (long long)E * C;
    } else if (valid) {
      out[i] = (long long)E * C;
    }
    __syncthreads();
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
      int s = 0;
      for (int w = 0; w < nwarps; ++w) {
        s += wcnt[w * E + x];
        wcnt[w * E + x] = 0;
      }
      base[x] += s;
    }
    __syncthreads();
  }
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// row of buf [E, nb, C, d] addressed by (slot in the block's [E * C] buffer, block); -1 when the assignment was dropped
__device__ __forceinline__ long long buf_row(long long s, int blk, int E, int C, int nb) {
  if (s < 0 || s >= (long long)E * C) return -1;
  const long long e = s / C, c = s % C;
  return (e * nb + blk) * C + c;
}

// one warp per assignment
template <typename T>
__global__ void moe_scatter_kernel(const T* __restrict__ src, const long long* __restrict__ slot, const float* __restrict__ w,
                                   T* __restrict__ buf, long long Tn, int k, int d, int E, int C, int nb) {
  const long long a = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (a >= Tn * k) return;
  const long long t = a / k;
  const long long row = buf_row(slot[a], (int)(t / (Tn / nb)), E, C, nb);
  if (row < 0) return;
  const T* x = src + t * d;
  T* y = buf + row * d;
  const float wt = w[a];
  for (int i = lane; i < d; i += 32) y[i] = from_f<T>(to_f<T>(x[i]) * wt);
}

// one CTA per token
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ buf, const long long* __restrict__ slot, const float* __restrict__ w,
                                  T* __restrict__ out, long long Tn, int k, int d, int E, int C, int nb) {
  const long long t = blockIdx.x;
  const int blk = (int)(t / (Tn / nb));
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j) {
      const long long row = buf_row(slot[t * k + j], blk, E, C, nb);
      if (row >= 0) acc += w[t * k + j] * to_f<T>(buf[row * d + i]);
    }
    out[t * d + i] = from_f<T>(acc);
  }
}

// one warp per assignment
template <typename T>
__global__ void moe_gate_grad_kernel(const T* __restrict__ buf, const long long* __restrict__ slot, const T* __restrict__ g,
                                     float* __restrict__ dw, long long Tn, int k, int d, int E, int C, int nb) {
  const long long a = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (a >= Tn * k) return;
  const long long t = a / k;
  const long long row = buf_row(slot[a], (int)(t / (Tn / nb)), E, C, nb);
  float acc = 0.f;
  if (row >= 0) {
    const T* x = buf + row * d;
    const T* y = g + t * d;
    for (int i = lane; i < d; i += 32) acc += to_f<T>(x[i]) * to_f<T>(y[i]);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dw[a] = acc;
}

}  // namespace apb

using namespace apb;

static int launch_status() { return (int)cudaGetLastError(); }

// Largest expert count the slot kernel takes with `threads` threads per block (48 KB of static-limit shared memory).
extern "C" int apb_moe_slots_max_experts(int threads) { return (48 * 1024 / 4) / ((threads >> 5) + 1); }

extern "C" int apb_moe_slots(const long long* gate_idx, long long* slot, int num_blocks, int per_block, int E, int C,
                             cudaStream_t st) {
  if (num_blocks <= 0 || per_block <= 0 || E <= 0 || C <= 0) return (int)cudaErrorInvalidValue;
  int threads = per_block >= 1024 ? 1024 : ((per_block + 31) / 32) * 32;
  if (E > apb_moe_slots_max_experts(threads)) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)E * ((threads >> 5) + 1) * sizeof(int);
  moe_slots_kernel<<<num_blocks, threads, smem, st>>>(gate_idx, slot, per_block, E, C);
  return launch_status();
}

extern "C" int apb_moe_scatter(const void* src, const long long* slot, const float* w, void* buf, long long T, int k, int d,
                               int E, int C, int nb, int is_bf16, cudaStream_t st) {
  if (T <= 0 || k <= 0 || d <= 0 || nb <= 0 || T % nb) return (int)cudaErrorInvalidValue;
  const int warps = 8;
  const long long blocks = (T * k + warps - 1) / warps;
  if (is_bf16)
    moe_scatter_kernel<__nv_bfloat16><<<(unsigned)blocks, warps * 32, 0, st>>>((const __nv_bfloat16*)src, slot, w, (__nv_bfloat16*)buf, T,
                                                                              k, d, E, C, nb);
  else
    moe_scatter_kernel<float><<<(unsigned)blocks, warps * 32, 0, st>>>((const float*)src, slot, w, (float*)buf, T, k, d, E, C, nb);
  return launch_status();
}

extern "C" int apb_moe_gather(const void* buf, const long long* slot, const float* w, void* out, long long T, int k, int d, int E,
                              int C, int nb, int is_bf16, cudaStream_t st) {
  if (T <= 0 || k <= 0 || d <= 0 || nb <= 0 || T % nb) return (int)cudaErrorInvalidValue;
  const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
  if (is_bf16)
    moe_gather_kernel<__nv_bfloat16><<<(unsigned)T, threads, 0, st>>>((const __nv_bfloat16*)buf, slot, w, (__nv_bfloat16*)out, T, k, d, E,
                                                                     C, nb);
  else
    moe_gather_kernel<float><<<(unsigned)T, threads, 0, st>>>((const float*)buf, slot, w, (float*)out, T, k, d, E, C, nb);
  return launch_status();
}

extern "C" int apb_moe_gate_grad(const void* buf, const long long* slot, const void* g, float* dw, long long T, int k, int d, int E,
                                 int C, int nb, int is_bf16, cudaStream_t st) {
  if (T <= 0 || k <= 0 || d <= 0 || nb <= 0 || T % nb) return (int)cudaErrorInvalidValue;
  const int warps = 8;
  const long long blocks = (T * k + warps - 1) / warps;
  if (is_bf16)
    moe_gate_grad_kernel<__nv_bfloat16><<<(unsigned)blocks, warps * 32, 0, st>>>((const __nv_bfloat16*)buf, slot, (const __nv_bfloat16*)g,
                                                                                dw, T, k, d, E, C, nb);
  else
    moe_gate_grad_kernel<float><<<(unsigned)blocks, warps * 32, 0, st>>>((const float*)buf, slot, (const float*)g, dw, T, k, d, E, C, nb);
  return launch_status();
}
