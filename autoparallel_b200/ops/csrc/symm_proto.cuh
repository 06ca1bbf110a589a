// Flag protocol shared by every kernel that touches a symmetric workspace (symm_comm.cu and the
// fused GEMM+collective kernels).  Workspace of each rank: [ header | staging ].
//   ready[r]   on rank p: rank r's staging content for epoch e is complete
//   done[r]    on rank p: rank r will not touch p's staging for epoch e any more
//   contrib[r] on rank p: rank r has finished all its reductions into p's staging (GEMM -> reduce-scatter)
// Epochs only grow; waits are bounded (~2 s) and record ST_TIMEOUT_PEER on expiry.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace apbs {

constexpr int MAX_RANKS = 16;
constexpr unsigned long long kPeerWaitLimitNs = 2000000000ull;
constexpr uint32_t ST_TIMEOUT_PEER = 5;

constexpr int FLAG_STRIDE = 128;
constexpr int OFF_READY = 0;
constexpr int OFF_DONE = MAX_RANKS * FLAG_STRIDE;
constexpr int OFF_CONTRIB = 2 * MAX_RANKS * FLAG_STRIDE;
constexpr int OFF_COUNTERS = 3 * MAX_RANKS * FLAG_STRIDE;  // local atomic counters (uint32 each, 128-B apart)
constexpr int HEADER_BYTES = 8192;

struct Peers {
  uint8_t* base[MAX_RANKS];
};

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for *flag >= target (wrap-safe signed difference).  SYS: the flag is written by another GPU.
// On expiry the status word gets ST_TIMEOUT_PEER (first error wins) and the caller returns.
template <bool SYS>
__device__ __forceinline__ bool wait_ge(const uint32_t* flag, uint32_t target, uint32_t* status,
                                        unsigned long long limit_ns = kPeerWaitLimitNs) {
  uint32_t v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
  if ((int32_t)(v - target) >= 0) return true;
  const unsigned long long t0 = gtime();
  for (uint32_t i = 1;; ++i) {
    v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if ((int32_t)(v - target) >= 0) return true;
    if ((i & 31u) == 0u) {
      if (gtime() - t0 > limit_ns) {
        atomicCAS(status, 0u, ST_TIMEOUT_PEER);
        return false;
      }
      __nanosleep(64);
    }
  }
}

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* ws, int off, int idx) {
  return reinterpret_cast<uint32_t*>(ws + off + idx * FLAG_STRIDE);
}

// "Last CTA of this role" detection: every participating CTA arrives once; true for the one that
// brings the (monotonic) counter to ``target``.  Issues a system-scope fence first so that the
// caller's writes precede any flag the last CTA raises.
__device__ __forceinline__ bool arrive_is_last(uint32_t* counter, uint32_t target) {
  __shared__ uint32_t is_last_s;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) is_last_s = (atomicAdd(counter, 1u) + 1u == target) ? 1u : 0u;
  __syncthreads();
  return is_last_s != 0u;
}

// copy ``bytes`` (multiple of 16, both 16-B aligned) with CTAs [cta, cta+ncta) of this launch.
// Eight independent 16-byte loads are in flight per thread before the first store, which is what
// keeps an NVLink pull (about 2 us round trip) near link bandwidth with a few dozen CTAs.
__device__ __forceinline__ void coop_copy16(uint8_t* dst, const uint8_t* src, long long bytes, int cta, int ncta) {
  const long long nvec = bytes >> 4;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  const long long stride = (long long)ncta * blockDim.x;
  long long i = (long long)cta * blockDim.x + threadIdx.x;
  for (; i + 7 * stride < nvec; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = s[i + k * stride];
#pragma unroll
    for (int k = 0; k < 8; ++k) d[i + k * stride] = v[k];
  }
  for (; i < nvec; i += stride) d[i] = s[i];
}

}  // namespace apbs
