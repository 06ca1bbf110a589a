// Collectives over NVLink peer memory, written as plain CUDA kernels on a symmetric workspace.
//
// Every rank owns one workspace buffer of identical layout that all ranks of the group can address
// (peer pointers obtained once at rendezvous): [ flags | staging ].  One kernel launch per rank
// performs a whole collective:
//   phase 0  wait until every peer has finished reading my staging area from the previous
//            collective, copy my input into it, then raise my "ready" flag on every peer;
//   phase 1  for each peer (own rank first, then rotating) wait for its ready flag and PULL my part of
//            its staging area with 16-byte loads over NVLink - all-gather copies, reduce-scatter
//            sums in fp32, all-to-all copies the chunk addressed to me;
//   phase 2  the last CTA to finish raises my "done" flag on every peer.
// Reduce-scatter has a second form (opt-in) that sums through NVSwitch: one ``multimem.ld_reduce`` on the
// workspace's multicast address per 16 bytes instead of one load per peer.
// Flags carry a monotonically increasing epoch, so nothing is ever reset.  Every wait is bounded
// (~2 s): on expiry the kernel records ST_TIMEOUT_PEER_FLAG in the status word and returns.
//
// These kernels are the stand-alone collectives (unfused leftovers, user local_map collectives,
// calibration of the planner's cost table); the reference uses NCCL through c10d functional
// collectives for the same graph nodes (autoparallel/collectives.py:89-154).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "symm_proto.cuh"

namespace apbs {

enum Mode : int { ALL_GATHER = 0, REDUCE_SCATTER = 1, ALL_TO_ALL = 2 };

struct CollParams {
  Peers peers;
  int rank, n;
  uint32_t epoch;
  const uint8_t* src;  // this rank's input (outside the workspace)
  uint8_t* dst;        // this rank's output (outside the workspace)
  long long outer;     // number of outer slices
  long long inner_bytes;  // all-gather: bytes per rank per outer slice of the INPUT
                          // reduce-scatter / all-to-all: bytes per rank-chunk per outer slice of the INPUT
  int elem_kind;       // reduce-scatter: 0 = fp32, 1 = bf16 (summed in fp32)
  float scale;         // reduce-scatter: result multiplied by this
  uint32_t* status;
  uint32_t target0, target1;  // arrival-counter values that mark the last CTA of phases 0 and 1
  // reduce-scatter through the switch (NVLS): multicast address of the staging area (bound to every rank's
  // workspace), or null.  One ``multimem.ld_reduce`` then returns the sum over all ranks, added inside NVSwitch,
  // instead of n peer loads; this rank's own contribution is read through the same address, so its staging copy
  // must be complete too (the rank raises its "ready" flag on itself as well).
  const uint8_t* mc_stage;
};

__device__ __forceinline__ float4 multimem_sum_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// eight bf16 values, accumulated in fp32 inside the switch, returned as four packed pairs
__device__ __forceinline__ uint4 multimem_sum_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

template <int MODE>
__global__ void __launch_bounds__(512) symm_collective_kernel(CollParams p) {
  uint8_t* my_ws = p.peers.base[p.rank];
  uint8_t* my_stage = my_ws + HEADER_BYTES;
  const int n = p.n;
  // bytes of this rank's input
  const long long in_bytes = (MODE == ALL_GATHER) ? p.outer * p.inner_bytes : p.outer * p.inner_bytes * n;
  const bool nvls = MODE == REDUCE_SCATTER && p.mc_stage != nullptr;
  __shared__ uint32_t ok_s;
  if (threadIdx.x == 0) ok_s = 1u;
  __syncthreads();

  // ---- phase 0: my staging is free once every peer has finished the previous collective
  if (threadIdx.x < n && threadIdx.x != p.rank) {
    if (!wait_ge<true>(reinterpret_cast<uint32_t*>(my_ws + OFF_DONE + threadIdx.x * FLAG_STRIDE), p.epoch - 1, p.status)) ok_s = 0u;
  }
  __syncthreads();
  if (!ok_s) return;
  coop_copy16(my_stage, p.src, in_bytes, blockIdx.x, gridDim.x);
  if (arrive_is_last(flag_ptr(my_ws, OFF_COUNTERS, 0), p.target0)) {
    if (threadIdx.x < n && (threadIdx.x != p.rank || nvls))
      st_release_sys(reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + OFF_READY + p.rank * FLAG_STRIDE), p.epoch);
  }

  // ---- phase 1
  if (MODE == ALL_GATHER) {
    for (int k = 0; k < n; ++k) {
      const int peer = (p.rank + k) % n;
      const uint8_t* src;
      if (peer == p.rank) {
        src = p.src;
      } else {
        if (threadIdx.x == 0 &&
            !wait_ge<true>(reinterpret_cast<uint32_t*>(my_ws + OFF_READY + peer * FLAG_STRIDE), p.epoch, p.status))
          ok_s = 0u;
        __syncthreads();
        if (!ok_s) return;
        src = p.peers.base[peer] + HEADER_BYTES;
      }
      if (p.outer == 1) {
        coop_copy16(p.dst + (long long)peer * p.inner_bytes, src, p.inner_bytes, blockIdx.x, gridDim.x);
      } else {
        // dst[o][peer][inner] <- src[o][inner]
        const long long vec_per = p.inner_bytes >> 4;
        const long long total = p.outer * vec_per;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
          const long long o = i / vec_per, v = i % vec_per;
          reinterpret_cast<uint4*>(p.dst + (o * n + peer) * p.inner_bytes)[v] =
              reinterpret_cast<const uint4*>(src + o * p.inner_bytes)[v];
        }
      }
    }
  } else {
    // wait for everybody, then read chunk ``rank`` of every peer
    if (threadIdx.x < n && (threadIdx.x != p.rank || nvls)) {
      if (!wait_ge<true>(reinterpret_cast<uint32_t*>(my_ws + OFF_READY + threadIdx.x * FLAG_STRIDE), p.epoch, p.status)) ok_s = 0u;
    }
    __syncthreads();
    if (!ok_s) return;
    const long long vec_per = p.inner_bytes >> 4;  // 16-B vectors per chunk per outer slice
    const long long total = p.outer * vec_per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      long long o = 0, v = i;
      if (p.outer != 1) {
        o = i / vec_per;
        v = i - o * vec_per;
      }
      const long long src_off = (o * n + p.rank) * p.inner_bytes + (v << 4);
      if (MODE == REDUCE_SCATTER && nvls) {
        if (p.elem_kind == 0) {
          float4 acc = multimem_sum_f32x4(p.mc_stage + src_off);
          acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale;
          reinterpret_cast<float4*>(p.dst + o * p.inner_bytes)[v] = acc;
        } else {
          uint4 raw = multimem_sum_bf16x8(p.mc_stage + src_off);
          if (p.scale != 1.f) {
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(h[j]);
              h[j] = __floats2bfloat162_rn(f.x * p.scale, f.y * p.scale);
            }
          }
          reinterpret_cast<uint4*>(p.dst + o * p.inner_bytes)[v] = raw;
        }
      } else if (MODE == REDUCE_SCATTER) {
        if (p.elem_kind == 0) {
          float4 xs[MAX_RANKS];
#pragma unroll
          for (int k = 0; k < MAX_RANKS; ++k) {  // all loads issued before the first add
            if (k < n) {
              const int peer = (p.rank + k) % n;
              const uint8_t* base = (peer == p.rank) ? p.src : p.peers.base[peer] + HEADER_BYTES;
              xs[k] = *reinterpret_cast<const float4*>(base + src_off);
            }
          }
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int k = 0; k < MAX_RANKS; ++k)
            if (k < n) { acc.x += xs[k].x; acc.y += xs[k].y; acc.z += xs[k].z; acc.w += xs[k].w; }
          acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale;
          reinterpret_cast<float4*>(p.dst + o * p.inner_bytes)[v] = acc;
        } else {
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int k = 0; k < n; ++k) {
            const int peer = (p.rank + k) % n;
            const uint8_t* base = (peer == p.rank) ? p.src : p.peers.base[peer] + HEADER_BYTES;
            const uint4 raw = *reinterpret_cast<const uint4*>(base + src_off);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(h[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
          uint4 outv;
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&outv);
#pragma unroll
          for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j] * p.scale, acc[2 * j + 1] * p.scale);
          reinterpret_cast<uint4*>(p.dst + o * p.inner_bytes)[v] = outv;
        }
      } else {  // ALL_TO_ALL: dst[o][peer][inner] <- peer.src[o][rank][inner]
        for (int k = 0; k < n; ++k) {
          const int peer = (p.rank + k) % n;
          const uint8_t* base = (peer == p.rank) ? p.src : p.peers.base[peer] + HEADER_BYTES;
          reinterpret_cast<uint4*>(p.dst + (o * n + peer) * p.inner_bytes)[v] = *reinterpret_cast<const uint4*>(base + src_off);
        }
      }
    }
  }

  // ---- phase 2: tell the peers their staging areas are no longer being read by me
  if (arrive_is_last(flag_ptr(my_ws, OFF_COUNTERS, 1), p.target1)) {
    if (threadIdx.x < n && threadIdx.x != p.rank)
      st_release_sys(reinterpret_cast<uint32_t*>(p.peers.base[threadIdx.x] + OFF_DONE + p.rank * FLAG_STRIDE), p.epoch);
  }
}

}  // namespace apbs

using namespace apbs;

extern "C" {

int apb_symm_header_bytes() { return HEADER_BYTES; }

// One thread waits for ``*flag >= target`` with the kernels' bounded wait and a caller-chosen limit.
// With a flag that nothing raises this is the error path of every collective in miniature: the wait
// runs out, the status word is set, the kernel returns and the context stays usable.
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t target, uint32_t* status, unsigned long long limit_ns) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_ge<false>(flag, target, status, limit_ns);
}

int apb_symm_wait_probe(const uint32_t* flag, unsigned target, unsigned limit_ms, uint32_t* status, cudaStream_t st) {
  if (limit_ms > 2000u) limit_ms = 2000u;
  wait_probe_kernel<<<1, 32, 0, st>>>(flag, target, status, (unsigned long long)limit_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// peer_ptrs: host array of n workspace base pointers (this process's mappings of every rank's buffer).
// mode: 0 all-gather, 1 reduce-scatter (sum), 2 all-to-all.  ``multicast_base``: multicast address of the workspace for
// the reduce-scatter to sum through (NVLS), or 0 for plain peer loads.  Returns 0 or an error code.
int apb_symm_collective(int mode, const unsigned long long* peer_ptrs, int rank, int n, unsigned epoch, const void* src,
                        void* dst, long long outer, long long inner_bytes, int elem_kind, float scale, long long stage_capacity,
                        uint32_t* status, int num_ctas, unsigned target0, unsigned target1, unsigned long long multicast_base,
                        cudaStream_t st) {
  if (n > MAX_RANKS || n < 1) return 3;
  if ((inner_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return 3;
  const long long in_bytes = (mode == ALL_GATHER) ? outer * inner_bytes : outer * inner_bytes * n;
  if (in_bytes > stage_capacity) return 7;
  CollParams p;
  for (int i = 0; i < n; ++i) p.peers.base[i] = reinterpret_cast<uint8_t*>(peer_ptrs[i]);
  p.rank = rank; p.n = n; p.epoch = epoch;
  p.src = static_cast<const uint8_t*>(src); p.dst = static_cast<uint8_t*>(dst);
  p.outer = outer; p.inner_bytes = inner_bytes; p.elem_kind = elem_kind; p.scale = scale; p.status = status; p.target0 = target0; p.target1 = target1;
  p.mc_stage = (mode == REDUCE_SCATTER && multicast_base != 0ull)
                   ? reinterpret_cast<const uint8_t*>(multicast_base) + HEADER_BYTES : nullptr;
  if (mode == ALL_GATHER) symm_collective_kernel<ALL_GATHER><<<num_ctas, 512, 0, st>>>(p);
  else if (mode == REDUCE_SCATTER) symm_collective_kernel<REDUCE_SCATTER><<<num_ctas, 512, 0, st>>>(p);
  else if (mode == ALL_TO_ALL) symm_collective_kernel<ALL_TO_ALL><<<num_ctas, 512, 0, st>>>(p);
  else return 3;
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // extern "C"
