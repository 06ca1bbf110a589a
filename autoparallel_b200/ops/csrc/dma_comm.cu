// Copy-engine collectives over NVLink peer memory: the data movement of an all-gather is issued as
// plain asynchronous device-to-device copies whose source is a peer GPU's mapping of a symmetric
// arena, so it runs on the GPU's copy engines and takes no SM, no shared memory and no register
// from the persistent tensor-core kernels that own every SM during a training step.
//
// What makes this safe without a handshake per collective: the tensors gathered this way are the
// low-precision parameter shards that the optimizer writes once per step into the arena.  Two
// arena-wide barriers per step (before and after the optimizer kernel) order every pull of the
// forward and backward pass against the only writer.  The barrier is one tiny kernel per rank: each
// rank raises its epoch on every peer's flag block and waits (bounded, ~2 s) for every peer's epoch
// on its own; on expiry it records ST_TIMEOUT_PEER in the status word and returns.
//
// Reduce-scatter, second half of this file: the partial results are pushed by the copy engines into
// the owner's slots of a symmetric staging ring and the owner adds the slots with a light kernel
// (no shared memory, so it becomes resident beside a persistent GEMM CTA).  "Pushed" / "consumed"
// notifications are tiny kernels on the communication stream that raise or wait for sequence numbers.
//
// Reference counterpart: c10d functional all_gather_into_tensor / reduce_scatter_tensor on NCCL
// (autoparallel/collectives.py:89-154 in the reference), whose kernels compete with compute for SMs.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "symm_proto.cuh"

namespace apbd {
using namespace apbs;

// Flag block of one communicator (one per process group; lives inside the arena, zeroed once):
//   [ barrier: MAX_RANKS x 128 B | pushed[ring entry][rank] | consumed[ring entry][rank] ]
constexpr int ARENA_OFF_BARRIER = 0;
constexpr int RING_MAX = 8;
// pushed[b][r] on owner: rank r's partial for ring entry b, sequence number s, has landed
constexpr int ARENA_OFF_PUSHED = MAX_RANKS * FLAG_STRIDE;
// consumed[b][r] on pusher r': owner r has summed ring entry b of sequence s (so r' may overwrite its slot there)
constexpr int ARENA_OFF_CONSUMED = ARENA_OFF_PUSHED + RING_MAX * MAX_RANKS * FLAG_STRIDE;
constexpr int ARENA_FLAG_BYTES = ARENA_OFF_CONSUMED + RING_MAX * MAX_RANKS * FLAG_STRIDE;

struct RankList {
  unsigned long long base[MAX_RANKS];  // flag block of every rank of the group, as mapped in this process
};

__global__ void arena_barrier_kernel(RankList peers, int rank, int n, uint32_t epoch, uint32_t* status) {
  const int t = threadIdx.x;
  if (t < n && t != rank) {
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[t] + ARENA_OFF_BARRIER + rank * FLAG_STRIDE), epoch);
    wait_ge<true>(reinterpret_cast<const uint32_t*>(peers.base[rank] + ARENA_OFF_BARRIER + t * FLAG_STRIDE), epoch, status);
  }
}

// raise flag ``idx`` of block ``off`` to ``value`` on every peer (thread t -> peer t)
__global__ void arena_signal_kernel(RankList peers, int rank, int n, int off, int idx, uint32_t value) {
  const int t = threadIdx.x;
  if (t < n && t != rank) st_release_sys(reinterpret_cast<uint32_t*>(peers.base[t] + off + idx * FLAG_STRIDE), value);
}

// wait until flags [idx0 + t] (t < n, t != rank) of my block ``off`` are >= value
__global__ void arena_wait_kernel(unsigned long long my_base, int rank, int n, int off, int idx0, uint32_t value, uint32_t* status) {
  const int t = threadIdx.x;
  if (t < n && t != rank) wait_ge<true>(reinterpret_cast<const uint32_t*>(my_base + off + (idx0 + t) * FLAG_STRIDE), value, status);
}

// out[i] = scale * (own[i] + sum over the n-1 peer slots), fp32, 16 bytes per thread per step.  ``slots`` is
// [n][elems] in the owner's staging entry; slot ``rank`` is unused (the owner's partial is read in place).
template <int N>
__global__ void __launch_bounds__(256) slot_sum_kernel(const float4* __restrict__ own, const float4* __restrict__ slots, float4* __restrict__ out,
                                                       long long vecs, long long slot_vecs, int rank, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
    float4 acc = own[i];
    float4 v[N];
#pragma unroll
    for (int k = 0; k < N; ++k)
      if (k != rank) v[k] = slots[k * slot_vecs + i];
#pragma unroll
    for (int k = 0; k < N; ++k)
      if (k != rank) {
        acc.x += v[k].x;
        acc.y += v[k].y;
        acc.z += v[k].z;
        acc.w += v[k].w;
      }
    acc.x *= scale;
    acc.y *= scale;
    acc.z *= scale;
    acc.w *= scale;
    out[i] = acc;
  }
}

}  // namespace apbd

using namespace apbd;

extern "C" {

int apb_dma_flag_bytes() { return ARENA_FLAG_BYTES; }
int apb_dma_ring_max() { return RING_MAX; }

static int fill(RankList& l, const unsigned long long* bases, int n) {
  if (n < 1 || n > MAX_RANKS) return 3;
  for (int i = 0; i < n; ++i) l.base[i] = bases[i];
  return 0;
}

// ``flags``: flag block of every group member; ``bases``: the arena base of every group member (both as mapped here).
int apb_dma_barrier(const unsigned long long* flags, int rank, int n, unsigned epoch, uint32_t* status, cudaStream_t st) {
  RankList l;
  if (fill(l, flags, n)) return 3;
  arena_barrier_kernel<<<1, 32, 0, st>>>(l, rank, n, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// All-gather of a tensor that sits at byte ``offset`` of every rank's arena: dst[o][r][inner] <- rank r's src[o][inner].
// ``bases`` are the arena bases of the n group members as mapped here; copies start at the next rank and rotate, so
// at any moment the n ranks read from n different peers.
int apb_dma_all_gather(void* dst, const unsigned long long* bases, long long offset, long long outer, long long inner_bytes,
                       int rank, int n, cudaStream_t st) {
  if (n < 1 || n > MAX_RANKS || outer < 1 || inner_bytes < 1) return 3;
  for (int k = 1; k <= n; ++k) {
    const int peer = (rank + k) % n;
    const char* src = reinterpret_cast<const char*>(bases[peer]) + offset;
    char* d = static_cast<char*>(dst) + (long long)peer * inner_bytes;
    cudaError_t e;
    if (outer == 1) e = cudaMemcpyAsync(d, src, (size_t)inner_bytes, cudaMemcpyDeviceToDevice, st);
    else e = cudaMemcpy2DAsync(d, (size_t)(inner_bytes * n), src, (size_t)inner_bytes, (size_t)inner_bytes, (size_t)outer,
                               cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return 4;
  }
  return 0;
}

// Reduce-scatter, push half.  ``src`` is this rank's partial [n][chunk_bytes] (chunk r belongs to rank r).  Ring entry
// ``entry`` of every owner's staging area holds n slots of ``slot_bytes``; this rank writes slot ``rank``.  Before
// the copies the stream waits until every owner has consumed the entry's previous use (sequence ``seq - ring``);
// after them it raises pushed[entry][rank] = seq on every owner.
int apb_dma_rs_push(const void* src, const unsigned long long* bases, const unsigned long long* flags, long long stage_offset,
                    long long slot_bytes, long long chunk_bytes, int entry, int ring, unsigned seq, int rank, int n,
                    uint32_t* status, cudaStream_t st) {
  RankList l;
  if (fill(l, flags, n) || entry < 0 || entry >= RING_MAX || ring < 1 || ring > RING_MAX || chunk_bytes > slot_bytes) return 3;
  if (seq > (unsigned)ring)
    arena_wait_kernel<<<1, 32, 0, st>>>(flags[rank], rank, n, ARENA_OFF_CONSUMED, entry * MAX_RANKS, seq - (unsigned)ring, status);
  for (int k = 1; k < n; ++k) {
    const int owner = (rank + k) % n;
    char* d = reinterpret_cast<char*>(bases[owner]) + stage_offset + ((long long)entry * n + rank) * slot_bytes;
    if (cudaMemcpyAsync(d, static_cast<const char*>(src) + (long long)owner * chunk_bytes, (size_t)chunk_bytes,
                        cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return 4;
  }
  arena_signal_kernel<<<1, 32, 0, st>>>(l, rank, n, ARENA_OFF_PUSHED, entry * MAX_RANKS + rank, seq);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// Reduce-scatter, owner half: wait for every peer's push of sequence ``seq`` into ring entry ``entry``, add the
// slots to this rank's own chunk of ``src`` and write ``dst`` (fp32, scaled); then tell the peers the entry is free.
int apb_dma_rs_sum(const void* src, void* dst, const unsigned long long* bases, const unsigned long long* flags,
                   long long stage_offset, long long slot_bytes, long long chunk_bytes, int entry, unsigned seq, float scale,
                   int rank, int n, int num_ctas, uint32_t* status, cudaStream_t st) {
  RankList l;
  if (fill(l, flags, n) || entry < 0 || entry >= RING_MAX || (chunk_bytes & 15) || (slot_bytes & 15)) return 3;
  arena_wait_kernel<<<1, 32, 0, st>>>(flags[rank], rank, n, ARENA_OFF_PUSHED, entry * MAX_RANKS, seq, status);
  const float4* own = reinterpret_cast<const float4*>(static_cast<const char*>(src) + (long long)rank * chunk_bytes);
  const float4* slots = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(bases[rank]) + stage_offset +
                                                        (long long)entry * n * slot_bytes);
  const long long vecs = chunk_bytes >> 4, slot_vecs = slot_bytes >> 4;
  long long want = (vecs + 255) / 256;
  const int grid = (int)(want < num_ctas ? (want < 1 ? 1 : want) : num_ctas);
#define APB_SUM(NN) \
  case NN: slot_sum_kernel<NN><<<grid, 256, 0, st>>>(own, slots, static_cast<float4*>(dst), vecs, slot_vecs, rank, scale); break;
  switch (n) {
    APB_SUM(2) APB_SUM(3) APB_SUM(4) APB_SUM(5) APB_SUM(6) APB_SUM(7) APB_SUM(8)
    default: return 3;
  }
#undef APB_SUM
  arena_signal_kernel<<<1, 32, 0, st>>>(l, rank, n, ARENA_OFF_CONSUMED, entry * MAX_RANKS + rank, seq);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // extern "C"
