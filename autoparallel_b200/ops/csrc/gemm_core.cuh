// Body of the persistent tcgen05 GEMM CTA, shared by the plain GEMM (gemm_tcgen05.cu) and the GEMM
// kernels fused with a collective (gemm_fused.cu).
//
//   PAIR = false: one CTA per tile of 128 x 256 x 64, 4 TMA stages, two 256-column TMEM accumulators
//   PAIR = true:  a cluster of two CTAs per tile of 256 x 256 x 64 (tcgen05 cta_group::2): each CTA
//                 owns 128 rows of A, 128 of the 256 B rows (output columns) and 128 accumulator rows
//                 in its own TMEM; the MMA of the even CTA reads both halves of B, so every SM stages
//                 32 KB per k-block instead of 48 KB and six stages fit.  TMA transaction bytes and
//                 the epilogues' "accumulator free" arrivals go to the even CTA's barriers; "stage
//                 free" and "accumulator full" are committed by the MMA thread to each CTA's barrier
//                 separately (two plain commits; no multicast anywhere).
//   warp 0: TMA producer | warp 1: TMEM owner + MMA issuer | warps 2..5: epilogue
//   warp 6 (gather-fused kernels only): copy engine driver, see gather_comm_warp
//
// FUSE selects what the CTA does beyond a plain GEMM:
//   FUSE_NONE       nothing
//   FUSE_GATHER_A   rows (M) of A arrive shard by shard from peer GPUs: a seventh warp of every CTA
//                   pulls this CTA's share of each shard with bulk copies (TMA engine, no SM taken
//                   from the GEMM) and the producer waits for the per-shard "landed" counter
//                   before loading a tile of that shard
//   FUSE_GATHER_B   same for B; with a K-major B the shards partition N, with an MN-major B
//                   (stored [K, N]) they partition K, and the k-loop starts at the local shard
//   FUSE_REDUCE_SCATTER  the epilogue stores each fp32 tile into this rank's slot of the OWNER
//                   rank's staging area in peer memory (16-byte stores over NVLink); the owner
//                   sums the n slots once every rank has signalled completion
#pragma once
#include "ptx.cuh"
#include "symm_proto.cuh"

namespace apb {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16, GROUP_M = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int CHUNK_BYTES = BK * 128;  // one [BK x 64-element] MN-major box
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
constexpr int PAIR_STAGES = 6;  // 6 x (16 KB of A + 16 KB of B) = the same 192 KB as 4 x 48 KB
constexpr int EPI_STAGE_FLOATS = 32 * 33;  // per epilogue warp: one 32x32 fp32 block, padded
constexpr int GEMM_FUSED_RS_SMEM_BYTES = GEMM_SMEM_BYTES + 4 * EPI_STAGE_FLOATS * 4;
constexpr int AG_NBUF = 4, AG_CHUNK = 8192;  // bounce ring of the gather warp: 3 bulk loads in flight per CTA
constexpr int GEMM_FUSED_AG_SMEM_BYTES = GEMM_SMEM_BYTES + AG_NBUF * AG_CHUNK;
constexpr int GEMM_AG_THREADS = GEMM_THREADS + 32;

enum : int { FUSE_NONE = 0, FUSE_GATHER_A = 1, FUSE_GATHER_B = 2, FUSE_REDUCE_SCATTER = 3 };

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  int num_m_tiles, num_n_tiles;
  uint32_t* status;
  int groups = 1;  // grouped GEMM: G independent problems of the same M, N, K, stacked along a third tensor-map dim
  // dynamic tile scheduling (DYN): {next tile, pairs that have left, SM-pair requests, pairs that gave up their SMs};
  // all but the requests are zero between launches
  int* tile_counter = nullptr;
};

struct FuseParams {
  apbs::Peers peers;
  int rank, n;
  uint32_t epoch;
  // gather
  int rows_per_shard;          // rows of the gathered operand per rank (in its stored layout)
  uint32_t* landed;            // [n] local counters; shard s usable once landed[s] >= landed_target
  uint32_t landed_target;
  const uint8_t* shard_src;    // this rank's shard (any local memory)
  uint8_t* gbuf;               // local full-size operand, [n][shard_bytes]
  long long shard_bytes;
  uint32_t t_publish, t_pulled;  // running totals of the two arrival counters
  // reduce-scatter
  int rows_per_rank;           // rows of C owned by each rank (multiple of BM)
  int slot_bf16;               // partial tiles travel as bf16 (bf16 result) instead of fp32
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& tm, int& tn) {
  const int per_group = GROUP_M * num_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int r = t % per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

__device__ __forceinline__ void red_add_v4_sys(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Epilogue store of one accumulator row chunk: 32 consecutive columns of ``row`` starting at ``col``.
// ``c_off``: element offset of the output matrix inside C (grouped GEMM: group * M * ldc).
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, long long row, int col, const uint32_t (&r)[32], long long c_off = 0) {
  if (row >= p.M || col >= p.N) return;
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + c_off + row * p.ldc + col;
    if (col + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col + i < p.N) dst[i] = __uint_as_float(r[i]);
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + row * p.ldc + col;
    if (col + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
        v.y = pack_bf16(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
        v.z = pack_bf16(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
        v.w = pack_bf16(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
        reinterpret_cast<uint4*>(dst)[i] = v;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col + i < p.N) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
    }
  }
}

// ---------------------------------------------------------------------------- gather warp
// One lane per CTA drives the copy engine: it publishes this CTA's share of the local shard into the
// rank's symmetric staging area (and into the local full-size operand), then pulls the same share of
// every peer's staging area over NVLink.  Data moves global -> shared -> global as bulk copies through
// a ring of AG_NBUF bounce buffers, so AG_NBUF-1 loads are in flight per CTA (one per SM: a few MB
// in flight on the GPU, enough to cover the NVLink round trip) while the tensor cores run.
struct BounceRing {
  uint8_t* buf;
  uint64_t* bars;  // [AG_NBUF]
  uint32_t it;     // chunks moved so far by this CTA (buffer = it % AG_NBUF, parity from it / AG_NBUF)
};

// Copies chunks cta, cta+ncta, ... of [src, src+bytes) to dst0 (and dst1 if non-null); returns after
// every store has completed.  False on a timed-out load.
__device__ __forceinline__ bool ring_copy(BounceRing& r, const uint8_t* src, uint8_t* dst0, uint8_t* dst1, long long bytes,
                                          int cta, int ncta, volatile uint32_t* abort_flag) {
  const long long nchunks = (bytes + AG_CHUNK - 1) / AG_CHUNK;
  const int total = cta < nchunks ? (int)((nchunks - cta + ncta - 1) / ncta) : 0;
  auto off_of = [&](int j) { return ((long long)cta + (long long)j * ncta) * AG_CHUNK; };
  auto size_of = [&](long long off) { return (uint32_t)min((long long)AG_CHUNK, bytes - off); };
  auto issue_load = [&](int j) {
    const long long off = off_of(j);
    const uint32_t sz = size_of(off);
    const uint32_t b = (r.it + j) % AG_NBUF;
    mbar_expect_tx(&r.bars[b], sz);
    bulk_load(r.buf + b * AG_CHUNK, src + off, sz, &r.bars[b]);
  };
  for (int j = 0; j < AG_NBUF - 1 && j < total; ++j) issue_load(j);
  bool ok = true;
  for (int j = 0; j < total; ++j) {
    const uint32_t it = r.it + j, b = it % AG_NBUF, parity = (it / AG_NBUF) & 1u;
    if (!mbar_wait(&r.bars[b], parity, abort_flag)) {
      ok = false;
      break;
    }
    const long long off = off_of(j);
    const uint32_t sz = size_of(off);
    bulk_store(dst0 + off, r.buf + b * AG_CHUNK, sz);
    if (dst1 != nullptr) bulk_store(dst1 + off, r.buf + b * AG_CHUNK, sz);
    tma_store_commit();
    if (j + AG_NBUF - 1 < total) {
      bulk_store_wait_read_1();  // the buffer stored one iteration ago has been read: refill it
      issue_load(j + AG_NBUF - 1);
    }
  }
  r.it += total;
  tma_store_wait_all();
  return ok;
}

// Called by one lane.  ``cta`` / ``ncta``: this CTA among the GEMM CTAs (all of them resident).
__device__ __forceinline__ void gather_comm_warp(const GemmParams& p, const FuseParams& f, int cta, int ncta, BounceRing& ring,
                                                 volatile uint32_t* abort_flag) {
  using namespace apbs;
  uint8_t* my_ws = f.peers.base[f.rank];
  uint8_t* stage = my_ws + HEADER_BYTES;
  auto fail = [&]() {
    atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_PEER_FLAG);
    *abort_flag = 1;
  };
  // my staging area may be overwritten once every peer has finished pulling the previous epoch
  for (int k = 1; k < f.n; ++k)
    if (!wait_ge<true>(flag_ptr(my_ws, OFF_DONE, (f.rank + k) % f.n), f.epoch - 1, p.status)) return fail();
  if (!ring_copy(ring, f.shard_src, stage, f.gbuf + (long long)f.rank * f.shard_bytes, f.shard_bytes, cta, ncta, abort_flag)) return fail();
  fence_proxy_async_global();
  __threadfence_system();
  atomicAdd(f.landed + f.rank, 1u);
  if (atomicAdd(flag_ptr(my_ws, OFF_COUNTERS, 2), 1u) + 1u == f.t_publish) {
    __threadfence_system();  // every other CTA's share was fenced before its arrival
    for (int k = 1; k < f.n; ++k) st_release_sys(flag_ptr(f.peers.base[(f.rank + k) % f.n], OFF_READY, f.rank), f.epoch);
  }
  // Pull: one chunk sequence over all peers, so that loads from the next peer are already in flight
  // while the last stores of the previous one complete (a shard is only a few chunks per CTA).
  {
    const long long nchunks = (f.shard_bytes + AG_CHUNK - 1) / AG_CHUNK;
    const int per = cta < nchunks ? (int)((nchunks - cta + ncta - 1) / ncta) : 0;  // my chunks of each shard
    const int total = per * (f.n - 1);
    auto peer_of = [&](int q) { return (f.rank + 1 + q / per) % f.n; };
    auto off_of = [&](int q) { return ((long long)cta + (long long)(q % per) * ncta) * AG_CHUNK; };
    auto size_of = [&](long long off) { return (uint32_t)min((long long)AG_CHUNK, f.shard_bytes - off); };
    bool ok = true;
    auto issue_load = [&](int q) {
      const int peer = peer_of(q);
      if (q % per == 0) {  // first chunk of this peer: its staging area must be complete
        if (!wait_ge<true>(flag_ptr(my_ws, OFF_READY, peer), f.epoch, p.status)) {
          ok = false;
          return;
        }
        fence_proxy_async_global();
      }
      const long long off = off_of(q);
      const uint32_t sz = size_of(off);
      const uint32_t b = (ring.it + q) % AG_NBUF;
      mbar_expect_tx(&ring.bars[b], sz);
      bulk_load(ring.buf + b * AG_CHUNK, f.peers.base[peer] + HEADER_BYTES + off, sz, &ring.bars[b]);
    };
    int issued = 0;
    for (; issued < AG_NBUF - 1 && issued < total && ok; ++issued) issue_load(issued);
    for (int q = 0; q < total && ok; ++q) {
      const uint32_t it = ring.it + q, b = it % AG_NBUF, parity = (it / AG_NBUF) & 1u;
      if (!mbar_wait(&ring.bars[b], parity, abort_flag)) {
        ok = false;
        break;
      }
      const int peer = peer_of(q);
      const long long off = off_of(q);
      bulk_store(f.gbuf + (long long)peer * f.shard_bytes + off, ring.buf + b * AG_CHUNK, size_of(off));
      tma_store_commit();
      if (issued < total) {
        bulk_store_wait_read_1();  // the buffer stored one iteration ago has been read: refill it
        issue_load(issued++);
      }
      if (q % per == per - 1) {  // last chunk of this peer: publish the shard once its stores are complete
        tma_store_wait_all();
        fence_proxy_async_global();
        __threadfence();
        atomicAdd(f.landed + peer, 1u);
      }
    }
    ring.it += total;
    tma_store_wait_all();
    if (!ok) return fail();
    if (per == 0) {  // nothing to move for this CTA: still one arrival per shard
      for (int k = 1; k < f.n; ++k) atomicAdd(f.landed + (f.rank + k) % f.n, 1u);
    }
  }
  __threadfence_system();
  if (atomicAdd(flag_ptr(my_ws, OFF_COUNTERS, 3), 1u) + 1u == f.t_pulled) {
    __threadfence_system();
    for (int k = 1; k < f.n; ++k) st_release_sys(flag_ptr(f.peers.base[(f.rank + k) % f.n], OFF_DONE, f.rank), f.epoch);
  }
}

// cta / num_ctas: index of this CTA among the GEMM CTAs of the launch (fused kernels also run
// communication CTAs that are not counted here).  With PAIR, CTAs 2i and 2i+1 form cluster i.
// GROUPED: p.groups problems; operands are 3-D tensor maps [group][rows][inner] (FUSE_NONE only).
// ST_ARG: number of TMA stages (0 = as many as fit: 6 for pairs, 4 for single CTAs); fewer stages leave
// shared memory for a communication kernel's CTA to share the SM.
//
// DYN (CTA pairs, FUSE_NONE): tiles are handed out at run time.  The even CTA's producer thread takes the
// next tile index from a global counter and publishes it through a four-entry ring in BOTH CTAs'
// shared memory (remote store + remote mbarrier arrive); the odd CTA's producer, the MMA thread and
// the eight epilogue warps of the pair read it there and release the entry on the even CTA's
// barrier.  A pair that starts late or shares its SMs with another kernel (a communication kernel on
// another stream) simply takes fewer tiles, so nothing waits for the slowest pair's fixed share.
// Before each fetch the producer also looks at a request counter: a collective that is about to launch on
// another stream asks for some SM pairs (its kernel cannot become resident while every SM holds a
// persistent GEMM CTA), and that many pairs - never more than half of the launch - leave early; the tiles
// they would have taken go to the pairs that stay.
constexpr int TILE_RING = 4;
template <bool A_MN, bool B_MN, int FUSE, bool PAIR = false, bool GROUPED = false, int ST_ARG = 0, bool DYN = false>
__device__ __forceinline__ void gemm_cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                         const FuseParams& f, int cta, int num_ctas, uint8_t* smem_raw) {
  constexpr int ST = ST_ARG > 0 ? ST_ARG : (PAIR ? PAIR_STAGES : STAGES);
  constexpr int A_BYTES = A_STAGE_BYTES;                          // 128 rows of A per CTA
  constexpr int B_BYTES = PAIR ? B_STAGE_BYTES / 2 : B_STAGE_BYTES;  // PAIR: this CTA's 128 of the 256 B rows
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;
  constexpr int TM = PAIR ? 2 * BM : BM;                          // tile rows
  static_assert(ST * (A_BYTES + B_BYTES) <= STAGES * (A_STAGE_BYTES + B_STAGE_BYTES), "stages must fit the launch's shared memory");
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + ST * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ST * (A_BYTES + B_BYTES));
  uint64_t* full = bars;                     // [ST]  PAIR: the even CTA's are used
  uint64_t* empty = bars + ST;               // [ST]
  uint64_t* tmem_full = bars + 2 * ST;       // [2]
  uint64_t* tmem_empty = bars + 2 * ST + 2;  // [2]   PAIR: the even CTA's are used (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * ST + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint64_t* ring_bars = bars + 2 * ST + 6;   // [AG_NBUF], gather-fused kernels only
  static_assert(!DYN || (PAIR && FUSE == FUSE_NONE), "dynamic tiles: CTA pairs, plain GEMM");
  uint64_t* tile_ready = bars + 2 * ST + 10;  // [TILE_RING] DYN: entry published (1 arrival, in each CTA)
  uint64_t* tile_free = tile_ready + TILE_RING;  // [TILE_RING] DYN: entry read by all 10 readers of the pair (even CTA's)
  volatile int* tile_ring = reinterpret_cast<volatile int*>(tile_free + TILE_RING);  // [TILE_RING]
  static_assert((2 * PAIR_STAGES + 10 + 2 * TILE_RING) * 8 + TILE_RING * 4 <= 256, "barrier block");
  constexpr bool GATHER = FUSE == FUSE_GATHER_A || FUSE == FUSE_GATHER_B;
  const uint32_t half = PAIR ? cluster_ctarank() : 0u;  // 0 = even CTA: issues the MMAs, owns the shared barriers
  const int unit = PAIR ? (cta >> 1) : cta;             // tiles are dealt to CTAs or to CTA pairs
  const int num_units = PAIR ? (num_ctas >> 1) : num_ctas;
  const int num_m_units = (p.M + TM - 1) / TM;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_group = num_m_units * p.num_n_tiles;
  const int num_tiles = tiles_per_group * (GROUPED ? p.groups : 1);
  const int num_kb = (p.K + BK - 1) / BK;
  // rotation that makes every rank start on data it already owns
  int m_rot = 0, n_rot = 0, k_rot = 0;
  if (FUSE == FUSE_GATHER_A && !A_MN) m_rot = (f.rank * f.rows_per_shard) / TM;
  // N-partitioned gather (B shards are blocks of output columns): visit the tiles shard by shard,
  // local shard first, so that shard k is first touched after k/n of the GEMM (possible when a
  // shard is a whole number of tile columns); otherwise only rotate the start.
  int shard_n_tiles = 0;
  if (FUSE == FUSE_GATHER_B && !B_MN) {
    if (f.rows_per_shard % BN == 0 && p.num_n_tiles == (f.rows_per_shard / BN) * f.n) shard_n_tiles = f.rows_per_shard / BN;
    else n_rot = (f.rank * f.rows_per_shard) / BN;
  }
  auto map_tile = [&](int t, int& tm, int& tn) {
    if (GROUPED) t %= tiles_per_group;
    if (shard_n_tiles > 0) {
      const int per_shard = num_m_units * shard_n_tiles;
      const int s = t / per_shard;
      tile_coords(t - s * per_shard, num_m_units, shard_n_tiles, tm, tn);
      tn += ((s + f.rank) % f.n) * shard_n_tiles;
    } else {
      tile_coords(t, num_m_units, p.num_n_tiles, tm, tn);
      tm = (tm + m_rot) % num_m_units;
      tn = (tn + n_rot) % p.num_n_tiles;
    }
  };
  if (FUSE == FUSE_GATHER_B && B_MN) k_rot = (f.rank * f.rows_per_shard) / BK;
  if (FUSE == FUSE_GATHER_A && A_MN) k_rot = (f.rank * f.rows_per_shard) / BK;
  if (FUSE == FUSE_REDUCE_SCATTER) m_rot = (((f.rank + 1) % f.n) * f.rows_per_rank) / TM;  // own rows last

  // Tile sequence of one role (each role keeps its own position ``it``).  Static: unit, unit + num_units, ...
  // Dynamic: entry ``it`` of the ring; -1 ends the sequence (also after a timed-out wait).
  auto read_tile = [&](int& it) -> int {
    if (!DYN) {
      const long long t = (long long)unit + (long long)it * num_units;
      ++it;
      return t < num_tiles ? (int)t : -1;
    }
    const int slot = it % TILE_RING;
    if (!mbar_wait_cluster(&tile_ready[slot], (it / TILE_RING) & 1, abort_flag)) {
      atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_FULL);
      *abort_flag = 1;
      return -1;
    }
    const int t = tile_ring[slot];
    mbar_arrive_cluster(map_to_cta(&tile_free[slot], 0));
    ++it;
    return t;
  };
  // Even CTA's producer thread (DYN): take the next tile and publish it to both CTAs.
  auto fetch_tile = [&](int& it) -> int {
    const int slot = it % TILE_RING;
    if (!mbar_wait_cluster(&tile_free[slot], ((it / TILE_RING) & 1) ^ 1, abort_flag)) {
      atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_EMPTY);
      *abort_flag = 1;
      return -1;
    }
    int t = -1;
    bool leave = false;
    if (*reinterpret_cast<volatile int*>(p.tile_counter + 2) > 0) {
      if (atomicSub(p.tile_counter + 2, 1) > 0) {
        if (atomicAdd(p.tile_counter + 3, 1) < num_units / 2) {
          leave = true;  // this pair hands its two SMs to the waiting kernel
        } else {
          atomicSub(p.tile_counter + 3, 1);
          atomicAdd(p.tile_counter + 2, 1);
        }
      } else {
        atomicAdd(p.tile_counter + 2, 1);  // somebody else took the last request
      }
    }
    if (!leave) {
      t = atomicAdd(p.tile_counter, 1);
      if (t >= num_tiles) t = -1;
    }
    tile_ring[slot] = t;
    st_cluster_u32(map_to_cta(const_cast<int*>(&tile_ring[slot]), 1), (uint32_t)t);
    mbar_arrive_cluster(map_to_cta(&tile_ready[slot], 0));
    mbar_arrive_cluster(map_to_cta(&tile_ready[slot], 1));
    ++it;
    if (t < 0 && atomicAdd(p.tile_counter + 1, 1) == num_units - 1) {
      // every pair has left: zero the per-launch counters for the next launch (requests carry over)
      p.tile_counter[0] = 0;
      p.tile_counter[1] = 0;
      p.tile_counter[3] = 0;
      __threadfence();
    }
    return t;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], PAIR ? 256 : 128);
    }
    if (DYN)
      for (int b = 0; b < TILE_RING; ++b) {
        mbar_init(&tile_ready[b], 1);
        mbar_init(&tile_free[b], 10);  // odd CTA: producer + 4 epilogue warps; even CTA: MMA thread + 4 epilogue warps
      }
    if (GATHER)
      for (int b = 0; b < AG_NBUF; ++b) mbar_init(&ring_bars[b], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) {
    cluster_arrive();  // the other CTA's barriers are initialised before anything is signalled to them
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t landed_mask = 0;  // shards already seen as landed: checked once, never polled again
      auto shard_ready = [&](int s) -> bool {
        if (landed_mask & (1u << s)) return true;
        if (!apbs::wait_ge<false>(f.landed + s, f.landed_target, p.status)) return false;
        fence_proxy_async_global();
        landed_mask |= 1u << s;
        return true;
      };
      int tile_it = 0;
      for (int t = (DYN && half == 0) ? fetch_tile(tile_it) : read_tile(tile_it); t >= 0 && ok;
           t = (DYN && half == 0) ? fetch_tile(tile_it) : read_tile(tile_it)) {
        int tm, tn;
        map_tile(t, tm, tn);
        // rows of A and of B that THIS CTA stages
        const int m0 = tm * TM + (int)half * BM, n0 = tn * BN + (int)half * B_ROWS;
        const int grp = GROUPED ? t / tiles_per_group : 0;
        if ((FUSE == FUSE_GATHER_A && !A_MN) || (FUSE == FUSE_GATHER_B && !B_MN)) {
          // the tile's rows of the gathered operand must have landed
          const int r0 = (FUSE == FUSE_GATHER_A) ? m0 : n0;
          const int extent = max(1, (FUSE == FUSE_GATHER_A) ? min(BM, p.M - m0) : min(B_ROWS, p.N - n0));
          const int s0 = r0 / f.rows_per_shard, s1 = (r0 + extent - 1) / f.rows_per_shard;
          for (int s = s0; s <= s1 && ok; ++s) ok = shard_ready(s);
          if (!ok) {
            *abort_flag = 1;
            break;
          }
        }
        for (int kb0 = 0; kb0 < num_kb; ++kb0) {
          const int kb = (kb0 + k_rot) % num_kb;
          if ((FUSE == FUSE_GATHER_B && B_MN) || (FUSE == FUSE_GATHER_A && A_MN)) {
            const int r0 = kb * BK;
            const int s0 = r0 / f.rows_per_shard, s1 = (min(r0 + BK, p.K) - 1) / f.rows_per_shard;
            for (int s = s0; s <= s1 && ok; ++s) ok = shard_ready(s);
            if (!ok) {
              *abort_flag = 1;
              break;
            }
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            break;
          }
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          // one load helper for the four cases (pair or not, 2-D or grouped 3-D)
          const uint32_t full_addr = PAIR ? map_to_cta(&full[stage], 0) : 0u;
          auto load = [&](uint8_t* dst, const CUtensorMap* tm_, int x, int y) {
            if (PAIR) {
              if (GROUPED) tma_load_3d_pair(dst, tm_, full_addr, x, y, grp);
              else tma_load_2d_pair(dst, tm_, full_addr, x, y);
            } else {
              if (GROUPED) tma_load_3d(dst, tm_, &full[stage], x, y, grp);
              else tma_load_2d(dst, tm_, &full[stage], x, y);
            }
          };
          if (PAIR) {
            if (half == 0) mbar_expect_tx(&full[stage], 2 * (A_BYTES + B_BYTES));  // both CTAs' bytes land on the even CTA's barrier
          } else {
            mbar_expect_tx(&full[stage], A_BYTES + B_BYTES);
          }
          if (!A_MN) {
            load(a_dst, &tmA, kb * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) load(a_dst + c * CHUNK_BYTES, &tmA, m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            load(b_dst, &tmB, kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < B_ROWS / 64; ++c) load(b_dst + c * CHUNK_BYTES, &tmB, n0 + c * 64, kb * BK);
          }
          if (++stage == ST) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && half == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      int tile_it = 0;
      for (int t = read_tile(tile_it); t >= 0 && ok; t = read_tile(tile_it)) {
        if (!mbar_wait(&tmem_empty[buf], buf_phase ^ 1, abort_flag)) {
          atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_FULL);
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + k * (UMMA_K * 128), CHUNK_BYTES, 1024)
                                         : make_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + k * (UMMA_K * 128), CHUNK_BYTES, 1024)
                                         : make_smem_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
            if (PAIR) umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // stage reusable once these MMAs have read it (PAIR: in both CTAs)
          if (PAIR) {
            umma_commit_pair(map_to_cta(&empty[stage], 0));
            umma_commit_pair(map_to_cta(&empty[stage], 1));
          } else {
            umma_commit(&empty[stage]);
          }
          if (++stage == ST) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (PAIR) {
          umma_commit_pair(map_to_cta(&tmem_full[buf], 0));
          umma_commit_pair(map_to_cta(&tmem_full[buf], 1));
        } else {
          umma_commit(&tmem_full[buf]);
        }
        if (++buf == 2) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
    }
  } else if (GATHER && warp == 6) {
    // ------------------------------------------------------------------ gather warp
    if (lane == 0) {
      BounceRing ring{smem + ST * (A_BYTES + B_BYTES) + 256, ring_bars, 0u};
      gather_comm_warp(p, f, cta, num_ctas, ring, abort_flag);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int buf = 0;
    uint32_t buf_phase = 0;
    int tile_it = 0;
    auto next_epi_tile = [&]() -> int {  // lane 0 reads the sequence, the warp follows
      int t = 0;
      if (lane == 0) t = read_tile(tile_it);
      return __shfl_sync(0xffffffffu, t, 0);
    };
    for (int t = next_epi_tile(); t >= 0; t = next_epi_tile()) {
      int tm, tn;
      map_tile(t, tm, tn);
      const long long cta_row0 = (long long)tm * TM + (long long)half * BM;  // first of this CTA's 128 rows
      if (!mbar_wait(&tmem_full[buf], buf_phase, abort_flag)) {
        atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const long long row = cta_row0 + q * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
      float* rs_base = nullptr;
      if (FUSE == FUSE_REDUCE_SCATTER) {
        const int owner = (int)(cta_row0 / f.rows_per_rank);
        // the owner zeroes its accumulation buffer at the start of the step and then raises "ready"
        bool ok = true;
        if (owner != f.rank) {
          if (lane == 0) ok = apbs::wait_ge<true>(apbs::flag_ptr(f.peers.base[f.rank], apbs::OFF_READY, owner), f.epoch, p.status);
        } else {
          if (lane == 0) ok = apbs::wait_ge<false>(apbs::flag_ptr(f.peers.base[f.rank], apbs::OFF_READY, owner), f.epoch, p.status);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) {
          *abort_flag = 1;
          break;
        }
        // slot ``rank`` of the owner's staging area: [n][rows_per_rank][N], fp32 or bf16; rs_base is kept
        // in units of fp32 elements of an fp32 slot and halved below for bf16 slots
        rs_base = reinterpret_cast<float*>(f.peers.base[owner] + apbs::HEADER_BYTES) +
                  ((long long)f.rank * f.rows_per_rank + (row - (long long)owner * f.rows_per_rank)) * p.N;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (FUSE == FUSE_REDUCE_SCATTER) {
          // Transpose the warp's 32x32 block through shared memory so that every store instruction
          // writes four 128-byte row segments: NVLink moves full segments instead of 16-byte crumbs.
          float* stg = reinterpret_cast<float*>(smem + ST * (A_BYTES + B_BYTES) + 256) + (warp - 2) * EPI_STAGE_FLOATS;
#pragma unroll
          for (int i = 0; i < 32; ++i) stg[lane * 33 + i] = __uint_as_float(r[i]);
          __syncwarp();
          const long long row0 = cta_row0 + q * 32;  // first row of this warp's block
          float* blk = rs_base - (long long)lane * p.N;         // rs_base points at this lane's row
          if (f.slot_bf16) {
            // 8 bf16 (16 bytes) per lane, 4 lanes per 64-byte row segment, 8 rows per instruction
            __nv_bfloat16* blk16 = reinterpret_cast<__nv_bfloat16*>(f.peers.base[(int)(cta_row0 / f.rows_per_rank)] + apbs::HEADER_BYTES) +
                                   (blk - reinterpret_cast<float*>(f.peers.base[(int)(cta_row0 / f.rows_per_rank)] + apbs::HEADER_BYTES));
            const int sub8 = lane >> 2, seg8 = (lane & 3) * 8;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int rr = sub8 + 8 * j;
              if (row0 + rr < p.M) {
                const float* sp = stg + rr * 33 + seg8;
                __nv_bfloat16* dst = blk16 + (long long)rr * p.N + col + seg8;
                if (col + seg8 + 8 <= p.N) {
                  uint4 v;
                  v.x = pack_bf16(sp[0], sp[1]);
                  v.y = pack_bf16(sp[2], sp[3]);
                  v.z = pack_bf16(sp[4], sp[5]);
                  v.w = pack_bf16(sp[6], sp[7]);
                  *reinterpret_cast<uint4*>(dst) = v;
                } else {
                  for (int e = 0; e < 8; ++e)
                    if (col + seg8 + e < p.N) dst[e] = __float2bfloat16(sp[e]);
                }
              }
            }
            __syncwarp();
            continue;
          }
          const int sub = lane >> 3, seg = (lane & 7) * 4;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rr = sub + 4 * j;
            if (row0 + rr < p.M) {
              const float* sp = stg + rr * 33 + seg;
              float* dst = blk + (long long)rr * p.N + col + seg;
              if (col + seg + 4 <= p.N) {
                *reinterpret_cast<float4*>(dst) = make_float4(sp[0], sp[1], sp[2], sp[3]);
              } else {
                for (int e = 0; e < 4; ++e)
                  if (col + seg + e < p.N) dst[e] = sp[e];
              }
            }
          }
          __syncwarp();
          continue;
        }
        store_row_chunk(p, row, col, r, GROUPED ? (long long)(t / tiles_per_group) * p.M * p.ldc : 0);
      }
      tc_fence_before();
      if (PAIR) mbar_arrive_cluster(map_to_cta(&tmem_empty[buf], 0));
      else mbar_arrive(&tmem_empty[buf]);
      if (++buf == 2) {
        buf = 0;
        buf_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) {
    cluster_arrive();  // neither CTA frees TMEM (or exits) while the other may still read or signal
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------ host helpers
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map, innermost extent ``inner`` (contiguous), 128-byte swizzle, box 64 x box_outer.
inline int make_map(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld_elems, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return 1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {64, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

// 3-D bf16 tensor map [groups][outer][inner] (dense: group stride = outer * ld), box 64 x box_outer x 1.
inline int make_map_3d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t groups, uint64_t ld_elems,
                       uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return 1;
  cuuint64_t dims[3] = {inner, outer, groups};
  cuuint64_t strides[2] = {ld_elems * 2, ld_elems * outer * 2};
  cuuint32_t box[3] = {64, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

// Tensor maps of both operands for C[M,N] = opA * opB (see gemm_tcgen05.cu for the conventions).
// ``pair``: the CTA-pair kernels load a K-major B in boxes of 128 rows (each CTA stages half of the tile columns).
inline int make_operand_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, const void* B, int M, int N, int K,
                             long long lda, long long ldb, int a_mn_major, int b_mn_major, bool pair = false) {
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return 3;
  int e = !a_mn_major ? make_map(tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BM)
                      : make_map(tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BK);
  if (e) return e;
  return !b_mn_major ? make_map(tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, pair ? BN / 2 : BN)
                     : make_map(tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BK);
}

}  // namespace apb
