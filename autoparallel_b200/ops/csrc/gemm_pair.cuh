// Body of the persistent tcgen05 GEMM run by a PAIR of CTAs (cluster of two, tcgen05 cta_group::2).
//
//   pair tile 256 x 256 x 64; each CTA owns 128 rows of A, 128 of the 256 B rows (output columns)
//   and 128 accumulator rows in its own TMEM; the MMA of the even CTA reads both halves of B, so
//   every SM stages 32 KB per k-block instead of 48 KB and six stages fit in shared memory.
//
//   warp 0: TMA producer (both CTAs; completion is counted on the even CTA's barrier)
//   warp 1: TMEM owner (both CTAs); MMA issuer (even CTA only)
//   warps 2..5: epilogue of the CTA's own 128 accumulator rows
//
// Signals that cross the pair: TMA transaction bytes and epilogue "accumulator free" arrivals go to
// the even CTA's barriers; "stage free" and "accumulator full" are committed by the MMA thread to
// the barrier of each CTA separately (two plain commits, no multicast anywhere in this file).
// All mbarrier waits are bounded as in gemm_core.cuh.
#pragma once
#include "gemm_core.cuh"

namespace apb {

constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = BM * BK * 2;         // 128 rows of A
constexpr int P_B_BYTES = (BN / 2) * BK * 2;   // this CTA's half of the 256 B rows
constexpr int GEMM_PAIR_SMEM_BYTES = P_STAGES * (P_A_BYTES + P_B_BYTES) + 1024 /*align*/ + 256 /*barriers*/;

// pair / num_pairs: index of this CTA pair among the pairs of the launch.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void gemm_pair_cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int pair,
                                              int num_pairs, uint8_t* smem_raw) {
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + P_STAGES * P_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * (P_A_BYTES + P_B_BYTES));
  uint64_t* full = bars;                           // [P_STAGES]  used in the even CTA
  uint64_t* empty = bars + P_STAGES;               // [P_STAGES]  one per CTA
  uint64_t* tmem_full = bars + 2 * P_STAGES;       // [2]         one per CTA
  uint64_t* tmem_empty = bars + 2 * P_STAGES + 2;  // [2]         used in the even CTA (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = even CTA: issues the MMAs, owns the shared barriers
  const int num_m_pairs = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = num_m_pairs * p.num_n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // the other CTA's barriers are initialised before anything is signalled to them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < num_tiles; t += num_pairs) {
        int tm, tn;
        tile_coords(t, num_m_pairs, p.num_n_tiles, tm, tn);
        const int m0 = tm * 2 * BM + (int)cta * BM;
        const int n0 = tn * BN + (int)cta * (BN / 2);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            break;
          }
          const uint32_t full_addr = map_to_cta(&full[stage], 0);
          if (cta == 0) mbar_expect_tx(&full[stage], 2 * (P_A_BYTES + P_B_BYTES));  // both CTAs' bytes
          uint8_t* a_dst = sA + stage * P_A_BYTES;
          uint8_t* b_dst = sB + stage * P_B_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, &tmA, full_addr, kb * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(a_dst + c * CHUNK_BYTES, &tmA, full_addr, m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, &tmB, full_addr, kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c) tma_load_2d_pair(b_dst + c * CHUNK_BYTES, &tmB, full_addr, n0 + c * 64, kb * BK);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
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
          const uint32_t a_addr = smem_u32(sA + stage * P_A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * P_B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + k * (UMMA_K * 128), CHUNK_BYTES, 1024)
                                         : make_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + k * (UMMA_K * 128), CHUNK_BYTES, 1024)
                                         : make_smem_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
            umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is reusable in BOTH CTAs once these MMAs have read it
          umma_commit_pair(map_to_cta(&empty[stage], 0));
          umma_commit_pair(map_to_cta(&empty[stage], 1));
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(map_to_cta(&tmem_full[buf], 0));
        umma_commit_pair(map_to_cta(&tmem_full[buf], 1));
        if (++buf == 2) {
          buf = 0;
          buf_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int buf = 0;
    uint32_t buf_phase = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int tm, tn;
      tile_coords(t, num_m_pairs, p.num_n_tiles, tm, tn);
      if (!mbar_wait(&tmem_full[buf], buf_phase, abort_flag)) {
        atomicCAS(p.status, 0u, (uint32_t)ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const long long row = (long long)tm * 2 * BM + (long long)cta * BM + q * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        store_row_chunk(p, row, n0 + c * 32, r);
      }
      tc_fence_before();
      mbar_arrive_cluster(map_to_cta(&tmem_empty[buf], 0));
      if (++buf == 2) {
        buf = 0;
        buf_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // neither CTA frees TMEM (or exits) while the other may still read or signal
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace apb
