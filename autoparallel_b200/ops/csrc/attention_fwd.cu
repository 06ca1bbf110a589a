// Causal / full attention forward for head dim 128 on tcgen05 (sm_100a), grouped-query heads read in place.
//
//   q [B, S, H, 128]  k, v [B, Sk, Hkv, 128]  (bf16, contiguous)  ->  out [B, S, H, 128] bf16, lse [B, H, S] fp32
//
// One CTA owns 256 query rows of one (batch, head): two 128-row tiles that share every K / V tile.
//   warp 0      TMA producer: Q once, then K_0 V_0 K_1 V_1 ... through a ring of three 32-KB slots
//   warp 1      MMA issuer:   S_t = Q_t K_j^T   (M 128, N 128, K 128; both operands K-major)
//                             PV_t = P_t V_j    (A = P_t K-major from shared memory, B = V_j MN-major)
//   warps 2-3   idle (they complete the first warpgroup, which gives most of its registers away)
//   warps 4-7   softmax of tile 0, one query row per thread;  warps 8-11: tile 1 (224 registers per thread)
// TMEM (512 columns): S_0 | S_1 | PV_0 | PV_1, 128 fp32 columns each.  The output row lives in registers:
// every PV_t product is a fresh accumulator that the row's thread adds to its running sum, rescaled when the
// row maximum moves.  While one tile's threads are in the softmax, the tensor core works for the other tile.
//
// Barriers (all waits bounded; a wait that runs out records a status code, raises the CTA's abort flag and
// every role falls through to the common exit, where TMEM is freed):
//   kv_full[slot] / kv_empty[slot]   TMA -> MMA / MMA (commit) -> TMA
//   s_full[t]    MMA commit: S_t of iteration j is in TMEM
//   p_full[t]    128 softmax threads: P_t of iteration j is in shared memory, S_t and PV_t(j-1) have been read
//   pv_full[t]   MMA commit: PV_t of iteration j is in TMEM (and P_t may be overwritten)
//
// Reference counterpart: the fused SDPA call in examples/llama3 of the reference (cuDNN / flash kernels).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_core.cuh"
#include "ptx.cuh"

namespace apb_attn {
using namespace apb;

constexpr int HD = 128;                  // head dim
constexpr int TQ = 128;                  // rows of one query tile
constexpr int NQ = 2;                    // query tiles per CTA
constexpr int TK = 128;                  // keys per K / V tile
constexpr int HALF_BYTES = TQ * 128;     // [128 rows x 64 bf16] swizzled sub-tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;
constexpr int RING = 3;
constexpr int OFF_Q = 0;
constexpr int OFF_P = OFF_Q + NQ * TILE_BYTES;
constexpr int OFF_RING = OFF_P + NQ * TILE_BYTES;
constexpr int OFF_BARS = OFF_RING + RING * TILE_BYTES;
constexpr int ATTN_SMEM_BYTES = OFF_BARS + 256 + 1024;  // + barriers + slack for the 1024-byte alignment
constexpr int ATTN_THREADS = 128 * (1 + NQ);  // one warpgroup of producer / MMA / idle warps, one per query tile
static_assert(ATTN_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

enum : uint32_t { ST_ATTN_KV_FULL = 7, ST_ATTN_KV_EMPTY = 8, ST_ATTN_ACC_FULL = 9, ST_ATTN_ACC_EMPTY = 10 };

struct AttnParams {
  __nv_bfloat16* out;  // [B * S, H * 128]
  float* lse;          // [B, H, S]
  int B, S, Sk, H, Hkv;
  int causal;          // requires S == Sk
  float scale_log2;    // softmax scale * log2(e)
  uint32_t* status;
};

// Register reallocation between warpgroups (all four warps of a group execute the same instruction): the first
// group keeps 56 registers per thread, the softmax groups grow to 224: 4 x 32 x 56 + 8 x 32 x 224 = 64512 <= 65536.
__device__ __forceinline__ void regs_shrink() { asm volatile("setmaxnreg.dec.sync.aligned.u32 56;"); }
__device__ __forceinline__ void regs_grow() { asm volatile("setmaxnreg.inc.sync.aligned.u32 224;"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(ATTN_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
  uint64_t* q_full = bars;             // 1
  uint64_t* kv_full = bars + 1;        // RING
  uint64_t* kv_empty = kv_full + RING; // RING
  uint64_t* s_full = kv_empty + RING;  // NQ
  uint64_t* p_full = s_full + NQ;      // NQ
  uint64_t* pv_full = p_full + NQ;     // NQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_full + NQ);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest CTAs (last query rows of a causal mask) first; neighbouring CTAs are heads of one key/value group
  const int n_qblk = p.S / (NQ * TQ);
  const int h = blockIdx.x % p.H;
  const int b = (blockIdx.x / p.H) % p.B;
  const int qi = n_qblk - 1 - blockIdx.x / (p.H * p.B);
  const int hkv = h / (p.H / p.Hkv);
  const int q_row0 = b * p.S + qi * NQ * TQ;  // row of the [B*S, H*128] matrix
  const int kv_row0 = b * p.Sk;
  int n_it[NQ];
#pragma unroll
  for (int t = 0; t < NQ; ++t) n_it[t] = p.causal ? (NQ * qi + 1 + t) : p.Sk / TK;
  const int n_max = n_it[NQ - 1];

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < NQ; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&pv_full[t], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&](uint32_t code) {
    atomicCAS(p.status, 0u, code);
    *abort_flag = 1;
  };

  if (warp < 4) {
  regs_shrink();  // (each role's code sits behind its own register setting, so the compiler knows its budget)
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, NQ * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < NQ; ++t)
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
          tma_load_2d(smem + OFF_Q + t * TILE_BYTES + kb * HALF_BYTES, &tmQ, q_full, h * HD + kb * 64, q_row0 + t * TQ);
      for (int i = 0; i < 2 * n_max; ++i) {
        const int slot = i % RING;
        if (!mbar_wait(&kv_empty[slot], ((i / RING) & 1) ^ 1, abort_flag)) {
          fail(ST_ATTN_KV_EMPTY);
          break;
        }
        const CUtensorMap* tm = (i & 1) ? &tmV : &tmK;
        uint8_t* dst = smem + OFF_RING + slot * TILE_BYTES;
        mbar_expect_tx(&kv_full[slot], TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
          tma_load_2d(dst + kb * HALF_BYTES, tm, &kv_full[slot], hkv * HD + kb * 64, kv_row0 + (i >> 1) * TK);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(TQ, TK, 0u, 0u);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TQ, HD, 0u, 1u);
      bool ok = true;
      auto wait_kv = [&](int i) {
        if (!mbar_wait(&kv_full[i % RING], (i / RING) & 1, abort_flag)) {
          fail(ST_ATTN_KV_FULL);
          ok = false;
        }
        tc_fence_after();
      };
      // S_t = Q_t K^T: K runs over the 128 head-dim elements, two 64-element halves of four MMA steps each
      auto issue_qk = [&](int t, int slot) {
        const uint32_t q_addr = smem_u32(smem + OFF_Q + t * TILE_BYTES);
        const uint32_t k_addr = smem_u32(smem + OFF_RING + slot * TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + t * TK, make_smem_desc(q_addr + kb * HALF_BYTES + k * 32, 16, 1024),
                     make_smem_desc(k_addr + kb * HALF_BYTES + k * 32, 16, 1024), idesc_qk, (kb | k) ? 1u : 0u);
        umma_commit(&s_full[t]);
      };
      // PV_t = P_t V: K runs over the 128 keys (rows of V, 16 per step); V's two 64-column halves are HALF_BYTES apart
      auto issue_pv = [&](int t, int slot) {
        const uint32_t p_addr = smem_u32(smem + OFF_P + t * TILE_BYTES);
        const uint32_t v_addr = smem_u32(smem + OFF_RING + slot * TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + NQ * TK + t * HD, make_smem_desc(p_addr + kb * HALF_BYTES + k * 32, 16, 1024),
                     make_smem_desc(v_addr + (kb * 4 + k) * (16 * 128), HALF_BYTES, 1024), idesc_pv, (kb | k) ? 1u : 0u);
        umma_commit(&pv_full[t]);
      };
      if (!mbar_wait(q_full, 0, abort_flag)) {
        fail(ST_ATTN_KV_FULL);
        ok = false;
      }
      if (ok) wait_kv(0);
      if (ok) {
#pragma unroll
        for (int t = 0; t < NQ; ++t) issue_qk(t, 0);
        umma_commit(&kv_empty[0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        const bool more = j + 1 < n_max;
        wait_kv(iv);
        if (ok && more) wait_kv(ik);
        if (!ok) break;
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
          if (j >= n_it[t]) continue;
          // P_t(j) is in shared memory; its threads have also finished reading S_t(j) and PV_t(j-1)
          if (!mbar_wait(&p_full[t], j & 1, abort_flag)) {
            fail(ST_ATTN_ACC_EMPTY);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_pv(t, iv % RING);
          if (j + 1 < n_it[t]) issue_qk(t, ik % RING);
        }
        if (!ok) break;
        umma_commit(&kv_empty[iv % RING]);
        if (more) umma_commit(&kv_empty[ik % RING]);
      }
    }
  }
  } else {
    regs_grow();
    // ------------------------------------------------------------------ softmax + output (warps 4..11)
    const int t = (warp - 4) >> 2;        // query tile of this warp
    const int quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int r = quarter * 32 + lane;    // row of the tile owned by this thread
    const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint32_t s_addr = lane_base + t * TK;
    const uint32_t pv_addr = lane_base + NQ * TK + t * HD;
    uint8_t* p_row = smem + OFF_P + t * TILE_BYTES + r * 128;
    const int n_mine = n_it[t];
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < n_mine; ++j) {
      // (the TMEM loads below are warp-wide instructions: the warp leaves together or not at all)
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, abort_flag))) {
        fail(ST_ATTN_ACC_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      // keys of this tile that the row may see: all of them, except on the tile that holds the diagonal
      const int visible = (p.causal && j == n_mine - 1) ? r + 1 : TK;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < TK / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i < visible) mx = fmaxf(mx, __uint_as_float(v[i]));
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float alpha = fast_exp2(m_run - m_new);  // 0 on the first tile (m_run = -inf)
      // the product of the previous iteration joins the running sum before the frame moves to m_new
      if (j > 0) {
        if (!__all_sync(0xffffffffu, mbar_wait(&pv_full[t], (j - 1) & 1, abort_flag))) {
          fail(ST_ATTN_ACC_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(pv_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(v[i])) * alpha;
        }
      }
      l_run *= alpha;
      m_run = m_new;
      // pass 2: probabilities (bf16) into the swizzled K-major tile that the P V product reads
#pragma unroll
      for (int c = 0; c < TK / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c * 32, v);
        tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float x = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_new));
          e[i] = (c * 32 + i < visible) ? x : 0.f;
          l_run += e[i];
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // four 16-byte chunks of eight probabilities
          const int ch = c * 4 + g;     // chunk 0..15 of the 128-key row
          uint4 w;
          w.x = pack_bf16(e[g * 8 + 0], e[g * 8 + 1]);
          w.y = pack_bf16(e[g * 8 + 2], e[g * 8 + 3]);
          w.z = pack_bf16(e[g * 8 + 4], e[g * 8 + 5]);
          w.w = pack_bf16(e[g * 8 + 6], e[g * 8 + 7]);
          // 128-byte swizzle: the 16-byte unit index is XORed with the row index modulo 8
          *reinterpret_cast<uint4*>(p_row + (ch >> 3) * HALF_BYTES + (((ch & 7) ^ (r & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();  // the tensor core reads shared memory through the async proxy
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }

    if (ok) {  // (``ok`` is uniform across the warp: every exit above is taken by the whole warp)
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_full[t], (n_mine - 1) & 1, abort_flag))) {
        fail(ST_ATTN_ACC_FULL);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_run;
      const long long row = (long long)q_row0 + t * TQ + r;
      __nv_bfloat16* dst = p.out + row * ((long long)p.H * HD) + h * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(pv_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = (o[c * 32 + g * 8 + i] + __uint_as_float(v[g * 8 + i])) * inv;
          uint4 w;
          w.x = pack_bf16(f[0], f[1]);
          w.y = pack_bf16(f[2], f[3]);
          w.z = pack_bf16(f[4], f[5]);
          w.w = pack_bf16(f[6], f[7]);
          *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = w;
        }
      }
      // natural-log sum of exponentials of the scaled scores
      p.lse[((long long)b * p.H + h) * p.S + (qi * NQ * TQ + t * TQ + r)] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace apb_attn

// Returns 0 on launch, 3 for shapes this kernel does not cover (the caller then uses another path), other
// values for tensor-map or launch errors.
extern "C" int apb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Sk,
                                 int H, int Hkv, int D, int causal, float scale, uint32_t* status, cudaStream_t stream) {
  using namespace apb_attn;
  if (D != HD || B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0) return 3;
  if (S <= 0 || S % (NQ * TQ) != 0 || Sk <= 0 || Sk % TK != 0 || (causal && S != Sk)) return 3;
  if ((long long)B * S >= (1ll << 31) || (long long)B * Sk >= (1ll << 31)) return 3;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return 3;
  CUtensorMap tmQ, tmK, tmV;
  int e = apb::make_map(&tmQ, q, (uint64_t)H * HD, (uint64_t)B * S, (uint64_t)H * HD, TQ);
  if (!e) e = apb::make_map(&tmK, k, (uint64_t)Hkv * HD, (uint64_t)B * Sk, (uint64_t)Hkv * HD, TK);
  if (!e) e = apb::make_map(&tmV, v, (uint64_t)Hkv * HD, (uint64_t)B * Sk, (uint64_t)Hkv * HD, TK);
  if (e) return 10 + e;
  AttnParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = B;
  p.S = S;
  p.Sk = Sk;
  p.H = H;
  p.Hkv = Hkv;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  // (the attribute belongs to the current device's instance of the kernel: set on every launch, so a second device of
  // the same process is configured too)
  if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATTN_SMEM_BYTES) != cudaSuccess)
    return 20;
  const long long ctas = (long long)(S / (NQ * TQ)) * H * B;
  if (ctas >= (1ll << 31)) return 3;
  attn_fwd_kernel<<<(unsigned)ctas, ATTN_THREADS, ATTN_SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 21;
}
