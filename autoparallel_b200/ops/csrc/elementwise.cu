// Bandwidth-bound kernels of the transformer step for sm_100a: RMSNorm fwd/bwd, RoPE, SwiGLU
// fwd/bwd, cross-entropy fwd/bwd, dtype cast, embedding backward, multi-tensor AdamW.
// All use 16-byte vector accesses, fp32 math, and grids sized as multiples of the 148 SMs.
// They replace the ATen / Inductor-generated kernels the reference reaches for the same nodes
// (autoparallel/_testing/models/llama3.py:187-213, 355-356, 396-397).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace apb {

template <typename T> struct Vec8;  // 8 elements
template <> struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ void to_float(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  __device__ void from_float(const float (&f)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <> struct Vec8<float> {
  float4 a, b;
  __device__ void load(const float* p) {
    a = reinterpret_cast<const float4*>(p)[0];
    b = reinterpret_cast<const float4*>(p)[1];
  }
  __device__ void store(float* p) const {
    reinterpret_cast<float4*>(p)[0] = a;
    reinterpret_cast<float4*>(p)[1] = b;
  }
  __device__ void to_float(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  __device__ void from_float(const float (&f)[8]) {
    a = make_float4(f[0], f[1], f[2], f[3]);
    b = make_float4(f[4], f[5], f[6], f[7]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; ``red`` is >= 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < nw) ? red[l] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < nw) ? red[l] : -INFINITY;
  return warp_max(r);
}

// ------------------------------------------------------------------------------------ RMSNorm
// Forward.  A group of ``TPR`` threads owns a row and keeps its NVEC x 8 elements per thread in registers between the
// sum of squares and the scaling, so x is read once.  TPR = 32: one warp per row, reduction by shuffles only, no
// block barrier; several rows per block keep enough loads in flight.  TPR = blockDim.x: one block per row for wide rows.
// D % 8 == 0 and D <= TPR * 8 * NVEC.
template <typename T, int NVEC, bool WARP_ROWS>
__global__ void rms_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                    float* __restrict__ rstd, long long rows, int D, float eps) {
  __shared__ float red[32];
  const int tpr = WARP_ROWS ? 32 : blockDim.x;
  const int t = WARP_ROWS ? (threadIdx.x & 31) : threadIdx.x;
  const long long rows_per_block = WARP_ROWS ? (blockDim.x >> 5) : 1;
  const long long first = (long long)blockIdx.x * rows_per_block + (WARP_ROWS ? (threadIdx.x >> 5) : 0);
  const long long step = (long long)gridDim.x * rows_per_block;
  for (long long row = first; WARP_ROWS ? (row < rows) : (row - (WARP_ROWS ? (threadIdx.x >> 5) : 0) < rows); row += step) {
    if (!WARP_ROWS && row >= rows) break;
    const T* xr = x + row * D;
    T* yr = y + row * D;
    Vec8<T> v[NVEC];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      const int c = (t + j * tpr) * 8;
      if (c < D) {
        v[j].load(xr + c);
        float f[8]; v[j].to_float(f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
    }
    ss = WARP_ROWS ? warp_sum(ss) : block_sum(ss, red);
    const float r = rsqrtf(ss / D + eps);
    if (t == 0) rstd[row] = r;
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      const int c = (t + j * tpr) * 8;
      if (c < D) {
        Vec8<T> wv; wv.load(w + c);
        float f[8], g[8]; v[j].to_float(f); wv.to_float(g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
        Vec8<T> o; o.from_float(f); o.store(yr + c);
      }
    }
  }
}

// block-wide sums of R values at once (one barrier pair for all of them); ``red`` holds 32 * R floats
template <int R>
__device__ __forceinline__ void block_sum_multi(float (&v)[R], float* red) {
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int k = 0; k < R; ++k) v[k] = warp_sum(v[k]);
  __syncthreads();
  if (l == 0) {
#pragma unroll
    for (int k = 0; k < R; ++k) red[k * 32 + w] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < R; ++k) v[k] = warp_sum(l < nw ? red[k * 32 + l] : 0.f);
}

// Backward.  One persistent block per SM (a single wave).  Every iteration takes ROWS rows at once and the loads of
// the next iteration are issued before the current one is reduced and stored (two register sets that swap roles, so
// nothing is copied): the row loop is bound by memory bandwidth rather than by one load-reduce-store round trip per
// row.  The ROWS dot products share one block reduction.  Math per element: g*x once, then two fused multiply-adds
// (weight-gradient partial and dot product); the second pass forms dx = g*(r*w) - x*(r*r*mean) with two more.
// EXACT: D == blockDim.x * 8 * NVEC and rows % ROWS == 0, so no bounds predicate is needed anywhere.
// dw partial sums per thread-owned columns are added into ``dw_acc`` (fp32 [D], zeroed by the caller) with one
// atomicAdd per column per block.  Requires D <= blockDim.x * 8 * RMS_BWD_MAX_VEC.
constexpr int RMS_BWD_MAX_VEC = 4;
template <typename T, int NVEC, int ROWS, bool EXACT>
__global__ void __launch_bounds__(512) rms_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                                           const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_acc,
                                                           long long rows, int D) {
  __shared__ float red[32 * ROWS];
  float wreg[NVEC][8];
  float dwreg[NVEC][8];
  int col[NVEC];
#pragma unroll
  for (int j = 0; j < NVEC; ++j) {
    col[j] = (threadIdx.x + j * blockDim.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dwreg[j][i] = 0.f;
      wreg[j][i] = 0.f;
    }
    if (EXACT || col[j] < D) {
      Vec8<T> wv; wv.load(w + col[j]); wv.to_float(wreg[j]);
    }
  }
  const long long step = (long long)gridDim.x * ROWS;
  const float inv_d = 1.f / D;
  Vec8<T> xa[ROWS][NVEC], ga[ROWS][NVEC], xb[ROWS][NVEC], gb[ROWS][NVEC];
  float ra[ROWS], rb[ROWS];

  auto fetch = [&](Vec8<T> (&xs)[ROWS][NVEC], Vec8<T> (&gs)[ROWS][NVEC], float (&rs)[ROWS], long long row0) {
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const long long row = row0 + k;
      const bool row_ok = EXACT || row < rows;
      rs[k] = row_ok ? rstd[row] : 0.f;
      const T* xr = x + row * D;
      const T* gr = dy + row * D;
#pragma unroll
      for (int j = 0; j < NVEC; ++j) {
        if (row_ok && (EXACT || col[j] < D)) {
          xs[k][j].load(xr + col[j]);
          gs[k][j].load(gr + col[j]);
        }
      }
    }
  };
  auto process = [&](Vec8<T> (&xs)[ROWS][NVEC], Vec8<T> (&gs)[ROWS][NVEC], float (&rs)[ROWS], long long row0) {
    float dot[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      dot[k] = 0.f;
      const bool row_ok = EXACT || row0 + k < rows;
#pragma unroll
      for (int j = 0; j < NVEC; ++j) {
        if (row_ok && (EXACT || col[j] < D)) {
          float xf[8], gf[8]; xs[k][j].to_float(xf); gs[k][j].to_float(gf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float gx = gf[i] * xf[i];
            dwreg[j][i] = fmaf(gx, rs[k], dwreg[j][i]);
            dot[k] = fmaf(gx, wreg[j][i], dot[k]);
          }
        }
      }
    }
    block_sum_multi<ROWS>(dot, red);
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const long long row = row0 + k;
      const bool row_ok = EXACT || row < rows;
      const float r = rs[k];
      const float c = r * r * r * dot[k] * inv_d;  // (sum g w x) * r is the dot product with x-hat; times r*r for the formula below
      T* dr = dx + row * D;
#pragma unroll
      for (int j = 0; j < NVEC; ++j) {
        if (row_ok && (EXACT || col[j] < D)) {
          float xf[8], gf[8], o[8]; xs[k][j].to_float(xf); gs[k][j].to_float(gf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = fmaf(gf[i], r * wreg[j][i], -xf[i] * c);
          Vec8<T> ov; ov.from_float(o); ov.store(dr + col[j]);
        }
      }
    }
  };

  long long row0 = (long long)blockIdx.x * ROWS;
  if (row0 < rows) fetch(xa, ga, ra, row0);
  while (row0 < rows) {
    if (row0 + step < rows) fetch(xb, gb, rb, row0 + step);
    process(xa, ga, ra, row0);
    row0 += step;
    if (row0 >= rows) break;
    if (row0 + step < rows) fetch(xa, ga, ra, row0 + step);
    process(xb, gb, rb, row0);
    row0 += step;
  }
#pragma unroll
  for (int j = 0; j < NVEC; ++j) {
    if (EXACT || col[j] < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(dw_acc + col[j] + i, dwreg[j][i]);
    }
  }
}

// Backward, bulk-copy form (the one the launcher prefers).  The rows of x and dy travel global -> shared memory as
// untiled bulk copies (``cp.async.bulk``, completion on an mbarrier) through a ring of RMS_STAGES stages of ROWS rows,
// issued two stages ahead by one thread, so the prefetch costs no registers and the copy engine keeps the memory
// system busy while the block reduces and stores the current rows.  Each thread reads its 16-byte column groups from
// shared memory twice (dot product / weight-gradient pass, then the dx pass) instead of holding them in registers.
// One block per SM; waits are bounded: if a stage never arrives the block stops (its rows keep whatever dx held).
constexpr int RMS_STAGES = 3;
template <typename T, int NVEC, int ROWS>
__global__ void __launch_bounds__(512) rms_norm_bwd_bulk_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                                                const float* __restrict__ rstd, T* __restrict__ dx,
                                                                float* __restrict__ dw_acc, long long rows, int D) {
  extern __shared__ uint8_t rms_smem_raw[];
  __shared__ uint32_t abort_word;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(rms_smem_raw) + 127) & ~uintptr_t(127));
  const int row_bytes = D * (int)sizeof(T);
  const int stage_bytes = ROWS * row_bytes;  // per tensor
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RMS_STAGES * 2 * stage_bytes);
  float* red = reinterpret_cast<float*>(bars + RMS_STAGES);
  volatile uint32_t* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    for (int s_ = 0; s_ < RMS_STAGES; ++s_) mbar_init(&bars[s_], 1);
    abort_word = 0;
    mbar_fence_init();
  }
  __syncthreads();

  float wreg[NVEC][8], dwreg[NVEC][8];
  int col[NVEC];
#pragma unroll
  for (int j = 0; j < NVEC; ++j) {
    col[j] = (threadIdx.x + j * blockDim.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dwreg[j][i] = 0.f;
      wreg[j][i] = 0.f;
    }
    if (col[j] < D) {
      Vec8<T> wv; wv.load(w + col[j]); wv.to_float(wreg[j]);
    }
  }
  const float inv_d = 1.f / D;
  const long long step = (long long)gridDim.x * ROWS;
  const long long first = (long long)blockIdx.x * ROWS;
  auto issue = [&](long long it) {  // one thread: start the copies of this block's iteration ``it``
    const long long row0 = first + it * step;
    if (row0 >= rows) return;
    const int st = (int)(it % RMS_STAGES);
    const long long nrows = rows - row0 < ROWS ? rows - row0 : ROWS;
    const uint32_t bytes = (uint32_t)(nrows * row_bytes);
    mbar_expect_tx(&bars[st], 2u * bytes);
    bulk_load(smem + (2 * st) * stage_bytes, x + row0 * D, bytes, &bars[st]);
    bulk_load(smem + (2 * st + 1) * stage_bytes, dy + row0 * D, bytes, &bars[st]);
  };
  if (threadIdx.x == 0)
    for (int it = 0; it < RMS_STAGES - 1; ++it) issue(it);

  long long it = 0;
  for (long long row0 = first; row0 < rows; row0 += step, ++it) {
    if (threadIdx.x == 0) issue(it + RMS_STAGES - 1);  // refills the stage every thread left at the end of the last iteration
    const int st = (int)(it % RMS_STAGES);
    if (!mbar_wait(&bars[st], (uint32_t)((it / RMS_STAGES) & 1), abort_flag)) {
      *abort_flag = 1;
      break;
    }
    const uint8_t* xs = smem + (2 * st) * stage_bytes;
    const uint8_t* gs = xs + stage_bytes;
    float dot[ROWS], r[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      dot[k] = 0.f;
      const bool row_ok = row0 + k < rows;
      r[k] = row_ok ? rstd[row0 + k] : 0.f;
#pragma unroll
      for (int j = 0; j < NVEC; ++j) {
        if (row_ok && col[j] < D) {
          Vec8<T> xv, gv;
          xv.load(reinterpret_cast<const T*>(xs + k * row_bytes) + col[j]);
          gv.load(reinterpret_cast<const T*>(gs + k * row_bytes) + col[j]);
          float xf[8], gf[8]; xv.to_float(xf); gv.to_float(gf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float gx = gf[i] * xf[i];
            dwreg[j][i] = fmaf(gx, r[k], dwreg[j][i]);
            dot[k] = fmaf(gx, wreg[j][i], dot[k]);
          }
        }
      }
    }
    block_sum_multi<ROWS>(dot, red);
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const long long row = row0 + k;
      const float c = r[k] * r[k] * r[k] * dot[k] * inv_d;
      if (row < rows) {
#pragma unroll
        for (int j = 0; j < NVEC; ++j) {
          if (col[j] < D) {
            Vec8<T> xv, gv;
            xv.load(reinterpret_cast<const T*>(xs + k * row_bytes) + col[j]);
            gv.load(reinterpret_cast<const T*>(gs + k * row_bytes) + col[j]);
            float xf[8], gf[8], o[8]; xv.to_float(xf); gv.to_float(gf);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = fmaf(gf[i], r[k] * wreg[j][i], -xf[i] * c);
            Vec8<T> ov; ov.from_float(o); ov.store(dx + row * D + col[j]);
          }
        }
      }
    }
    __syncthreads();  // every thread has read this stage for the last time: it may be refilled
  }
#pragma unroll
  for (int j = 0; j < NVEC; ++j) {
    if (col[j] < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(dw_acc + col[j] + i, dwreg[j][i]);
    }
  }
}

template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    Vec8<float> v; v.load(src + i);
    float f[8]; v.to_float(f);
    Vec8<T> o; o.from_float(f); o.store(dst + i);
  }
  if (i < n && i + 8 > n)
    for (long long k = i; k < n; ++k) dst[k] = T(src[k]);
}
template <typename T>
__global__ void cast_to_f32_kernel(const T* __restrict__ src, float* __restrict__ dst, long long n) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    Vec8<T> v; v.load(src + i);
    float f[8]; v.to_float(f);
    Vec8<float> o; o.from_float(f); o.store(dst + i);
  }
  if (i < n && i + 8 > n)
    for (long long k = i; k < n; ++k) dst[k] = float(src[k]);
}

// ------------------------------------------------------------------------------------ RoPE
// x [B, S, H, D] with interleaved pairs; cos/sin fp32 [S, D/2].  One thread owns eight consecutive elements of a
// head (one 16-byte vector) at one position and walks over the heads: the 32 bytes of cos / sin it needs are read
// once per position instead of once per head (the tables would otherwise be twice the traffic of x itself).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            T* __restrict__ y, long long total_pos_vec, int S, int H, int D, float sign) {
  const int vec_per_head = D / 8;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total_pos_vec;
       v += (long long)gridDim.x * blockDim.x) {
    const int dv = v % vec_per_head;
    const long long bs = v / vec_per_head;  // b * S + s
    const int s = bs % S;
    const float4 c = *reinterpret_cast<const float4*>(cs + (long long)s * (D / 2) + dv * 4);
    const float4 n = *reinterpret_cast<const float4*>(sn + (long long)s * (D / 2) + dv * 4);
    const float cc[4] = {c.x, c.y, c.z, c.w};
    const float nn[4] = {n.x * sign, n.y * sign, n.z * sign, n.w * sign};
    const long long base = (bs * H) * D + dv * 8;
    int h = 0;
    for (; h + 4 <= H; h += 4) {  // four independent loads in flight
      Vec8<T> xv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) xv[k].load(x + base + (long long)(h + k) * D);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[8], o[8];
        xv[k].to_float(f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          o[2 * i] = f[2 * i] * cc[i] - f[2 * i + 1] * nn[i];
          o[2 * i + 1] = f[2 * i] * nn[i] + f[2 * i + 1] * cc[i];
        }
        Vec8<T> ov; ov.from_float(o); ov.store(y + base + (long long)(h + k) * D);
      }
    }
    for (; h < H; ++h) {
      Vec8<T> xv; xv.load(x + base + (long long)h * D);
      float f[8], o[8]; xv.to_float(f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[2 * i] = f[2 * i] * cc[i] - f[2 * i + 1] * nn[i];
        o[2 * i + 1] = f[2 * i] * nn[i] + f[2 * i + 1] * cc[i];
      }
      Vec8<T> ov; ov.from_float(o); ov.store(y + base + (long long)h * D);
    }
  }
}

// ------------------------------------------------------------------------------------ SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long nvec) {
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    Vec8<T> av, bv; av.load(a + v * 8); bv.load(b + v * 8);
    float fa[8], fb[8], o[8]; av.to_float(fa); bv.to_float(fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = fa[i] / (1.f + __expf(-fa[i])) * fb[i];
    Vec8<T> ov; ov.from_float(o); ov.store(y + v * 8);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ a, const T* __restrict__ b,
                                  T* __restrict__ da, T* __restrict__ db, long long nvec) {
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    Vec8<T> gv, av, bv; gv.load(dy + v * 8); av.load(a + v * 8); bv.load(b + v * 8);
    float g[8], fa[8], fb[8], oa[8], ob[8]; gv.to_float(g); av.to_float(fa); bv.to_float(fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sig = 1.f / (1.f + __expf(-fa[i]));
      const float silu = fa[i] * sig;
      oa[i] = g[i] * fb[i] * (sig * (1.f + fa[i] * (1.f - sig)));
      ob[i] = g[i] * silu;
    }
    Vec8<T> o1, o2; o1.from_float(oa); o2.from_float(ob); o1.store(da + v * 8); o2.store(db + v * 8);
  }
}

// ------------------------------------------------------------------------------------ cross-entropy
// one block per row of V logits (V % 8 == 0): online (max, sum-exp); loss = lse - logit[label].
template <typename T>
__global__ void xent_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                float* __restrict__ loss, float* __restrict__ lse, int V) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* lr = logits + row * V;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    Vec8<T> v; v.load(lr + c);
    float f[8]; v.to_float(f);
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += __expf(f[i] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float l = gm + logf(s);
    lse[row] = l;
    loss[row] = l - float(lr[labels[row]]);
  }
}
template <typename T>
__global__ void xent_bwd_kernel(const float* __restrict__ dloss, const T* __restrict__ logits,
                                const long long* __restrict__ labels, const float* __restrict__ lse,
                                T* __restrict__ dlogits, int V) {
  const long long row = blockIdx.x;
  const T* lr = logits + row * V;
  T* dr = dlogits + row * V;
  const float l = lse[row], g = dloss[row];
  const int lab = (int)labels[row];
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    Vec8<T> v; v.load(lr + c);
    float f[8]; v.to_float(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = (__expf(f[i] - l) - ((c + i) == lab ? 1.f : 0.f)) * g;
    Vec8<T> o; o.from_float(f); o.store(dr + c);
  }
}

// ------------------------------------------------------------------------------------ embedding forward
// out[token] = weight[ids[token]]: one block per token, 16-byte vectors (D % 8 == 0 for bf16, % 4 for fp32).
template <typename T>
__global__ void embedding_fwd_kernel(const T* __restrict__ weight, const long long* __restrict__ ids, T* __restrict__ out, int D,
                                     long long num_rows) {
  const long long tok = blockIdx.x;
  long long r = ids[tok];
  r = r < 0 ? 0 : (r >= num_rows ? num_rows - 1 : r);  // (an id outside the table is the caller's bug; never read outside)
  const uint4* src = reinterpret_cast<const uint4*>(weight + r * D);
  uint4* dst = reinterpret_cast<uint4*>(out + tok * D);
  const int nvec = D * (int)sizeof(T) / 16;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) dst[c] = src[c];
}

// ------------------------------------------------------------------------------------ embedding backward
// out fp32 [rows, D] (zeroed by caller) += dy[token] for each token; one block per token.
template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dy, const long long* __restrict__ ids, float* __restrict__ out,
                                     int D) {
  const long long tok = blockIdx.x;
  const long long r = ids[tok];
  for (int c = threadIdx.x; c < D; c += blockDim.x) atomicAdd(out + r * D + c, float(dy[tok * D + c]));
}

// ------------------------------------------------------------------------------------ AdamW
// Multi-tensor: ``table`` lists chunks (tensor id, offset); each block handles one chunk.
struct AdamTensor {
  float* p;        // fp32 master / parameter
  const float* g;  // fp32 gradient
  float* m;
  float* v;
  __nv_bfloat16* p_lp;  // optional low-precision copy to emit (may be null)
  long long n;
};
constexpr int ADAM_CHUNK = 65536;
// ``hyper`` (optional, device memory): {lr, bc1, bc2} read at run time instead of the launch arguments, so that a step
// captured in a CUDA graph follows the learning-rate schedule and the bias corrections of the step it is replayed for.
__global__ void adamw_kernel(const AdamTensor* __restrict__ tensors, const int2* __restrict__ chunks, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                             const float* __restrict__ hyper) {
  if (hyper != nullptr) {
    lr = hyper[0];
    bc1 = hyper[1];
    bc2 = hyper[2];
  }
  const int2 ch = chunks[blockIdx.x];
  const AdamTensor t = tensors[ch.x];
  const long long base = (long long)ch.y * ADAM_CHUNK;
  const long long end = min(base + (long long)ADAM_CHUNK, t.n);
  for (long long i = base + threadIdx.x * 4; i < end; i += blockDim.x * 4) {
    if (i + 4 <= end && ((reinterpret_cast<uintptr_t>(t.p + i) & 15) == 0)) {
      float4 p = *reinterpret_cast<float4*>(t.p + i);
      const float4 g4 = *reinterpret_cast<const float4*>(t.g + i);
      float4 m = *reinterpret_cast<float4*>(t.m + i);
      float4 v = *reinterpret_cast<float4*>(t.v + i);
      float* pp = &p.x; const float* gg = &g4.x; float* mm = &m.x; float* vv = &v.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float g = gg[k] * grad_scale;
        mm[k] = beta1 * mm[k] + (1.f - beta1) * g;
        vv[k] = beta2 * vv[k] + (1.f - beta2) * g * g;
        const float mh = mm[k] / bc1;
        const float vh = vv[k] / bc2;
        pp[k] = pp[k] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
      }
      *reinterpret_cast<float4*>(t.p + i) = p;
      *reinterpret_cast<float4*>(t.m + i) = m;
      *reinterpret_cast<float4*>(t.v + i) = v;
      if (t.p_lp) {
        t.p_lp[i] = __float2bfloat16(p.x); t.p_lp[i + 1] = __float2bfloat16(p.y);
        t.p_lp[i + 2] = __float2bfloat16(p.z); t.p_lp[i + 3] = __float2bfloat16(p.w);
      }
    } else {
      for (long long k = i; k < min(i + 4, end); ++k) {
        const float g = t.g[k] * grad_scale;
        const float m = beta1 * t.m[k] + (1.f - beta1) * g;
        const float v = beta2 * t.v[k] + (1.f - beta2) * g * g;
        t.m[k] = m; t.v[k] = v;
        const float pn = t.p[k] * (1.f - lr * wd) - lr * (m / bc1) / (sqrtf(v / bc2) + eps);
        t.p[k] = pn;
        if (t.p_lp) t.p_lp[k] = __float2bfloat16(pn);
      }
    }
  }
}

// Launch configuration of rms_norm_bwd_kernel: as many threads as 8-element vectors in a row (up to
// 1024) so each thread keeps ONE vector per operand in registers; that keeps the register count low
// enough for several resident blocks per SM, which is what a latency-bound row loop needs.
template <typename T>
static inline int launch_rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_acc,
                                      long long rows, int D, int num_sms, cudaStream_t st) {
  int threads = 128;
  while (threads * 8 < D && threads < 512) threads *= 2;  // at most 512 threads: 128 registers each
  const int nvec = (D + threads * 8 - 1) / (threads * 8);
  if (nvec > RMS_BWD_MAX_VEC) return 3;
  // Preferred: the bulk-copy form, whenever three stages of at least one row of both tensors fit in shared memory.
  {
    const long long row_bytes = (long long)D * (long long)sizeof(T);
    int rows_per_stage = 0;
    for (int cand : {4, 2, 1})
      if (RMS_STAGES * 2 * cand * row_bytes + 1024 <= 200 * 1024) {
        rows_per_stage = cand;
        break;
      }
    if (rows_per_stage > 0 && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(dy) % 16 == 0)) {
      const int smem = (int)(RMS_STAGES * 2 * rows_per_stage * row_bytes + 128 + RMS_STAGES * 8 + 32 * rows_per_stage * 4 + 128);
      const long long iters = (rows + rows_per_stage - 1) / rows_per_stage;
      const int grid = (int)(iters < num_sms ? iters : num_sms);
#define APB_RMS_BULK(NV, RW)                                                                                                      \
  {                                                                                                                               \
    auto kern = rms_norm_bwd_bulk_kernel<T, NV, RW>;                                                                              \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 4;                   \
    kern<<<grid, threads, smem, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_acc, rows, D);                     \
    return 0;                                                                                                                     \
  }
#define APB_RMS_BULK_ROWS(NV)                                \
  {                                                          \
    if (rows_per_stage == 4) APB_RMS_BULK(NV, 4)             \
    else if (rows_per_stage == 2) APB_RMS_BULK(NV, 2)        \
    else APB_RMS_BULK(NV, 1)                                 \
  }
      if (nvec == 1) APB_RMS_BULK_ROWS(1)
      else if (nvec == 2) APB_RMS_BULK_ROWS(2)
      else APB_RMS_BULK_ROWS(4)
#undef APB_RMS_BULK_ROWS
#undef APB_RMS_BULK
    }
  }
  const int per_sm = threads >= 512 ? 1 : (threads >= 256 ? 2 : 4);  // resident blocks at 128 registers per thread: one wave
  const long long cap = (long long)num_sms * per_sm;
  // rows per iteration: as many as the registers hold (16-byte vectors for bf16, two per vector for fp32)
  constexpr bool wide = sizeof(T) == 4;
#define APB_RMS_BWD(NV, RW)                                                                                              \
  {                                                                                                                      \
    const long long iters = (rows + RW - 1) / RW;                                                                        \
    const int grid = (int)(iters < cap ? iters : cap);                                                                   \
    if (D == threads * 8 * NV && rows % RW == 0)                                                                         \
      rms_norm_bwd_kernel<T, NV, RW, true><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_acc, rows, D); \
    else                                                                                                                 \
      rms_norm_bwd_kernel<T, NV, RW, false><<<grid, threads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_acc, rows, D); \
  }
  if (nvec == 1) { if constexpr (wide) APB_RMS_BWD(1, 2) else APB_RMS_BWD(1, 4) }
  else if (nvec == 2) { if constexpr (wide) APB_RMS_BWD(2, 1) else APB_RMS_BWD(2, 2) }
  else APB_RMS_BWD(4, 1)  // (nvec 3 runs as 4 with the last vector masked)
#undef APB_RMS_BWD
  return 0;
}

static inline int grid_for(long long work_items, int threads, int num_sms) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = (long long)num_sms * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace apb

using namespace apb;
typedef __nv_bfloat16 bf16;

#define DISPATCH(is_bf16, ...)      \
  if (is_bf16) {                    \
    typedef bf16 T;                 \
    __VA_ARGS__;                    \
  } else {                          \
    typedef float T;                \
    __VA_ARGS__;                    \
  }

extern "C" {

int apb_rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int D, float eps, int is_bf16,
                     cudaStream_t st) {
  if (D % 8) return 3;
  if (rows == 0) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (D <= 32 * 8 * 4) {
    // one warp per row, eight rows per block
    const int nvec = (D + 255) / 256;
    const long long blocks = (rows + 7) / 8, cap = (long long)sms * 8;
    const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
#define APB_RMS_FWD_W(NV) DISPATCH(is_bf16, rms_norm_fwd_kernel<T, NV, true><<<grid, 256, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, rows, D, eps))
    if (nvec == 1) { APB_RMS_FWD_W(1); } else if (nvec == 2) { APB_RMS_FWD_W(2); } else { APB_RMS_FWD_W(4); }
#undef APB_RMS_FWD_W
  } else {
    int threads = 256;
    while (threads * 8 * 4 < D && threads < 1024) threads *= 2;
    const int nvec = (D + threads * 8 - 1) / (threads * 8);
    if (nvec > 4) return 3;
    const long long cap = (long long)sms * (threads >= 1024 ? 2 : (threads >= 512 ? 4 : 8));
    const unsigned grid = (unsigned)(rows < cap ? rows : cap);
#define APB_RMS_FWD_B(NV) DISPATCH(is_bf16, rms_norm_fwd_kernel<T, NV, false><<<grid, threads, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, rows, D, eps))
    if (nvec == 1) { APB_RMS_FWD_B(1); } else if (nvec == 2) { APB_RMS_FWD_B(2); } else { APB_RMS_FWD_B(4); }
#undef APB_RMS_FWD_B
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// dw_acc: fp32 [D] scratch, zeroed here; dw receives the cast result.
int apb_rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw, float* dw_acc,
                     long long rows, int D, int is_bf16, int num_sms, cudaStream_t st) {
  if (D % 8) return 3;
  if (D > 512 * 8 * RMS_BWD_MAX_VEC) return 3;
  cudaMemsetAsync(dw_acc, 0, sizeof(float) * D, st);
  if (rows > 0) {
    int e;
    DISPATCH(is_bf16, e = launch_rms_norm_bwd<T>(dy, x, w, rstd, dx, dw_acc, rows, D, num_sms, st));
    if (e) return e;
  }
  if (is_bf16) cast_from_f32_kernel<bf16><<<grid_for(D / 8, 256, num_sms), 256, 0, st>>>(dw_acc, (bf16*)dw, D);
  else cudaMemcpyAsync(dw, dw_acc, sizeof(float) * D, cudaMemcpyDeviceToDevice, st);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_cast(const void* src, void* dst, long long n, int src_bf16, int dst_bf16, int num_sms, cudaStream_t st) {
  if (n == 0) return 0;
  const int grid = grid_for((n + 7) / 8, 256, num_sms);
  if (src_bf16 && !dst_bf16) cast_to_f32_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)src, (float*)dst, n);
  else if (!src_bf16 && dst_bf16) cast_from_f32_kernel<bf16><<<grid, 256, 0, st>>>((const float*)src, (bf16*)dst, n);
  else return 3;
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_rope(const void* x, const float* cs, const float* sn, void* y, long long B, int S, int H, int D, int conj,
             int is_bf16, int num_sms, cudaStream_t st) {
  if (D % 8) return 3;
  const long long nvec = B * S * (D / 8);  // one thread per (position, 8-element group); the kernel walks the heads
  if (nvec == 0 || H == 0) return 0;
  const int grid = grid_for(nvec, 128, num_sms);
  DISPATCH(is_bf16, rope_kernel<T><<<grid, 128, 0, st>>>((const T*)x, cs, sn, (T*)y, nvec, S, H, D, conj ? -1.f : 1.f));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_swiglu_fwd(const void* a, const void* b, void* y, long long n, int is_bf16, int num_sms, cudaStream_t st) {
  if (n % 8) return 3;
  if (n == 0) return 0;
  DISPATCH(is_bf16, swiglu_fwd_kernel<T><<<grid_for(n / 8, 256, num_sms), 256, 0, st>>>((const T*)a, (const T*)b, (T*)y, n / 8));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_swiglu_bwd(const void* dy, const void* a, const void* b, void* da, void* db, long long n, int is_bf16, int num_sms,
                   cudaStream_t st) {
  if (n % 8) return 3;
  if (n == 0) return 0;
  DISPATCH(is_bf16, swiglu_bwd_kernel<T><<<grid_for(n / 8, 256, num_sms), 256, 0, st>>>((const T*)dy, (const T*)a, (const T*)b,
                                                                                       (T*)da, (T*)db, n / 8));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_xent_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long rows, int V, int is_bf16,
                 cudaStream_t st) {
  if (V % 8) return 3;
  if (rows == 0) return 0;
  const int threads = V >= 8192 ? 1024 : 256;
  DISPATCH(is_bf16, xent_fwd_kernel<T><<<(unsigned)rows, threads, 0, st>>>((const T*)logits, labels, loss, lse, V));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_xent_bwd(const float* dloss, const void* logits, const long long* labels, const float* lse, void* dlogits,
                 long long rows, int V, int is_bf16, cudaStream_t st) {
  if (V % 8) return 3;
  if (rows == 0) return 0;
  const int threads = V >= 8192 ? 1024 : 256;
  DISPATCH(is_bf16, xent_bwd_kernel<T><<<(unsigned)rows, threads, 0, st>>>(dloss, (const T*)logits, labels, lse, (T*)dlogits, V));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_embedding_fwd(const void* weight, const long long* ids, void* out, long long tokens, int D, long long num_rows,
                      int is_bf16, cudaStream_t st) {
  if (tokens == 0) return 0;
  if ((D * (is_bf16 ? 2 : 4)) % 16) return 3;
  DISPATCH(is_bf16, embedding_fwd_kernel<T><<<(unsigned)tokens, 128, 0, st>>>((const T*)weight, ids, (T*)out, D, num_rows));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_embedding_bwd(const void* dy, const long long* ids, float* out_f32, long long tokens, int D, int is_bf16,
                      cudaStream_t st) {
  if (tokens == 0) return 0;
  DISPATCH(is_bf16, embedding_bwd_kernel<T><<<(unsigned)tokens, 256, 0, st>>>((const T*)dy, ids, out_f32, D));
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

int apb_adamw(const void* tensors_dev, const void* chunks_dev, int num_chunks, float lr, float beta1, float beta2, float eps,
              float wd, float bc1, float bc2, float grad_scale, const float* hyper_dev, cudaStream_t st) {
  if (num_chunks == 0) return 0;
  adamw_kernel<<<num_chunks, 256, 0, st>>>((const AdamTensor*)tensors_dev, (const int2*)chunks_dev, lr, beta1, beta2, eps, wd,
                                           bc1, bc2, grad_scale, hyper_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (see apb_noalloc.h for the contract).
// ------------------------------------------------------------------------------------------------
#include <atomic>
#include <mutex>

#include "apb_noalloc.h"

// The weight-gradient accumulator.  In host code this name is only a handle for the runtime's
// symbol table, never a pointer a kernel could use: its device address is fetched once per device
// with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_dw_acc[APB_NOALLOC_MAX_D];

namespace {
constexpr int kMaxDevices = 64;
// The pointer is published with a release store after the SM count has been written, and read with
// an acquire load: a thread that sees the pointer also sees the count, without taking the mutex.
std::atomic<float*> g_noalloc_ptr[kMaxDevices] = {};
int g_noalloc_sms[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// One-time per-device set-up; the caller's current device is the one being set up.
int noalloc_setup(int dev) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev].load(std::memory_order_acquire) != nullptr) return APB_NOALLOC_OK;
  float* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dw_acc) != cudaSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return APB_NOALLOC_ERR_SETUP;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
    (void)cudaGetLastError();
    return APB_NOALLOC_ERR_SETUP;
  }
  g_noalloc_sms[dev] = sms;
  g_noalloc_ptr[dev].store(p, std::memory_order_release);
  return APB_NOALLOC_OK;
}
}  // namespace

extern "C" int apb_rms_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                                        long long rows, int D, int is_bf16, cudaStream_t st) {
  if (D <= 0 || rows < 0 || (D % 8) != 0) return APB_NOALLOC_ERR_BAD_SHAPE;
  if (D > APB_NOALLOC_MAX_D) return APB_NOALLOC_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return APB_NOALLOC_ERR_SETUP;
  float* acc = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (acc == nullptr) {
    const int e = noalloc_setup(dev);
    if (e != APB_NOALLOC_OK) return e;
    acc = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  }
  const int num_sms = g_noalloc_sms[dev];
  // the array keeps the previous call's sums: start from zero
  if (cudaMemsetAsync(acc, 0, sizeof(float) * D, st) != cudaSuccess) return APB_NOALLOC_ERR_LAUNCH;
  if (rows > 0) {
    int e;
    DISPATCH(is_bf16, e = launch_rms_norm_bwd<T>(dy, x, w, rstd, dx, acc, rows, D, num_sms, st));
    if (e) return APB_NOALLOC_ERR_BAD_SHAPE;
  }
  if (is_bf16) {
    cast_from_f32_kernel<bf16><<<grid_for(D / 8, 256, num_sms), 256, 0, st>>>(acc, (bf16*)dw, D);
  } else {
    if (cudaMemcpyAsync(dw, acc, sizeof(float) * D, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return APB_NOALLOC_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? APB_NOALLOC_OK : APB_NOALLOC_ERR_LAUNCH;
}

extern "C" const char* apb_noalloc_strerror(int code) {
  switch (code) {
    case APB_NOALLOC_OK: return "ok";
    case APB_NOALLOC_ERR_BAD_SHAPE: return "bad shape: D must be a positive multiple of 8 and rows >= 0";
    case APB_NOALLOC_ERR_LAUNCH: return "CUDA launch failed";
    case APB_NOALLOC_ERR_TOO_LARGE: return "D exceeds APB_NOALLOC_MAX_D (16384): the built-in scratch array is too small";
    case APB_NOALLOC_ERR_SETUP: return "could not obtain the device address of the built-in scratch array";
    default: return "unknown error code";
  }
}
