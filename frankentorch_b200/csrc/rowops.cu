// Row-wise kernels: LayerNorm / RMSNorm forward+backward, softmax, fused
// softmax-cross-entropy, fixed-tree reductions.  All memory bound: one pass over
// the data where it fits on chip, 16-byte vector accesses, fp32 statistics.
//
// Semantics follow the reference CPU kernels: two-pass LayerNorm with population
// variance (ft-kernel-cpu/src/lib.rs:5824), RMSNorm (:6418, backward :6503),
// cross-entropy = lse - logit[target] with gradient softmax - onehot (:6649,:6679),
// guarded row softmax of the Metal shader (ft-kernel-metal/src/fused.rs:321).
// Parameter-gradient reductions run in a fixed order (row blocks, then a serial
// pass over the block partials), so two runs give identical bits.
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

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
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  return u;
}

constexpr int ROW_WARPS = 8;     // rows per CTA
constexpr int ROW_CACHE = 8;     // 8 x (32 lanes x 8 elems) = 2048 columns kept in registers

// ----------------------------------------------------------------------------- LayerNorm fwd
constexpr int NF_CACHE = 4;      // forward: 4 x (32 lanes x 8 elems) = 1024 columns kept in registers
template <bool RMS>
__global__ void __launch_bounds__(ROW_WARPS * 32, 4)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ resid,
                __nv_bfloat16* __restrict__ sum_out, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int cols,
                float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ROW_WARPS + warp;
  if (row >= rows) return;
  const int nvec = cols >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
  const uint4* rr = resid ? reinterpret_cast<const uint4*>(resid + (size_t)row * cols) : nullptr;
  uint4* so = sum_out ? reinterpret_cast<uint4*>(sum_out + (size_t)row * cols) : nullptr;
  // The first NF_CACHE vectors of a lane (1024 columns) live in registers: every loop over
  // them is fully unrolled so the array never spills to local memory, and all loads of the row
  // are issued before any arithmetic (a lane that loads and reduces one vector at a time sits at
  // memory latency).  Columns beyond the cache are re-read.  Sums run in ascending vector order
  // in both parts, so results do not depend on the split.
  uint4 cache[NF_CACHE];
  uint4 rcache[NF_CACHE];
#pragma unroll
  for (int c = 0; c < NF_CACHE; ++c) {
    const int v = lane + 32 * c;
    if (v < nvec) {
      cache[c] = xr[v];
      if (rr) rcache[c] = rr[v];
    }
  }
  float s = 0.f;
  auto first_pass = [&](uint4 u, const uint4& r, int v) -> uint4 {
    float f[8];
    unpack8(u, f);
    if (rr) {
      float g[8];
      unpack8(r, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      u = pack8(f);
      unpack8(u, f);  // statistics are taken on the rounded sum that downstream kernels will read
      if (so) so[v] = u;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += RMS ? f[i] * f[i] : f[i];
    return u;
  };
#pragma unroll
  for (int c = 0; c < NF_CACHE; ++c) {
    const int v = lane + 32 * c;
    if (v < nvec) cache[c] = first_pass(cache[c], rcache[c], v);
  }
  for (int v = lane + 32 * NF_CACHE; v < nvec; v += 32)
    first_pass(xr[v], rr ? rr[v] : make_uint4(0u, 0u, 0u, 0u), v);
  s = warp_sum(s);
  float mean = 0.f, rstd;
  const uint4* src = rr ? reinterpret_cast<const uint4*>(so) : xr;
  if (RMS) {
    rstd = rsqrtf(s / cols + eps);
  } else {
    mean = s / cols;
    float q = 0.f;
    auto second_pass = [&](const uint4& u) {
      float f[8];
      unpack8(u, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float d = f[i] - mean;
        q += d * d;
      }
    };
#pragma unroll
    for (int c = 0; c < NF_CACHE; ++c)
      if (lane + 32 * c < nvec) second_pass(cache[c]);
    for (int v = lane + 32 * NF_CACHE; v < nvec; v += 32) second_pass(src[v]);
    q = warp_sum(q);
    rstd = rsqrtf(q / cols + eps);
  }
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  const uint4* gv = reinterpret_cast<const uint4*>(gamma);
  const uint4* bv = beta ? reinterpret_cast<const uint4*>(beta) : nullptr;
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * cols);
  auto write_out = [&](const uint4& u, int v) {
    float f[8], g[8], b[8];
    unpack8(u, f);
    unpack8(__ldg(gv + v), g);
    if (bv) unpack8(__ldg(bv + v), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float h = (f[i] - mean) * rstd * g[i];
      f[i] = bv ? h + b[i] : h;
    }
    yr[v] = pack8(f);
  };
#pragma unroll
  for (int c = 0; c < NF_CACHE; ++c)
    if (lane + 32 * c < nvec) write_out(cache[c], lane + 32 * c);
  for (int v = lane + 32 * NF_CACHE; v < nvec; v += 32) write_out(src[v], v);
}

// ----------------------------------------------------------------------------- LayerNorm bwd dx
template <bool RMS>
__global__ void __launch_bounds__(ROW_WARPS * 32)
norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                   const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                   __nv_bfloat16* __restrict__ dx, int rows, int cols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ROW_WARPS + warp;
  if (row >= rows) return;
  const int nvec = cols >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
  const uint4* dr = reinterpret_cast<const uint4*>(dy + (size_t)row * cols);
  const uint4* gv = reinterpret_cast<const uint4*>(gamma);
  const float mean = RMS ? 0.f : mean_in[row];
  const float rstd = rstd_in[row];
  // sums of g*dy and g*dy*xhat
  float s1 = 0.f, s2 = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    float fx[8], fd[8], g[8];
    unpack8(xr[v], fx);
    unpack8(dr[v], fd);
    unpack8(__ldg(gv + v), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float gd = g[i] * fd[i];
      float xh = (fx[i] - mean) * rstd;
      s1 += gd;
      s2 += gd * xh;
    }
  }
  s1 = warp_sum(s1) / cols;
  s2 = warp_sum(s2) / cols;
  if (RMS) s1 = 0.f;
  const uint4* av = dx_add ? reinterpret_cast<const uint4*>(dx_add + (size_t)row * cols) : nullptr;
  uint4* ov = reinterpret_cast<uint4*>(dx + (size_t)row * cols);
  for (int v = lane; v < nvec; v += 32) {
    float fx[8], fd[8], g[8], a[8];
    unpack8(xr[v], fx);
    unpack8(dr[v], fd);
    unpack8(__ldg(gv + v), g);
    if (av) unpack8(av[v], a);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float xh = (fx[i] - mean) * rstd;
      float r = rstd * (g[i] * fd[i] - s1 - xh * s2);
      fx[i] = av ? r + a[i] : r;
    }
    ov[v] = pack8(fx);
  }
}

// ----------------------------------------------------------------------------- LayerNorm bwd, one pass
// dx and the per-block column partials of dgamma / dbeta from a single read of dy and x.
// A CTA of 8 warps owns LNB_ROWS consecutive rows; warp w takes rows w, w + 8, ... in ascending
// order.  The loads of a warp's next row are issued before the arithmetic of the current one
// (register double buffer), so a warp always has a row in flight; gamma is read from shared
// memory.  Per-lane column accumulators of dy*xhat / dy are added over the 8 warps in warp order
// through one shared-memory pass per quantity (layout [warp][i][vector]: conflict-free both ways)
// and the CTA writes partial[blk][c].  NV = 16-byte vectors per lane.
constexpr int LNB_ROWS = 32;
template <int NV>
__global__ void __launch_bounds__(ROW_WARPS * 32, 2)
ln_bwd_fused_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                    const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                    __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int cols,
                    int nblk) {
  constexpr int VEC = NV * 32;                      // vectors of a (padded) row
  __shared__ float red[ROW_WARPS][8 * VEC];
  __shared__ uint4 sgam[VEC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  for (int v = threadIdx.x; v < VEC; v += blockDim.x)
    sgam[v] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(gamma) + v) : make_uint4(0u, 0u, 0u, 0u);
  float dg[NV][8], db[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[j][i] = db[j][i] = 0.f;
  const int row0 = blockIdx.x * LNB_ROWS + warp;
  const int row_end = min(rows, (int)(blockIdx.x + 1) * LNB_ROWS);
  uint4 xn[NV], dn[NV];
  float mean_n = 0.f, rstd_n = 0.f;
  auto fetch = [&](int row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + (size_t)row * cols);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      xn[j] = v < nvec ? __ldcs(xr + v) : make_uint4(0u, 0u, 0u, 0u);
      dn[j] = v < nvec ? __ldcs(dr + v) : make_uint4(0u, 0u, 0u, 0u);
    }
    mean_n = __ldg(mean_in + row);
    rstd_n = __ldg(rstd_in + row);
  };
  if (row0 < row_end) fetch(row0);
  __syncthreads();                                  // gamma is in shared memory
  for (int row = row0; row < row_end; row += ROW_WARPS) {
    uint4 xp[NV], dp[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      xp[j] = xn[j];
      dp[j] = dn[j];
    }
    const float mean = mean_n, rstd = rstd_n;
    if (row + ROW_WARPS < row_end) fetch(row + ROW_WARPS);     // in flight during this row's arithmetic
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (lane + 32 * j < nvec) {
        float fx[8], fd[8], g[8];
        unpack8(xp[j], fx);
        unpack8(dp[j], fd);
        unpack8(sgam[lane + 32 * j], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float gd = g[i] * fd[i];
          const float xh = (fx[i] - mean) * rstd;
          s1 += gd;
          s2 += gd * xh;
          dg[j][i] += fd[i] * xh;
          db[j][i] += fd[i];
        }
      }
    }
    s1 = warp_sum(s1) / cols;
    s2 = warp_sum(s2) / cols;
    const uint4* av = dx_add ? reinterpret_cast<const uint4*>(dx_add + (size_t)row * cols) : nullptr;
    uint4* ov = reinterpret_cast<uint4*>(dx + (size_t)row * cols);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      if (v < nvec) {
        float fx[8], fd[8], g[8], a[8];
        unpack8(xp[j], fx);
        unpack8(dp[j], fd);
        unpack8(sgam[v], g);
        if (av) unpack8(av[v], a);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = (fx[i] - mean) * rstd;
          const float r = rstd * (g[i] * fd[i] - s1 - xh * s2);
          fx[i] = av ? r + a[i] : r;
        }
        ov[v] = pack8(fx);
      }
    }
  }
  // the 8 warps' column accumulators, added in warp order: dgamma first, then dbeta
  float* pg = partial + (size_t)blockIdx.x * cols;
  float* pb = partial + ((size_t)nblk + blockIdx.x) * cols;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    if (pass) __syncthreads();                      // the sums of pass 0 have been read
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) red[warp][i * VEC + lane + 32 * j] = pass ? db[j][i] : dg[j][i];
    __syncthreads();
    for (int idx = threadIdx.x; idx < 8 * VEC; idx += blockDim.x) {
      const int i = idx / VEC, v = idx - i * VEC;
      if (v < nvec) {
        float t = red[0][idx];
#pragma unroll
        for (int w = 1; w < ROW_WARPS; ++w) t += red[w][idx];
        (pass ? pb : pg)[v * 8 + i] = t;
      }
    }
  }
}

// Fixed-order sum over many block partials, parallel over 8 interleaved groups of blocks:
// thread (g, c) adds partial[b][c] for b = g, g + 8, ... ascending, then the 8 group sums are
// added in group order.  `two` arrays per launch (dgamma and dbeta).
__global__ void __launch_bounds__(256)
col_final_wide_kernel(const float* __restrict__ partial, float* __restrict__ out,
                      const float* __restrict__ partial2, float* __restrict__ out2, int cols, int nblk,
                      int accumulate) {
  __shared__ float sm[2][8][32];
  const int cl = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float s = 0.f, t = 0.f;
  if (c < cols) {
#pragma unroll 4
    for (int b = g; b < nblk; b += 8) {
      s += partial[(size_t)b * cols + c];
      if (partial2) t += partial2[(size_t)b * cols + c];
    }
  }
  sm[0][g][cl] = s;
  sm[1][g][cl] = t;
  __syncthreads();
  if (g == 0 && c < cols) {
    float a = 0.f, b2 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a += sm[0][k][cl];
      b2 += sm[1][k][cl];
    }
    out[c] = accumulate ? out[c] + a : a;
    if (partial2) out2[c] = accumulate ? out2[c] + b2 : b2;
  }
}

// Column partials: partial[blk][c] = sum over this block's rows of dy*xhat, and of dy.
// MODE 0: LayerNorm (two outputs), 1: RMSNorm (dgamma only), 2: plain column sum of dy.
// A CTA covers 64 columns x COL_ROWS_PER_BLK rows with 8 row groups of 32 column pairs:
// each thread sums its rows in ascending order, then thread (group 0) adds the 8 group
// sums in ascending group order - a fixed tree, independent of scheduling.
constexpr int COL_ROWS_PER_BLK = 256;
constexpr int COL_GROUPS = 8;
template <int MODE>
__global__ void __launch_bounds__(256)
col_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                   float* __restrict__ partial, int rows, int cols, long long ld, int nblk) {
  __shared__ float sm[4][COL_GROUPS][32];
  const int cp = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + cp) * 2;
  const int blk = blockIdx.y;
  const int r0 = blk * COL_ROWS_PER_BLK;
  const int r1 = min(rows, r0 + COL_ROWS_PER_BLK);
  float g0 = 0.f, g1 = 0.f, b0 = 0.f, b1 = 0.f;
  if (c < cols) {
    for (int r = r0 + rg; r < r1; r += COL_GROUPS) {
      float2 d = unpack_bf16(*reinterpret_cast<const uint32_t*>(dy + (size_t)r * ld + c));
      if (MODE == 2) {
        b0 += d.x; b1 += d.y;
      } else {
        float2 xv = unpack_bf16(*reinterpret_cast<const uint32_t*>(x + (size_t)r * ld + c));
        float mu = MODE == 0 ? mean_in[r] : 0.f;
        float rs = rstd_in[r];
        g0 += d.x * (xv.x - mu) * rs;
        g1 += d.y * (xv.y - mu) * rs;
        b0 += d.x; b1 += d.y;
      }
    }
  }
  sm[0][rg][cp] = g0; sm[1][rg][cp] = g1; sm[2][rg][cp] = b0; sm[3][rg][cp] = b1;
  __syncthreads();
  if (rg == 0 && c < cols) {
    float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
#pragma unroll
    for (int k = 0; k < COL_GROUPS; ++k) {
      t0 += sm[0][k][cp]; t1 += sm[1][k][cp]; t2 += sm[2][k][cp]; t3 += sm[3][k][cp];
    }
    if (MODE == 2) {
      partial[(size_t)blk * cols + c] = t2;
      if (c + 1 < cols) partial[(size_t)blk * cols + c + 1] = t3;
    } else {
      partial[(size_t)blk * cols + c] = t0;
      if (c + 1 < cols) partial[(size_t)blk * cols + c + 1] = t1;
      if (MODE == 0) {
        float* pb = partial + (size_t)nblk * cols;
        pb[(size_t)blk * cols + c] = t2;
        if (c + 1 < cols) pb[(size_t)blk * cols + c + 1] = t3;
      }
    }
  }
}
// Serial (fixed-order) sum over block partials; `two` reduces a second array (dbeta) in the
// same launch.
__global__ void __launch_bounds__(128)
col_final_kernel(const float* __restrict__ partial, float* __restrict__ out,
                 const float* __restrict__ partial2, float* __restrict__ out2, int cols, int nblk,
                 int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f, t = 0.f;
#pragma unroll 8
  for (int b = 0; b < nblk; ++b) s += partial[(size_t)b * cols + c];
  out[c] = accumulate ? out[c] + s : s;
  if (partial2) {
#pragma unroll 8
    for (int b = 0; b < nblk; ++b) t += partial2[(size_t)b * cols + c];
    out2[c] = accumulate ? out2[c] + t : t;
  }
}

// ----------------------------------------------------------------------------- softmax
template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16(v);
}

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : (is_max ? -INFINITY : 0.f);
    t = is_max ? warp_max(t) : warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// One CTA per row; `limit` = number of valid columns in this row (causal rows pass row+1).
template <typename T>
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int cols, int S_causal,
                    float scale) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const int limit = S_causal > 0 ? (int)(row % S_causal) + 1 : cols;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) m = fmaxf(m, ldf(xr + c) * scale);
  m = block_reduce(m, red, true);
  const bool bad = !(fabsf(m) <= 3.0e38f);  // NaN or +-inf
  float s = 0.f;
  if (!bad)
    for (int c = threadIdx.x; c < limit; c += blockDim.x) s += __expf(ldf(xr + c) * scale - m);
  s = block_reduce(s, red, false);
  const float inv = (!bad && s > 0.f) ? 1.f / s : 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = (c < limit && inv > 0.f) ? __expf(ldf(xr + c) * scale - m) * inv : 0.f;
    stf(yr + c, v);
  }
}
// dx = scale * y * (dy - sum(dy*y))
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dy,
                   __nv_bfloat16* __restrict__ dx, int cols, float scale) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* yr = y + row * cols;
  const __nv_bfloat16* dr = dy + row * cols;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    s += __bfloat162float(yr[c]) * __bfloat162float(dr[c]);
  s = block_reduce(s, red, false);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float p = __bfloat162float(yr[c]);
    dx[row * cols + c] = __float2bfloat16(scale * p * (__bfloat162float(dr[c]) - s));
  }
}

// ----------------------------------------------------------------------------- cross entropy
// One CTA per row.  The bf16 row is staged in shared memory when it fits, so the logits are read from HBM once
// and the gradient is written once (in place allowed).  The kernel is bound by instruction issue and by the
// exponential unit (two exponentials per logit), so both walks over the row are written for a short instruction
// stream: bf16 pairs are widened with one shift / mask each, every exponential is one FFMA into ex2.approx
// (log2(e) folded into the operands), and the vectors past the vocabulary are not visited by the first walk.
constexpr int CE_THREADS = 1024;
constexpr float CE_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ce_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void ce_widen(const uint4& u, float* f) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}
__global__ void __launch_bounds__(CE_THREADS, 2)
cross_entropy_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                     float* __restrict__ losses, __nv_bfloat16* __restrict__ dlogits, int vocab,
                     int ld, float grad_scale, int use_smem) {
  extern __shared__ uint4 ce_smem[];
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = logits + row * ld;
  const uint4* xv = reinterpret_cast<const uint4*>(xr);
  const int nvec = ld >> 3;
  const int nfull = vocab >> 3;                 // vectors that lie wholly inside the vocabulary
  const int nvalid = (vocab + 7) >> 3;          // vectors that hold at least one logit
  const long long tgt = targets[row];
  // Online softmax statistics while the row streams in: each thread keeps a running maximum mt (in units of
  // log2, i.e. x * log2(e)) and the sum st of 2^(x' - mt) over its own vectors, rescaled when the maximum moves,
  // so the exponentials of the first walk run under the latency of the loads.
  float mt = -INFINITY, st = 0.f;
  auto absorb = [&](const uint4& u, int v) {
    float f[8];
    ce_widen(u, f);
    if (v >= nfull) {               // the one vector that straddles the end of the vocabulary: padding never counts
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (v * 8 + i >= vocab) f[i] = -INFINITY;
    }
    const float vm = fmaxf(fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])), fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7])));
    const float mn = fmaxf(mt, vm * CE_LOG2E);
    const float sc = (mt == mn) ? 1.f : ce_ex2(mt - mn);        // mt = -inf on the first vector: 2^-inf = 0
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      a0 += ce_ex2(fmaf(f[i], CE_LOG2E, -mn));
      a1 += ce_ex2(fmaf(f[i + 1], CE_LOG2E, -mn));
    }
    st = fmaf(st, sc, a0 + a1);
    mt = mn;
  };
  if (use_smem) {
    // The whole row is requested at once with 16-byte asynchronous copies straight into shared memory (no
    // registers hold data in flight), committed in groups of four per thread; each thread then waits for its
    // own groups in order and absorbs the vectors it copied itself, so no CTA barrier separates copy and use.
    const uint32_t sbase = smem_u32(ce_smem);
    int groups = 0;
    for (int v0 = threadIdx.x; v0 < nvalid; v0 += 4 * CE_THREADS) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = v0 + k * CE_THREADS;
        if (v < nvalid)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sbase + 16u * v), "l"(xv + v) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      ++groups;
    }
    int g = 0;
    for (int v0 = threadIdx.x; v0 < nvalid; v0 += 4 * CE_THREADS, ++g) {
      switch (groups - 1 - g) {     // groups still allowed to be in flight
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = v0 + k * CE_THREADS;
        if (v < nvalid) absorb(ce_smem[v], v);
      }
    }
  } else {
    // rows too long for shared memory: four 16-byte loads in flight per thread, second walk re-reads from L2
    for (int v0 = threadIdx.x; v0 < nvalid; v0 += 4 * CE_THREADS) {
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = v0 + k * CE_THREADS;
        if (v < nvalid) u[k] = xv[v];
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = v0 + k * CE_THREADS;
        if (v < nvalid) absorb(u[k], v);
      }
    }
  }
  const float m2 = block_reduce(mt, red, true);                  // row maximum times log2(e)
  // per-thread sums are brought to the common maximum and added in the fixed order of the block reduction
  const float s = block_reduce(mt == -INFINITY ? 0.f : st * ce_ex2(mt - m2), red, false);
  const uint4* src = use_smem ? ce_smem : xv;
  const bool ignore = !(tgt >= 0 && tgt < vocab);
  if (threadIdx.x == 0) {
    const float xt = ignore ? 0.f : __bfloat162float(use_smem ? reinterpret_cast<const __nv_bfloat16*>(ce_smem)[tgt] : xr[tgt]);
    losses[row] = ignore ? 0.f : (m2 + __log2f(s)) * 0.6931471805599453f - xt;
  }
  if (dlogits) {
    __syncthreads();  // the target logit was read before any in-place write
    uint4* ov = reinterpret_cast<uint4*>(dlogits + row * ld);
    if (ignore) {
      for (int v = threadIdx.x; v < nvec; v += CE_THREADS) ov[v] = make_uint4(0u, 0u, 0u, 0u);
      return;
    }
    const float k = grad_scale / s;                 // softmax normalisation and loss scale in one factor
    const int vt = (int)(tgt >> 3);                 // the vector that holds the target column
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      if (v >= nvalid) {                            // padding columns carry no gradient
        ov[v] = make_uint4(0u, 0u, 0u, 0u);
        continue;
      }
      float f[8];
      ce_widen(src[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = ce_ex2(fmaf(f[i], CE_LOG2E, -m2)) * k;
      if (v == vt || v >= nfull) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = v * 8 + i;
          if (c == tgt) f[i] -= grad_scale;
          if (c >= vocab) f[i] = 0.f;
        }
      }
      ov[v] = pack8(f);
    }
  }
}

// ----------------------------------------------------------------------------- reductions
// Single CTA, fixed tree: each thread sums a strided slice serially, then a fixed
// shuffle/shared tree combines the 1024 partials.  Result is independent of anything
// but n, so it replays bit-identically.
template <bool SQUARE>
__global__ void __launch_bounds__(1024)
reduce_one_block_kernel(const float* __restrict__ x, float* __restrict__ out, long long n,
                        float scale, int accumulate) {
  __shared__ float red[33];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += 1024) {
    float v = x[i];
    s += SQUARE ? v * v : v;
  }
  s = block_reduce(s, red, false);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s * scale : s * scale;
}
// Two-level version for large buffers: level 1 writes one partial per CTA.
template <bool SQUARE>
__global__ void __launch_bounds__(256)
reduce_level1_kernel(const float* __restrict__ x, float* __restrict__ partial, long long n) {
  __shared__ float red[33];
  const long long per = (n + gridDim.x - 1) / gridDim.x;
  const long long b = per * blockIdx.x, e = (b + per < n) ? b + per : n;
  float s = 0.f;
  for (long long i = b + threadIdx.x; i < e; i += 256) {
    float v = x[i];
    s += SQUARE ? v * v : v;
  }
  s = block_reduce(s, red, false);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

}  // namespace ftk

using namespace ftk;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFW(p) reinterpret_cast<__nv_bfloat16*>(p)

extern "C" int ftk_layernorm_fwd(const void* x, const void* resid_in, void* sum_out,
                                 const void* gamma, const void* beta, void* y, float* mean,
                                 float* rstd, int rows, int cols, float eps, void* stream) {
  if (cols % 8 || rows <= 0) return -2;
  if (resid_in && !sum_out) return -3;
  norm_fwd_kernel<false><<<(rows + ROW_WARPS - 1) / ROW_WARPS, ROW_WARPS * 32, 0, STREAM(stream)>>>(
      BF(x), BF(resid_in), BFW(sum_out), BF(gamma), BF(beta), BFW(y), mean, rstd, rows, cols, eps);
  return (int)cudaGetLastError();
}
extern "C" int ftk_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows,
                               int cols, float eps, void* stream) {
  if (cols % 8 || rows <= 0) return -2;
  norm_fwd_kernel<true><<<(rows + ROW_WARPS - 1) / ROW_WARPS, ROW_WARPS * 32, 0, STREAM(stream)>>>(
      BF(x), nullptr, nullptr, BF(gamma), nullptr, BFW(y), nullptr, rstd, rows, cols, eps);
  return (int)cudaGetLastError();
}
// number of partial blocks the caller must provide room for (2 * blocks * cols floats)
extern "C" int ftk_layernorm_bwd_blocks(int rows) { return (rows + LNB_ROWS - 1) / LNB_ROWS; }
static int norm_col_blocks(int rows) { return (rows + COL_ROWS_PER_BLK - 1) / COL_ROWS_PER_BLK; }

extern "C" int ftk_layernorm_bwd(const void* dy, const void* x, const void* gamma,
                                 const float* mean, const float* rstd, const void* dx_add, void* dx,
                                 float* dgamma, float* dbeta, float* partial, int rows, int cols,
                                 int accumulate, void* stream) {
  if (cols % 8 || rows <= 0) return -2;
  cudaStream_t s = STREAM(stream);
  if (dgamma && cols <= 768) {
    // one pass: dx + column partials, then the fixed-order sum over blocks (wider rows would
    // spill the per-lane column accumulators and take the three-kernel path below)
    const int nblk = ftk_layernorm_bwd_blocks(rows);
    ln_bwd_fused_kernel<3><<<nblk, ROW_WARPS * 32, 0, s>>>(BF(dy), BF(x), BF(gamma), mean, rstd, BF(dx_add),
                                                          BFW(dx), partial, rows, cols, nblk);
    col_final_wide_kernel<<<(cols + 31) / 32, 256, 0, s>>>(partial, dgamma, partial + (size_t)nblk * cols, dbeta,
                                                           cols, nblk, accumulate);
    return (int)cudaGetLastError();
  }
  norm_bwd_dx_kernel<false><<<(rows + ROW_WARPS - 1) / ROW_WARPS, ROW_WARPS * 32, 0, s>>>(
      BF(dy), BF(x), BF(gamma), mean, rstd, BF(dx_add), BFW(dx), rows, cols);
  if (dgamma) {
    const int nblk = norm_col_blocks(rows);
    dim3 g((cols / 2 + 31) / 32, nblk);
    col_partial_kernel<0><<<g, 256, 0, s>>>(BF(dy), BF(x), mean, rstd, partial, rows, cols, cols, nblk);
    col_final_kernel<<<(cols + 127) / 128, 128, 0, s>>>(partial, dgamma, partial + (size_t)nblk * cols,
                                                         dbeta, cols, nblk, accumulate);
  }
  return (int)cudaGetLastError();
}
extern "C" int ftk_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd,
                               void* dx, float* dgamma, float* partial, int rows, int cols,
                               int accumulate, void* stream) {
  if (cols % 8 || rows <= 0) return -2;
  cudaStream_t s = STREAM(stream);
  norm_bwd_dx_kernel<true><<<(rows + ROW_WARPS - 1) / ROW_WARPS, ROW_WARPS * 32, 0, s>>>(
      BF(dy), BF(x), BF(gamma), nullptr, rstd, nullptr, BFW(dx), rows, cols);
  if (dgamma) {
    const int nblk = norm_col_blocks(rows);
    dim3 g((cols / 2 + 31) / 32, nblk);
    col_partial_kernel<1><<<g, 256, 0, s>>>(BF(dy), BF(x), nullptr, rstd, partial, rows, cols, cols, nblk);
    col_final_wide_kernel<<<(cols + 31) / 32, 256, 0, s>>>(partial, dgamma, nullptr, nullptr, cols, nblk,
                                                           accumulate);
  }
  return (int)cudaGetLastError();
}
// Plain column sums with 16-byte loads: a CTA covers 256 columns x CSW_ROWS rows as 8 row groups of
// 32 lanes x 8 columns.  Each thread adds its rows (r0 + group, + 8, ...) in ascending order with four
// row loads in flight, then group 0 adds the 8 group sums in group order: a fixed tree again.
constexpr int CSW_ROWS = 64;
__global__ void __launch_bounds__(256)
colsum_wide_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ partial, int rows, int cols,
                   long long ld) {
  __shared__ float sm[COL_GROUPS][32][9];
  const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * 8;
  const int blk = blockIdx.y;
  const int r0 = blk * CSW_ROWS;
  const int r1 = min(rows, r0 + CSW_ROWS);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < cols) {
    int r = r0 + rg;
    for (; r + 3 * COL_GROUPS < r1; r += 4 * COL_GROUPS) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(r + u * COL_GROUPS) * ld + c));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 f0 = unpack_bf16(v[u].x), f1 = unpack_bf16(v[u].y), f2 = unpack_bf16(v[u].z),
                     f3 = unpack_bf16(v[u].w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
        acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
    }
    for (; r < r1; r += COL_GROUPS) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * ld + c));
      const float2 f0 = unpack_bf16(w.x), f1 = unpack_bf16(w.y), f2 = unpack_bf16(w.z), f3 = unpack_bf16(w.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
      acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm[rg][lane][i] = acc[i];
  __syncthreads();
  if (rg == 0 && c < cols) {
    float t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = 0.f;
#pragma unroll
    for (int k = 0; k < COL_GROUPS; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) t[i] += sm[k][lane][i];
    float* dst = partial + (size_t)blk * cols + c;
    reinterpret_cast<float4*>(dst)[0] = make_float4(t[0], t[1], t[2], t[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(t[4], t[5], t[6], t[7]);
  }
}

// Number of row blocks (= rows of the partial buffer the caller provides) for `rows` input rows.
extern "C" int ftk_colsum_blocks(int rows) { return (rows + CSW_ROWS - 1) / CSW_ROWS; }

extern "C" int ftk_colsum_bf16(const void* x, float* out, float* partial, int rows, int cols,
                               long long ld, int accumulate, void* stream) {
  if (cols % 2 || ld % 2 || rows <= 0) return -2;
  cudaStream_t s = STREAM(stream);
  const bool wide = (cols % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(partial) & 15) == 0);
  int nblk;
  if (wide) {
    nblk = ftk_colsum_blocks(rows);
    dim3 g((cols / 8 + 31) / 32, nblk);
    colsum_wide_kernel<<<g, 256, 0, s>>>(BF(x), partial, rows, cols, ld);
  } else {
    // odd extents / alignments: two columns per thread; needs fewer row blocks than were provided for
    nblk = (rows + COL_ROWS_PER_BLK - 1) / COL_ROWS_PER_BLK;
    dim3 g((cols / 2 + 31) / 32, nblk);
    col_partial_kernel<2><<<g, 256, 0, s>>>(BF(x), nullptr, nullptr, nullptr, partial, rows, cols, ld, nblk);
  }
  col_final_wide_kernel<<<(cols + 31) / 32, 256, 0, s>>>(partial, out, nullptr, nullptr, cols, nblk, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int ftk_softmax_rows(const void* x, void* y, int rows, int cols, int is_bf16,
                                void* stream) {
  if (rows <= 0 || cols <= 0) return -2;
  if (is_bf16)
    softmax_rows_kernel<__nv_bfloat16><<<rows, 256, 0, STREAM(stream)>>>(BF(x), BFW(y), cols, 0, 1.f);
  else
    softmax_rows_kernel<float><<<rows, 256, 0, STREAM(stream)>>>(
        reinterpret_cast<const float*>(x), reinterpret_cast<float*>(y), cols, 0, 1.f);
  return (int)cudaGetLastError();
}
extern "C" int ftk_softmax_causal_bf16(const void* x, void* y, int L, int S, float scale,
                                       void* stream) {
  if (L <= 0 || S <= 0) return -2;
  softmax_rows_kernel<__nv_bfloat16><<<(unsigned)((size_t)L * S), 256, 0, STREAM(stream)>>>(
      BF(x), BFW(y), S, S, scale);
  return (int)cudaGetLastError();
}
extern "C" int ftk_softmax_bwd_bf16(const void* y, const void* dy, void* dx, long long rows,
                                    int cols, float scale, void* stream) {
  if (rows <= 0 || cols <= 0) return -2;
  softmax_bwd_kernel<<<(unsigned)rows, 256, 0, STREAM(stream)>>>(BF(y), BF(dy), BFW(dx), cols, scale);
  return (int)cudaGetLastError();
}

extern "C" int ftk_cross_entropy_fwd_bwd(const void* logits, const long long* targets,
                                         float* losses, void* dlogits, int rows, int vocab, int ld,
                                         float grad_scale, void* stream) {
  if (ld % 8 || vocab > ld || rows <= 0) return -2;
  const size_t bytes = (size_t)ld * 2;
  const int use_smem = bytes <= 200 * 1024;     // longer rows are re-read from L2 by the second walk
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(cross_entropy_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  cross_entropy_kernel<<<rows, CE_THREADS, use_smem ? bytes : 0, STREAM(stream)>>>(
      BF(logits), targets, losses, BFW(dlogits), vocab, ld, grad_scale, use_smem);
  return (int)cudaGetLastError();
}

extern "C" int ftk_reduce_mean_f32(const float* x, float* out, long long n, float scale,
                                   void* stream) {
  if (n <= 0) return -2;
  reduce_one_block_kernel<false><<<1, 1024, 0, STREAM(stream)>>>(x, out, n, scale, 0);
  return (int)cudaGetLastError();
}
extern "C" int ftk_sumsq_f32(const float* x, float* out, float* partial, long long n,
                             int accumulate, void* stream) {
  if (n <= 0) return -2;
  if (n < (1 << 16) || !partial) {
    reduce_one_block_kernel<true><<<1, 1024, 0, STREAM(stream)>>>(x, out, n, 1.f, accumulate);
  } else {
    // level 1: FTK_SUMSQ_PARTIALS fixed slices; level 2: one block over the partials
    reduce_level1_kernel<true><<<FTK_SUMSQ_PARTIALS, 256, 0, STREAM(stream)>>>(x, partial, n);
    reduce_one_block_kernel<false><<<1, 1024, 0, STREAM(stream)>>>(partial, out, FTK_SUMSQ_PARTIALS,
                                                                    1.f, accumulate);
  }
  return (int)cudaGetLastError();
}
