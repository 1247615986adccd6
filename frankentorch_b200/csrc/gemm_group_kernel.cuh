// Grouped GEMM: several independent products with a common reduction length in ONE persistent launch.
//
//   D_p [M_p, N_p] (fp32) (+)= alpha * A_p . B_p      p = 0 .. n-1,  same K, same operand layouts
//
// Purpose: the four weight gradients of a transformer block (dW = dY^T X with K = tokens) have 24 - 96
// output tiles each, far fewer than the 148 SMs, so on their own they need split-K plus a reduction kernel.
// Together they are 288 tiles of 128 x 192: two full waves with no split at all - every output element is
// reduced over K by one CTA in k-block order, which is also the simplest deterministic order there is.
//
// The kernel is the single-CTA tcgen05 GEMM of gemm_kernel.cuh (TMA producer warp, MMA issuer warp, eight
// epilogue warps, operand ring, two TMEM accumulators, bounded waits with the shared status word)
// reduced to what a weight gradient needs - fp32 output with optional accumulation, no bias / activation /
// residual, no split, no collective - plus a table of problems: a work item is (problem, n tile, m tile),
// items are dealt round robin to the CTAs, and each problem brings its own pair of tensor maps.
// The reference has no grouped product (its CPU `mod gemm`, ft-kernel-cpu/src/lib.rs:18-1677, runs one
// matrix product per call).
#pragma once
#include "gemm_kernel.cuh"

namespace ftk {

constexpr int GG_MAX = 8;   // problems per launch
constexpr int GG_BN = 192;
// Five operand stages (the single-product kernel has four plus 32 KB of output staging tiles, which an fp32
// store epilogue does not need): with both operands MN-major a stage is five TMA boxes, and at four stages
// the tensor pipe sat at 50 % waiting for them.
constexpr int GG_STAGES = 5;
constexpr int GG_SMEM = GG_STAGES * (G_BM * G_BK * 2 + GG_BN * G_BK * 2) + 1024 /*align*/ + 256 /*barriers*/;

struct GroupArgs {
  int n;                       // number of problems
  int K;
  int a_mn, b_mn;
  int M[GG_MAX], N[GG_MAX];
  int tile_end[GG_MAX];        // running total of 128 x GG_BN tiles up to and including problem p
  float* D[GG_MAX];
  long long ldd[GG_MAX];
  int accumulate[GG_MAX];
  float alpha;
  int* status;
};
struct GroupMaps {
  CUtensorMap a[GG_MAX];
  CUtensorMap b[GG_MAX];
};

struct GroupTile {
  int p, m_t, n_t;
};
__device__ __forceinline__ GroupTile group_decode(int item, const GroupArgs& g) {
  GroupTile t;
  t.p = 0;
#pragma unroll
  for (int i = 0; i < GG_MAX - 1; ++i)
    if (i + 1 < g.n && item >= g.tile_end[i]) t.p = i + 1;
  const int local = item - (t.p > 0 ? g.tile_end[t.p - 1] : 0);
  const int tiles_m = (g.M[t.p] + G_BM - 1) / G_BM;
  t.m_t = local % tiles_m;
  t.n_t = local / tiles_m;
  return t;
}

__global__ void __launch_bounds__(G_THREADS, 1)
gemm_group_bf16_sm100_kernel(const __grid_constant__ GroupMaps maps, const GroupArgs g) {
  constexpr int BN = GG_BN;
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + GG_STAGES * Cfg::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GG_STAGES * (Cfg::A_BYTES + Cfg::B_BYTES));
  uint64_t* full = bars;
  uint64_t* empty = bars + GG_STAGES;
  uint64_t* tfull = bars + 2 * GG_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx ctx{g.status, abort_f};

  if (threadIdx.x == 0) {
    for (int i = 0; i < GG_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], G_EPI_WARPS);
    }
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total = g.tile_end[g.n - 1];
  const int kblocks = (g.K + G_BK - 1) / G_BK;
  const int n_ctas = (int)gridDim.x;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total; item += n_ctas) {
      const GroupTile t = group_decode(item, g);
      const CUtensorMap* mapA = &maps.a[t.p];
      const CUtensorMap* mapB = &maps.b[t.p];
      if (lane == 0) {
        tma_prefetch_desc(mapA);
        tma_prefetch_desc(mapB);
      }
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!mbar_wait(&empty[s], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
          uint8_t* a_dst = sA + s * Cfg::A_BYTES;
          uint8_t* b_dst = sB + s * Cfg::B_BYTES;
          if (!g.a_mn) {
            tma_load_4d(a_dst, mapA, &full[s], kb * G_BK, t.m_t * G_BM, 0, 0);
          } else {
#pragma unroll
            for (int cc = 0; cc < G_BM / 64; ++cc)
              tma_load_4d(a_dst + cc * (G_BK * 128), mapA, &full[s], t.m_t * G_BM + cc * 64, kb * G_BK, 0, 0);
          }
          if (!g.b_mn) {
            tma_load_4d(b_dst, mapB, &full[s], kb * G_BK, t.n_t * BN, 0, 0);
          } else {
#pragma unroll
            for (int cc = 0; cc < BN / 64; ++cc)
              tma_load_4d(b_dst + cc * (G_BK * 128), mapB, &full[s], t.n_t * BN + cc * 64, kb * G_BK, 0, 0);
          }
        }
        __syncwarp();
        if (++s == GG_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_bf16(G_BM, BN, g.a_mn, g.b_mn);
    const uint32_t a_lbo = g.a_mn ? G_BK * 128 : 16, a_adv = g.a_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
    const uint32_t b_lbo = g.b_mn ? G_BK * 128 : 16, b_adv = g.b_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
    const uint32_t a_lo0 = desc_lo(smem_u32(sA), a_lbo), b_lo0 = desc_lo(smem_u32(sB), b_lbo);
    const uint32_t a_adv16 = a_adv >> 4, b_adv16 = b_adv >> 4;
    int s = 0;
    uint32_t ph = 0;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total; item += n_ctas) {
      if (!mbar_wait(&tempty[acc], ((acc_ph >> acc) & 1u) ^ 1u, ctx, FT_ERR_WAIT_TMEM_EMPTY)) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!mbar_wait(&full[s], ph, ctx, FT_ERR_WAIT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_lo = a_lo0 + (uint32_t)s * (Cfg::A_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)s * (Cfg::B_BYTES >> 4);
          umma_bf16_lo(d_tmem, a_lo, b_lo, idesc, kb > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < G_BK / G_UMMA_K; ++k)
            umma_bf16_lo(d_tmem, a_lo + k * a_adv16, b_lo + k * b_adv16, idesc, 1u);
          umma_commit(&empty[s]);
          if (kb == kblocks - 1) umma_commit(&tfull[acc]);
        }
        __syncwarp();
        if (++s == GG_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      acc_ph ^= (1u << acc);
      acc ^= 1;
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps): fp32 store / accumulate
    const int ew = warp - 2;
    const int q = warp & 3;               // TMEM lane quarter this warp may read
    const int half = ew >> 2;             // which half of the tile's columns
    const int row_in_tile = q * 32 + lane;
    constexpr int CHUNKS = BN / 32;
    constexpr int C_HALF = (CHUNKS + 1) / 2;
    const int c_begin = half == 0 ? 0 : C_HALF;
    const int c_end = half == 0 ? C_HALF : CHUNKS;
    int acc = 0;
    uint32_t acc_ph = 0;
    for (int item = blockIdx.x; item < total; item += n_ctas) {
      const GroupTile t = group_decode(item, g);
      if (!mbar_wait(&tfull[acc], (acc_ph >> acc) & 1u, ctx, FT_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int M = g.M[t.p], N = g.N[t.p];
      const bool accum = g.accumulate[t.p] != 0;
      const long long row = (long long)t.m_t * G_BM + row_in_tile;
      float* drow = g.D[t.p] + row * g.ldd[t.p];
#pragma unroll 1
      for (int ci = c_begin; ci < c_end; ++ci) {
        const int c0 = ci * 32;
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * Cfg::ACC_STRIDE + c0 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int n0 = t.n_t * BN + c0;
        if (row < M && n0 < N) {
          float* dp = drow + n0;
          if (n0 + 32 <= N && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 o = make_float4(__uint_as_float(r[4 * i]) * g.alpha, __uint_as_float(r[4 * i + 1]) * g.alpha,
                                     __uint_as_float(r[4 * i + 2]) * g.alpha, __uint_as_float(r[4 * i + 3]) * g.alpha);
              if (accum) {
                const float4 old = reinterpret_cast<const float4*>(dp)[i];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              reinterpret_cast<float4*>(dp)[i] = o;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (n0 + i < N) {
                const float v = __uint_as_float(r[i]) * g.alpha;
                dp[i] = accum ? dp[i] + v : v;
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc_ph ^= (1u << acc);
      acc ^= 1;
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_f) {
    // give copies and MMAs still in flight time to land before smem/TMEM go away
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace ftk
