// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): one 256 x 256 output tile per 2-CTA cluster.
//
// Each CTA of the pair loads its own 128 rows of A and its own 128 columns of B per k-block
// (32 KB per stage instead of the 48 KB a lone 128 x 256 tile needs), which cuts the L2 -> SM
// operand traffic per FLOP by a third - the limiter of the single-CTA kernel.  The leader CTA
// (cluster rank 0) issues MMAs that read both CTAs' shared memory and write 128 accumulator rows
// x 256 columns into each CTA's TMEM; both CTAs run a TMA producer warp and 8 epilogue warps.
// TMA completion bytes of both CTAs go to the leader's `full` barrier; `empty` / `tmem full` are
// signalled in both CTAs by a commit multicast (no data multicast anywhere); the peer's
// epilogue releases accumulators with remote arrives on the leader's `tmem empty` barrier.
//
// Same operand forms (K-major / MN-major), epilogues and deterministic split-K as the single-CTA
// kernel in gemm_kernel.cuh; the k order of every output element is ascending and independent
// of the grid.
#pragma once
#include "gemm_kernel.cuh"

namespace ftk {

struct Gemm2Cfg {
  static constexpr int BN = 256;                   // tile columns (128 staged per CTA)
  static constexpr int A_BYTES = G_BM * G_BK * 2;  // per CTA and stage
  static constexpr int B_BYTES = 128 * G_BK * 2;
  static constexpr int STAGES = 6;
  static constexpr int ACC_STRIDE = 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/ +
                              G_EPI_WARPS * 4096 /*output staging tiles*/;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G_THREADS, 1)
gemm2_bf16_sm100_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB, const GemmArgs p) {
  using Cfg = Gemm2Cfg;
  constexpr int BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  // (the dynamic shared-memory base has the same offset in both CTAs, so do the aligned bases)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + Cfg::STAGES * Cfg::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES));
  uint64_t* full = bars;                       // leader's copy is the one in use
  uint64_t* empty = bars + Cfg::STAGES;        // per CTA
  uint64_t* tfull = bars + 2 * Cfg::STAGES;    // per CTA
  uint64_t* tempty = tfull + 2;                // leader's copy is the one in use
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const bool leader = rank == 0;
  WaitCtx ctx{p.status, abort_f};

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 2 * G_EPI_WARPS);
    }
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int pair = (int)blockIdx.x >> 1;
  const int n_pairs = (int)gridDim.x >> 1;
  const int tiles_m2 = (p.M + 2 * G_BM - 1) / (2 * G_BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_mn = tiles_m2 * tiles_n;
  const int nbatch = p.L0 * p.L1;
  const int total = tiles_mn * nbatch * p.splits;
  const int kblocks_all = (p.K + G_BK - 1) / G_BK;
  const int kb_per_split = (kblocks_all + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
    }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = pair; ok && item < total; item += n_pairs) {
      const int sp = item / (tiles_mn * nbatch);
      const int rem = item - sp * (tiles_mn * nbatch);
      const int l = rem / tiles_mn;
      const int t = rem - l * tiles_mn;
      const int a_row = (2 * (t % tiles_m2) + rank) * G_BM;
      const int b_row = (t / tiles_m2) * BN + rank * 128;
      const int l0 = l % p.L0, l1 = l / p.L0;
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(kblocks_all, kb0 + kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[s], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          // the leader's barrier collects the bytes of both CTAs
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * (Cfg::A_BYTES + Cfg::B_BYTES));
          uint8_t* a_dst = sA + s * Cfg::A_BYTES;
          uint8_t* b_dst = sB + s * Cfg::B_BYTES;
          if (!p.a_mn) {
            tma_load_4d_pair(a_dst, &tmA, &full[s], kb * G_BK, a_row, l0, l1);
          } else {
#pragma unroll
            for (int cc = 0; cc < G_BM / 64; ++cc)
              tma_load_4d_pair(a_dst + cc * (G_BK * 128), &tmA, &full[s], a_row + cc * 64, kb * G_BK, l0, l1);
          }
          if (!p.b_mn) {
            tma_load_4d_pair(b_dst, &tmB, &full[s], kb * G_BK, b_row, l0, l1);
          } else {
#pragma unroll
            for (int cc = 0; cc < 128 / 64; ++cc)
              tma_load_4d_pair(b_dst + cc * (G_BK * 128), &tmB, &full[s], b_row + cc * 64, kb * G_BK, l0, l1);
          }
        }
        __syncwarp();
        if (++s == Cfg::STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      const uint32_t idesc = make_idesc_bf16(2 * G_BM, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? G_BK * 128 : 16, a_adv = p.a_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
      const uint32_t b_lbo = p.b_mn ? G_BK * 128 : 16, b_adv = p.b_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
      const uint32_t a_lo0 = desc_lo(smem_u32(sA), a_lbo), b_lo0 = desc_lo(smem_u32(sB), b_lbo);
      const uint32_t a_adv16 = a_adv >> 4, b_adv16 = b_adv >> 4;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int item = pair; ok && item < total; item += n_pairs) {
        const int sp = item / (tiles_mn * nbatch);
        const int kb0 = sp * kb_per_split;
        const int kb1 = min(kblocks_all, kb0 + kb_per_split);
        if (!mbar_wait(&tempty[acc], ((acc_ph >> acc) & 1u) ^ 1u, ctx, FT_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, ctx, FT_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_lo = a_lo0 + (uint32_t)s * (Cfg::A_BYTES >> 4);
            const uint32_t b_lo = b_lo0 + (uint32_t)s * (Cfg::B_BYTES >> 4);
            umma_bf16_pair_lo(d_tmem, a_lo, b_lo, idesc, kb > kb0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < G_BK / G_UMMA_K; ++k)
              umma_bf16_pair_lo(d_tmem, a_lo + k * a_adv16, b_lo + k * b_adv16, idesc, 1u);
            umma_commit_pair(&empty[s], 3);                       // the stage is free in both CTAs
            if (kb == kb1 - 1) umma_commit_pair(&tfull[acc], 3);  // both epilogues may drain
          }
          __syncwarp();
          if (++s == Cfg::STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (kb1 <= kb0 && lane == 0) umma_commit_pair(&tfull[acc], 3);  // empty split
        __syncwarp();
        acc_ph ^= (1u << acc);
        acc ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps, both CTAs)
    const int ew = warp - 2;
    const int q = warp & 3;
    const int half = ew >> 2;
    const int row_in_tile = q * 32 + lane;
    constexpr int CHUNKS = BN / 32;
    constexpr int C_HALF = CHUNKS / 2;
    const int c_begin = half == 0 ? 0 : C_HALF;
    const int c_end = half == 0 ? C_HALF : CHUNKS;
    int acc = 0;
    uint32_t acc_ph = 0;
    for (int item = pair; item < total; item += n_pairs) {
      const int sp = item / (tiles_mn * nbatch);
      const int rem = item - sp * (tiles_mn * nbatch);
      const int l = rem / tiles_mn;
      const int t = rem - l * tiles_mn;
      const int m_t = 2 * (t % tiles_m2) + rank, n_t = t / tiles_m2;
      const int l0 = l % p.L0, l1 = l / p.L0;
      const bool empty_split = (sp * kb_per_split >= kblocks_all);
      if (!mbar_wait(&tfull[acc], (acc_ph >> acc) & 1u, ctx, FT_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const long long row = (long long)m_t * G_BM + row_in_tile;
      const long long d_off = l0 * p.d_s0 + l1 * p.d_s1 + row * p.ldd;
      const long long r_off = l0 * p.r_s0 + l1 * p.r_s1 + row * p.ldr;
      const bool need_r = p.resid != nullptr;
      // bf16 outputs leave through a per-warp transposing smem tile (see OutStager)
      OutStager stager(smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES) + 256 + ew * 4096, p,
                       reinterpret_cast<__nv_bfloat16*>(p.D) + l0 * p.d_s0 + l1 * p.d_s1,
                       (long long)m_t * G_BM + q * 32, lane);
#pragma unroll 1
      for (int ci = c_begin; ci < c_end; ++ci) {
        const int c0 = ci * 32;
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * Cfg::ACC_STRIDE + c0 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int n0 = n_t * BN + c0;
        const bool stage_this = stager.usable && n0 + 32 <= p.N;     // warp-uniform
        if (!stage_this) stager.flush();
        if (row < p.M && n0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = empty_split ? 0.f : __uint_as_float(r[i]) * p.alpha;
          const bool full_chunk = (n0 + 32 <= p.N);
          if (p.splits > 1) {
            float* wp = p.ws + (((long long)sp * nbatch + l) * p.M + row) * p.N + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(wp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(wp)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N) wp[i] = v[i];
            }
            continue;
          }
          if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (full_chunk || n0 + i < p.N) v[i] += __bfloat162float(__ldg(p.bias + n0 + i));
          }
          if (p.aux) {
            __nv_bfloat16* ap = p.aux + d_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(ap) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 o;
                o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
                o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
                o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
                reinterpret_cast<uint4*>(ap)[i] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N) ap[i] = __float2bfloat16(v[i]);
            }
          }
          float rr[32];
          if (need_r) {
            const __nv_bfloat16* rp = p.resid + r_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 u = __ldg(reinterpret_cast<const uint4*>(rp) + i);
                float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z),
                       f3 = unpack_bf16(u.w);
                rr[8 * i + 0] = f0.x; rr[8 * i + 1] = f0.y; rr[8 * i + 2] = f1.x;
                rr[8 * i + 3] = f1.y; rr[8 * i + 4] = f2.x; rr[8 * i + 5] = f2.y;
                rr[8 * i + 6] = f3.x; rr[8 * i + 7] = f3.y;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                rr[i] = (n0 + i < p.N) ? __bfloat162float(rp[i]) : 0.f;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = 0.f;
          }
          const bool r_is_operand = (p.epi >= FTK_EPI_MUL_DGELU_TANH);
          if (p.epi != FTK_EPI_NONE) apply_epi32(v, rr, p.epi);
          if (need_r && !r_is_operand) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += rr[i];
          }
          if (p.out_fp32) {
            float* dp = reinterpret_cast<float*>(p.D) + d_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                if (p.accumulate) {
                  float4 old = reinterpret_cast<float4*>(dp)[i];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4*>(dp)[i] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N) dp[i] = p.accumulate ? dp[i] + v[i] : v[i];
            }
          } else if (stage_this) {
            stager.put(v);
          } else {
            __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + d_off + n0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (p.accumulate) {
                  uint4 u = reinterpret_cast<uint4*>(dp)[i];
                  float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z),
                         f3 = unpack_bf16(u.w);
                  v[8 * i + 0] += f0.x; v[8 * i + 1] += f0.y; v[8 * i + 2] += f1.x;
                  v[8 * i + 3] += f1.y; v[8 * i + 4] += f2.x; v[8 * i + 5] += f2.y;
                  v[8 * i + 6] += f3.x; v[8 * i + 7] += f3.y;
                }
                uint4 o;
                o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
                o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
                o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
                reinterpret_cast<uint4*>(dp)[i] = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (n0 + i < p.N)
                  dp[i] = __float2bfloat16(p.accumulate ? __bfloat162float(dp[i]) + v[i] : v[i]);
            }
          }
        }
        if (stage_this) stager.chunk_done(n0);     // every lane of the warp, also rows past M
      }
      stager.flush();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[acc]);   // the MMA warp lives in the leader CTA
      acc_ph ^= (1u << acc);
      acc ^= 1;
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // neither CTA leaves while the other may still signal it
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace ftk
