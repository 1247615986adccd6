// Flash attention backward for sm_100a on tcgen05/TMEM, head_dim 64/128.
//
// Semantics (reference: ft-kernel-cpu/src/lib.rs:5300 sdpa_backward_f64; forward in
// ft-kernel-cpu/src/lib.rs:4572): P is recomputed from the saved log-sum-exp, then
//   dV = P^T dO, dP = dO V^T, dS = P o (dP - rowsum(dO o O)), dQ = scale dS K,
//   dK = scale dS^T Q.
//
// Layout: Q/K/V/O/dO are addressed in place inside the packed [B*S, 3*d] / [B*S, d]
// activations through 4-D TMA maps {head_dim, S, H, B}; no head split/merge copies.
//
// Two kernels, each 19 warps: warps 0-15 do the elementwise math, warp 16 is the TMA
// producer, warp 17 issues the score products (and owns TMEM), warp 18 the accumulating
// products.  The 16 math warps split every 128 x 128 score tile by columns (four groups of 32
// columns; a thread owns one tile row inside its group's columns), so one tcgen05.ld per
// operand brings a thread's whole share into registers, the TMEM score tiles are released at
// once and the tensor core computes the next block's scores under the exponentials of this
// one.  With head_dim 64, P^T / dS^T (or dS) go back to the tensor core through tensor memory
// (tcgen05.st by the row's thread, MMA with its A operand in TMEM); with head_dim 128 all 512
// columns hold accumulators and they go through 128B-swizzled bf16 tiles in shared memory.
//
// Determinism: dK/dV are accumulated in TMEM by the CTA that owns the key block, dQ by the
// CTA that owns the query block (second kernel), both in ascending block order; there are
// no atomics, so gradients are bit-identical run to run.
#include "attn_common.cuh"

namespace ftk {

constexpr int BW_THREADS = 608;
constexpr int BW_MATH = 16;         // one arrival per math warp on the math barriers
constexpr int BW_WARP_TMA = 16;
constexpr int BW_WARP_MMA = 17;      // issues the score products, owns TMEM
constexpr int BW_WARP_MMA2 = 18;     // issues the accumulating products

// =============================================================================== delta
// delta[b,h,s] = sum_e dO * O.  LPR = hd / 8 lanes share one (b, s, h) row (16 bytes each), so
// a warp covers 32 / LPR rows and every lane loads.
template <int LPR>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  float* __restrict__ delta, int B, int H, int S, long long bs, long long ss,
                  long long hs) {
  constexpr int RPW = 32 / LPR;                       // rows per warp
  const int lane = threadIdx.x & 31;
  const long long w = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW + lane / LPR;
  const int sub = lane % LPR;
  float acc = 0.f;
  const bool live = w < (long long)B * S * H;
  int h = 0, s = 0, b = 0;
  if (live) {
    h = (int)(w % H);
    const long long t = w / H;
    s = (int)(t % S);
    b = (int)(t / S);
    const long long off = (long long)b * bs + (long long)s * ss + (long long)h * hs + sub * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(o + off);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + off);
    float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
    float2 g0 = unpack_bf16(g.x), g1 = unpack_bf16(g.y), g2 = unpack_bf16(g.z), g3 = unpack_bf16(g.w);
    acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y +
          a3.x * g3.x + a3.y * g3.y;
  }
#pragma unroll
  for (int d = LPR / 2; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (live && sub == 0) delta[((long long)b * H + h) * S + s] = acc;
}

// Store 32 packed-bf16 columns (16 words) of one tile row into the swizzled K-major tile.
__device__ __forceinline__ void store_row32_packed(uint8_t* tile, int row, int col0,
                                                   const uint32_t* w) {
  uint8_t* base = tile + (col0 >> 6) * AT_REGION + row * 128;
  const int j0 = (col0 & 63) >> 3;
#pragma unroll
  for (int t = 0; t < 4; ++t)
    *reinterpret_cast<uint4*>(base + (((j0 + t) ^ (row & 7)) << 4)) =
        make_uint4(w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]);
}
// Scale 32 fp32 accumulator values and store them as 32 contiguous bf16.
__device__ __forceinline__ void store_out32(__nv_bfloat16* dst, const uint32_t* r, float scale) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint4 u;
    u.x = pack_bf16(__uint_as_float(r[8 * t + 0]) * scale, __uint_as_float(r[8 * t + 1]) * scale);
    u.y = pack_bf16(__uint_as_float(r[8 * t + 2]) * scale, __uint_as_float(r[8 * t + 3]) * scale);
    u.z = pack_bf16(__uint_as_float(r[8 * t + 4]) * scale, __uint_as_float(r[8 * t + 5]) * scale);
    u.w = pack_bf16(__uint_as_float(r[8 * t + 6]) * scale, __uint_as_float(r[8 * t + 7]) * scale);
    *reinterpret_cast<uint4*>(dst + 8 * t) = u;
  }
}

// =============================================================================== backward: dK, dV
#ifdef FT_ATTN_TRACE
// Optional timeline of CTA 0 of each backward kernel (development builds only):
// [kernel][role][iteration][point] clock64 values.
__device__ long long g_attn_bwd_trace[2 * 3 * 16 * 8];
#define FT_BTRACE(kern, role, it, pt)                                                              \
  do {                                                                                             \
    if (blockIdx.x == 0 && lane == 0 && (it) < 16)                                                 \
      g_attn_bwd_trace[(((kern) * 3 + (role)) * 16 + (it)) * 8 + (pt)] = clock64();                \
  } while (0)
#else
#define FT_BTRACE(kern, role, it, pt) do { } while (0)
#endif

template <int HD>
struct DkvCfg {
  static constexpr int TILE = (HD / 64) * AT_REGION;
  // head_dim 64 leaves 128 TMEM columns free: P^T and dS^T (packed bf16, 64 columns each) are
  // written there by the threads that own their rows, and the dV / dK products read their A
  // operand from tensor memory, so neither tile crosses shared memory (which a 128-row CTA tile
  // already saturates with its B operands).  head_dim 128 fills all 512 columns with
  // accumulators and stages both tiles in shared memory.
  static constexpr bool TS = (HD == 64);
  static constexpr int STAGES = (HD == 64) ? 4 : 1;          // Q / dO ring
  static constexpr int NBUF = 1;                             // P^T / dS^T buffers
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;                     // [STAGES]
  static constexpr int OFF_DO = OFF_Q + STAGES * TILE;       // [STAGES]
  static constexpr int OFF_PT = OFF_DO + STAGES * TILE;      // [NBUF] P^T  [keys x queries]
  static constexpr int OFF_DST = OFF_PT + (TS ? 0 : NBUF * 2 * AT_REGION);   // [NBUF] dS^T
  static constexpr int OFF_STAT = OFF_DST + (TS ? 0 : NBUF * 2 * AT_REGION); // [STAGES][2][128] floats
  static constexpr int OFF_BAR = OFF_STAT + STAGES * 2 * 128 * 4;
  static constexpr int SMEM = OFF_BAR + 512;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_ST = 0, TM_DPT = 128, TM_DV = 256, TM_DK = 256 + HD;
  static constexpr int TM_PT = 256 + 2 * HD, TM_DST = 256 + 2 * HD + 64;   // TS only
};

template <int HD>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const AttnArgs p) {
  using C = DkvCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;    // [4]
  uint64_t* qdo_empty = bars + 5;   // [4]
  uint64_t* st_full = bars + 9;     // S^T and dP^T in TMEM
  uint64_t* st_free = bars + 10;    // both copied to registers (one arrival per warp)
  uint64_t* pds_ready = bars + 11;  // [2] P^T and dS^T handed to the tensor core (one arrival per warp)
  uint64_t* acc_done = bars + 13;   // [2] dV/dK MMAs that read the buffer finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, FT_ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&pds_ready[i], BW_MATH);
      mbar_init(&acc_done[i], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(st_free, BW_MATH);
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == BW_WARP_MMA) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // linear grid, key blocks with the most query blocks (the early ones under a causal mask) first
  const int n_hb = p.H * p.B;
  const int kb = (int)blockIdx.x / n_hb;
  const int hb = (int)blockIdx.x % n_hb;
  const int h = hb % p.H, b = hb / p.H;
  const int k0 = kb * AT_T;
  const int nq_all = (p.S + AT_T - 1) / AT_T;
  const int qb_first = p.causal ? kb : 0;
  const int nit = nq_all - qb_first;
  float* stat = reinterpret_cast<float*>(smem + C::OFF_STAT);

  if (warp == BW_WARP_TMA) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_arrive_expect_tx(kv_full, 2 * C::TILE);
      load_tile<HD>(smem + C::OFF_K, &tmK, kv_full, k0, h, b);
      load_tile<HD>(smem + C::OFF_V, &tmV, kv_full, k0, h, b);
    }
    // Per-query statistics (-lse and delta) of a block travel with its Q / dO tiles: they are
    // fetched into registers one iteration ahead, so their global-memory latency is spent while
    // this warp waits for the stage, not between the stage becoming free and its TMA loads.
    const long long sbase = ((long long)b * p.H + h) * p.S;
    float nl_r[4], dl_r[4];
    auto fetch_stats = [&](int it) {
      const int q0 = (qb_first + it) * AT_T;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int gq = q0 + lane + 32 * u;
        nl_r[u] = gq < p.S ? -p.lse[sbase + gq] : -INFINITY;
        dl_r[u] = gq < p.S ? p.delta[sbase + gq] : 0.f;
      }
    };
    if (nit > 0) fetch_stats(0);
    for (int it = 0; it < nit; ++it) {
      const int st = it % C::STAGES;
      const uint32_t ph = (it / C::STAGES) & 1;
      if (!mbar_wait(&qdo_empty[st], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) break;
      const int q0 = (qb_first + it) * AT_T;
      float* sl = stat + st * 256;          // published by the arrive below
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        sl[lane + 32 * u] = nl_r[u];
        sl[128 + lane + 32 * u] = dl_r[u];
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(&qdo_full[st], 2 * C::TILE);
        load_tile<HD>(smem + C::OFF_Q + st * C::TILE, &tmQ, &qdo_full[st], q0, h, b);
        load_tile<HD>(smem + C::OFF_DO + st * C::TILE, &tmDO, &qdo_full[st], q0, h, b);
      }
      __syncwarp();
      if (it + 1 < nit) fetch_stats(it + 1);
    }
  } else if (warp == BW_WARP_MMA) {
    // ---------------------------------------------------------- issuer 1: S^T = K Q^T, dP^T = V dO^T
    // (two issuing warps: the issuing thread runs in step with the tensor pipe, so the waits and
    // descriptor steps of one product would otherwise idle the pipe for the other)
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t k_addr = smem_u32(smem + C::OFF_K), v_addr = smem_u32(smem + C::OFF_V);
    const uint32_t q_addr = smem_u32(smem + C::OFF_Q), do_addr = smem_u32(smem + C::OFF_DO);
    bool ok = mbar_wait(kv_full, 0, ctx, FT_ERR_WAIT_FULL);
    for (int i = 0; ok && i < nit; ++i) {
      const int st = i % C::STAGES;
      FT_BTRACE(0, 2, i, 0);
      // needs Q_i / dO_i and the score tiles of iteration i - 1 copied to registers
      if (!mbar_wait(&qdo_full[st], (i / C::STAGES) & 1, ctx, FT_ERR_WAIT_FULL)) break;
      if (i > 0 && !mbar_wait(st_free, (i - 1) & 1, ctx, FT_ERR_WAIT_TMEM_EMPTY)) break;
      FT_BTRACE(0, 2, i, 1);
      tc_fence_after();
      if (lane == 0) {
        mma_kmajor<HD>(tmem_base + C::TM_ST, k_addr, q_addr + st * C::TILE, idesc_s);
        mma_kmajor<HD>(tmem_base + C::TM_DPT, v_addr, do_addr + st * C::TILE, idesc_s);
        umma_commit(st_full);
      }
      __syncwarp();
      FT_BTRACE(0, 2, i, 2);
    }
  } else if (warp == BW_WARP_MMA2) {
    // ---------------------------------------------------------- issuer 2: dV += P^T dO, dK += dS^T Q
    const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + C::OFF_Q), do_addr = smem_u32(smem + C::OFF_DO);
    const uint32_t pt_addr = smem_u32(smem + C::OFF_PT), dst_addr = smem_u32(smem + C::OFF_DST);
    for (int it = 0; it < nit; ++it) {
      const int st = it % C::STAGES, buf = it % C::NBUF;
      if (!mbar_wait(&qdo_full[st], (it / C::STAGES) & 1, ctx, FT_ERR_WAIT_FULL)) break;
      FT_BTRACE(0, 2, it, 3);
      if (!mbar_wait(&pds_ready[buf], (it / C::NBUF) & 1, ctx, FT_ERR_WAIT_SOFTMAX)) break;
      FT_BTRACE(0, 2, it, 4);
      tc_fence_after();
      if (lane == 0) {
        if constexpr (C::TS) {
          mma_ptmem_times_rows(tmem_base + C::TM_DV, tmem_base + C::TM_PT, do_addr + st * C::TILE,
                               idesc_acc, it > 0);
          mma_ptmem_times_rows(tmem_base + C::TM_DK, tmem_base + C::TM_DST, q_addr + st * C::TILE,
                               idesc_acc, it > 0);
        } else {
          mma_p_times_rows(tmem_base + C::TM_DV, pt_addr + buf * 2 * AT_REGION, do_addr + st * C::TILE,
                           idesc_acc, it > 0);
          mma_p_times_rows(tmem_base + C::TM_DK, dst_addr + buf * 2 * AT_REGION, q_addr + st * C::TILE,
                           idesc_acc, it > 0);
        }
        umma_commit(&acc_done[buf]);
        umma_commit(&qdo_empty[st]);     // S^T / dP^T of this stage finished before the math ran
      }
      __syncwarp();
      FT_BTRACE(0, 2, it, 5);
    }
  } else if (warp < BW_MATH) {
    const int g = warp >> 2;               // column group: queries [32 g, 32 g + 32) of the block
    const int qd = warp & 3;
    const int row = qd * 32 + lane;        // key row of this thread
    const int gk = k0 + row;
    const int c0 = 32 * g;
    const uint32_t lane_sel = (uint32_t)(qd * 32) << 16;
    bool ok = true;
    for (int it = 0; it < nit; ++it) {
      const int st = it % C::STAGES, buf = it % C::NBUF;
      const int q0 = (qb_first + it) * AT_T;
      // statistics were written by the producer before its arrive on qdo_full
      FT_BTRACE(0, warp == 0 ? 0 : 1, it, 0);
      if (!mbar_wait(&qdo_full[st], (it / C::STAGES) & 1, ctx, FT_ERR_WAIT_FULL)) { ok = false; break; }
      if (!mbar_wait(st_full, it & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      FT_BTRACE(0, warp == 0 ? 0 : 1, it, 1);
      tc_fence_after();
      uint32_t rs[32], rd[32];
      tmem_ld32(tmem_base + C::TM_ST + c0 + lane_sel, rs);
      tmem_ld32(tmem_base + C::TM_DPT + c0 + lane_sel, rd);
      tmem_ld_wait();
      FT_BTRACE(0, warp == 0 ? 0 : 1, it, 2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(st_free);      // one arrival per warp
      const float4* sl4 = reinterpret_cast<const float4*>(stat + st * 256 + c0);
      const float4* dl4 = reinterpret_cast<const float4*>(stat + st * 256 + 128 + c0);
      const bool need_mask = (q0 + AT_T > p.S) || (k0 + AT_T > p.S) || (p.causal && q0 < k0 + AT_T - 1);
      uint32_t pw[16], dw[16];
      // masked scores become -inf in a pass of their own (diagonal and ragged blocks only), so
      // the main loop carries no per-element predicates
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int gq = q0 + c0 + i;
          if (gq >= p.S || gk >= p.S || (p.causal && gk > gq)) rs[i] = __float_as_uint(-INFINITY);
        }
      }
#pragma unroll
      for (int i4 = 0; i4 < 8; ++i4) {
        const float4 nl = sl4[i4], dl = dl4[i4];
        const float nls[4] = {nl.x, nl.y, nl.z, nl.w}, dls[4] = {dl.x, dl.y, dl.z, dl.w};
        float e[4], d[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = 4 * i4 + u;
          e[u] = fast_exp2(fmaf(__uint_as_float(rs[i]), p.sl2, nls[u]));
          d[u] = e[u] * (__uint_as_float(rd[i]) - dls[u]);
        }
        pw[2 * i4] = pack_bf16(e[0], e[1]);
        pw[2 * i4 + 1] = pack_bf16(e[2], e[3]);
        dw[2 * i4] = pack_bf16(d[0], d[1]);
        dw[2 * i4 + 1] = pack_bf16(d[2], d[3]);
      }
      FT_BTRACE(0, warp == 0 ? 0 : 1, it, 3);
      // the buffer's previous reader (dV/dK of iteration it - NBUF) must have finished
      if (it >= C::NBUF &&
          !mbar_wait(&acc_done[buf], ((it / C::NBUF) - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      FT_BTRACE(0, warp == 0 ? 0 : 1, it, 4);
      if constexpr (C::TS) {
        // this thread's 32 queries of its key row: 16 packed columns of each operand tile
        tc_fence_after();
        tmem_st16(tmem_base + C::TM_PT + 16 * g + lane_sel, pw);
        tmem_st16(tmem_base + C::TM_DST + 16 * g + lane_sel, dw);
        tmem_st_wait();
        tc_fence_before();
      } else {
        store_row32_packed(smem + C::OFF_PT + buf * 2 * AT_REGION, row, c0, pw);
        store_row32_packed(smem + C::OFF_DST + buf * 2 * AT_REGION, row, c0, dw);
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_ready[buf]);      // one arrival per warp
      FT_BTRACE(0, warp == 0 ? 0 : 1, it, 5);
    }
    if (ok && nit > 0)
      ok = mbar_wait(&acc_done[(nit - 1) % C::NBUF], ((nit - 1) / C::NBUF) & 1, ctx, FT_ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dvp = p.dv + (long long)b * p.dv_bs + (long long)gk * p.dv_ss + (long long)h * p.dv_hs;
      __nv_bfloat16* dkp = p.dk + (long long)b * p.dk_bs + (long long)gk * p.dk_ss + (long long)h * p.dk_hs;
      // 2 HD / 32 column chunks (dV first, then dK) spread over the four groups
#pragma unroll
      for (int ch = g; ch < 2 * HD / 32; ch += 4) {
        const bool is_dk = ch >= HD / 32;
        const int c = (is_dk ? ch - HD / 32 : ch) * 32;
        uint32_t r[32];
        if (nit > 0) {
          tmem_ld32(tmem_base + (is_dk ? C::TM_DK : C::TM_DV) + c + lane_sel, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (gk < p.S) store_out32((is_dk ? dkp : dvp) + c, r, is_dk ? p.scale : 1.f);
      }
      tc_fence_before();
    }
  }

  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BW_WARP_MMA) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// =============================================================================== backward: dQ
template <int HD>
struct DqCfg {
  static constexpr int TILE = (HD / 64) * AT_REGION;
  static constexpr bool TS = (HD == 64);                 // dS in tensor memory (see DkvCfg)
  static constexpr int STAGES = (HD == 64) ? 4 : 2;      // K / V ring
  static constexpr int NBUF = (HD == 64) ? 2 : 1;        // dS buffers
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;                 // [STAGES]
  static constexpr int OFF_V = OFF_K + STAGES * TILE;    // [STAGES]
  static constexpr int OFF_DS = OFF_V + STAGES * TILE;   // [NBUF] dS [queries x keys]
  static constexpr int OFF_BAR = OFF_DS + (TS ? 0 : NBUF * 2 * AT_REGION);
  static constexpr int SMEM = OFF_BAR + 512;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_DP = 128, TM_DQ = 256;
  static constexpr int TM_DS = 384;                      // TS: dS buffer i at TM_DS + 64 i
};

template <int HD>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const AttnArgs p) {
  using C = DqCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;    // [4]
  uint64_t* kv_empty = bars + 5;   // [4]
  uint64_t* s_full = bars + 9;     // S and dP in TMEM
  uint64_t* s_free = bars + 10;    // both copied to registers (one arrival per warp)
  uint64_t* ds_ready = bars + 11;  // [2] dS handed to the tensor core (one arrival per warp)
  uint64_t* acc_done = bars + 13;  // [2] dQ MMA that read the buffer finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, FT_ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ds_ready[i], BW_MATH);
      mbar_init(&acc_done[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, BW_MATH);
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == BW_WARP_MMA) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // linear grid, query blocks with the most key blocks (the late ones under a causal mask) first
  const int n_hb = p.H * p.B;
  const int qb = (int)gridDim.x / n_hb - 1 - (int)blockIdx.x / n_hb;
  const int hb = (int)blockIdx.x % n_hb;
  const int h = hb % p.H, b = hb / p.H;
  const int q0 = qb * AT_T;
  const int nkv_all = (p.S + AT_T - 1) / AT_T;
  const int nkv = p.causal ? min(qb + 1, nkv_all) : nkv_all;

  if (warp == BW_WARP_TMA) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_arrive_expect_tx(qdo_full, 2 * C::TILE);
      load_tile<HD>(smem + C::OFF_Q, &tmQ, qdo_full, q0, h, b);
      load_tile<HD>(smem + C::OFF_DO, &tmDO, qdo_full, q0, h, b);
    }
    for (int j = 0; j < nkv; ++j) {
      const int st = j % C::STAGES;
      const uint32_t ph = (j / C::STAGES) & 1;
      if (!mbar_wait(&kv_empty[st], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&kv_full[st], 2 * C::TILE);
        load_tile<HD>(smem + C::OFF_K + st * C::TILE, &tmK, &kv_full[st], j * AT_T, h, b);
        load_tile<HD>(smem + C::OFF_V + st * C::TILE, &tmV, &kv_full[st], j * AT_T, h, b);
      }
      __syncwarp();
    }
  } else if (warp == BW_WARP_MMA) {
    // ---------------------------------------------------------- issuer 1: S = Q K^T, dP = dO V^T
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t q_addr = smem_u32(smem + C::OFF_Q), do_addr = smem_u32(smem + C::OFF_DO);
    const uint32_t k_addr = smem_u32(smem + C::OFF_K), v_addr = smem_u32(smem + C::OFF_V);
    bool ok = mbar_wait(qdo_full, 0, ctx, FT_ERR_WAIT_FULL);
    for (int jj = 0; ok && jj < nkv; ++jj) {
      const int st = jj % C::STAGES;
      FT_BTRACE(1, 2, jj, 0);
      if (!mbar_wait(&kv_full[st], (jj / C::STAGES) & 1, ctx, FT_ERR_WAIT_FULL)) break;
      if (jj > 0 && !mbar_wait(s_free, (jj - 1) & 1, ctx, FT_ERR_WAIT_TMEM_EMPTY)) break;
      FT_BTRACE(1, 2, jj, 1);
      tc_fence_after();
      if (lane == 0) {
        mma_kmajor<HD>(tmem_base + C::TM_S, q_addr, k_addr + st * C::TILE, idesc_s);
        mma_kmajor<HD>(tmem_base + C::TM_DP, do_addr, v_addr + st * C::TILE, idesc_s);
        umma_commit(s_full);
      }
      __syncwarp();
      FT_BTRACE(1, 2, jj, 2);
    }
  } else if (warp == BW_WARP_MMA2) {
    // ---------------------------------------------------------- issuer 2: dQ += dS K
    const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);
    const uint32_t k_addr = smem_u32(smem + C::OFF_K);
    const uint32_t ds_addr = smem_u32(smem + C::OFF_DS);
    for (int j = 0; j < nkv; ++j) {
      const int st = j % C::STAGES, buf = j % C::NBUF;
      if (!mbar_wait(&kv_full[st], (j / C::STAGES) & 1, ctx, FT_ERR_WAIT_FULL)) break;
      FT_BTRACE(1, 2, j, 3);
      if (!mbar_wait(&ds_ready[buf], (j / C::NBUF) & 1, ctx, FT_ERR_WAIT_SOFTMAX)) break;
      FT_BTRACE(1, 2, j, 4);
      tc_fence_after();
      if (lane == 0) {
        if constexpr (C::TS)
          mma_ptmem_times_rows(tmem_base + C::TM_DQ, tmem_base + C::TM_DS + 64 * buf, k_addr + st * C::TILE,
                               idesc_acc, j > 0);
        else
          mma_p_times_rows(tmem_base + C::TM_DQ, ds_addr + buf * 2 * AT_REGION, k_addr + st * C::TILE,
                           idesc_acc, j > 0);
        umma_commit(&acc_done[buf]);
        umma_commit(&kv_empty[st]);      // S / dP of this stage finished before the math ran
      }
      __syncwarp();
      FT_BTRACE(1, 2, j, 5);
    }
  } else if (warp < BW_MATH) {
    const int g = warp >> 2;               // column group: keys [32 g, 32 g + 32) of the block
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const int c0 = 32 * g;
    const uint32_t lane_sel = (uint32_t)(qd * 32) << 16;
    const long long sbase = ((long long)b * p.H + h) * p.S;
    const float nlse = grow < p.S ? -p.lse[sbase + grow] : -INFINITY;
    const float dl = grow < p.S ? p.delta[sbase + grow] : 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      const int buf = j % C::NBUF;
      FT_BTRACE(1, warp == 0 ? 0 : 1, j, 0);
      if (!mbar_wait(s_full, j & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      FT_BTRACE(1, warp == 0 ? 0 : 1, j, 1);
      tc_fence_after();
      uint32_t rs[32], rd[32];
      tmem_ld32(tmem_base + C::TM_S + c0 + lane_sel, rs);
      tmem_ld32(tmem_base + C::TM_DP + c0 + lane_sel, rd);
      tmem_ld_wait();
      FT_BTRACE(1, warp == 0 ? 0 : 1, j, 2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);      // one arrival per warp
      const int k0 = j * AT_T;
      const bool need_mask = (k0 + AT_T > p.S) || (q0 + AT_T > p.S) || (p.causal && k0 + AT_T - 1 > q0);
      uint32_t dw[16];
      if (need_mask) {      // masked scores become -inf in a pass of their own
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kc = k0 + c0 + i;
          if (kc >= p.S || grow >= p.S || (p.causal && kc > grow)) rs[i] = __float_as_uint(-INFINITY);
        }
      }
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float e0 = fast_exp2(fmaf(__uint_as_float(rs[i]), p.sl2, nlse));
        const float e1 = fast_exp2(fmaf(__uint_as_float(rs[i + 1]), p.sl2, nlse));
        dw[i >> 1] = pack_bf16(e0 * (__uint_as_float(rd[i]) - dl), e1 * (__uint_as_float(rd[i + 1]) - dl));
      }
      FT_BTRACE(1, warp == 0 ? 0 : 1, j, 3);
      if (j >= C::NBUF &&
          !mbar_wait(&acc_done[buf], ((j / C::NBUF) - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      FT_BTRACE(1, warp == 0 ? 0 : 1, j, 4);
      if constexpr (C::TS) {
        tc_fence_after();
        tmem_st16(tmem_base + C::TM_DS + 64 * buf + 16 * g + lane_sel, dw);
        tmem_st_wait();
        tc_fence_before();
      } else {
        store_row32_packed(smem + C::OFF_DS + buf * 2 * AT_REGION, row, c0, dw);
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready[buf]);      // one arrival per warp
      FT_BTRACE(1, warp == 0 ? 0 : 1, j, 5);
    }
    if (ok && nkv > 0)
      ok = mbar_wait(&acc_done[(nkv - 1) % C::NBUF], ((nkv - 1) / C::NBUF) & 1, ctx, FT_ERR_WAIT_TMEM_FULL);
    if (ok && nkv > 0) {
      tc_fence_after();
      __nv_bfloat16* dqp = p.dq + (long long)b * p.dq_bs + (long long)grow * p.dq_ss + (long long)h * p.dq_hs;
#pragma unroll
      for (int ch = g; ch < HD / 32; ch += 4) {
        uint32_t r[32];
        tmem_ld32(tmem_base + C::TM_DQ + ch * 32 + lane_sel, r);
        tmem_ld_wait();
        if (grow < p.S) store_out32(dqp + ch * 32, r, p.scale);
      }
      tc_fence_before();
    }
  }

  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BW_WARP_MMA) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int HD>
static int attn_bwd_launch(const FtkAttnDesc* a, cudaStream_t s) {
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_map(&tq, a->q, a, a->q_bs, a->q_ss, a->q_hs))) return rc;
  if ((rc = make_map(&tk, a->k, a, a->k_bs, a->k_ss, a->k_hs))) return rc;
  if ((rc = make_map(&tv, a->v, a, a->v_bs, a->v_ss, a->v_hs))) return rc;
  if ((rc = make_map(&tdo, a->d_o, a, a->o_bs, a->o_ss, a->o_hs))) return rc;
  AttnArgs p;
  fill_args(p, a);
  if (!p.status) return -6;
  static bool attr = false;
  if (!attr) {
    if ((rc = set_smem(attn_bwd_dkv_kernel<HD>, DkvCfg<HD>::SMEM))) return rc;
    if ((rc = set_smem(attn_bwd_dq_kernel<HD>, DqCfg<HD>::SMEM))) return rc;
    attr = true;
  }
  const long long nrows = (long long)a->B * a->S * a->H;
  constexpr int LPR = HD / 8, ROWS_PER_CTA = 8 * (32 / LPR);
  attn_delta_kernel<LPR><<<(unsigned)((nrows + ROWS_PER_CTA - 1) / ROWS_PER_CTA), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(a->o), reinterpret_cast<const __nv_bfloat16*>(a->d_o),
      a->delta, a->B, a->H, a->S, a->o_bs, a->o_ss, a->o_hs);
  dim3 grid((unsigned)(((a->S + AT_T - 1) / AT_T) * a->H * a->B));
  attn_bwd_dkv_kernel<HD><<<grid, BW_THREADS, DkvCfg<HD>::SMEM, s>>>(tq, tk, tv, tdo, p);
  attn_bwd_dq_kernel<HD><<<grid, BW_THREADS, DqCfg<HD>::SMEM, s>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}

}  // namespace ftk

using namespace ftk;

#ifdef FT_ATTN_TRACE
extern "C" int ftk_attn_bwd_trace_read(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_attn_bwd_trace, sizeof(long long) * n);
}
#endif

extern "C" int ftk_attn_bwd(const FtkAttnDesc* a, void* stream) {
  if (!a || a->B <= 0 || a->H <= 0 || a->S <= 0 || !a->delta || !a->lse) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->hd == 64) return attn_bwd_launch<64>(a, s);
  if (a->hd == 128) return attn_bwd_launch<128>(a, s);
  return -5;
}
