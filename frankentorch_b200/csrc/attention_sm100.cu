// Flash attention for sm_100a on tcgen05/TMEM, forward and backward, head_dim 64/128.
//
// Semantics (reference: ft-kernel-cpu/src/lib.rs:4572 sdpa_forward_f64, :5300
// sdpa_backward_f64; Metal attn_flash2, ft-kernel-metal/src/fused.rs:407): blockwise
// QK^T -> stable online softmax -> PV with scores never materialised in HBM; causal
// masks j > i; backward recomputes P from the saved log-sum-exp:
//   dV = P^T dO, dP = dO V^T, dS = P o (dP - rowsum(dO o O)), dQ = scale dS K,
//   dK = scale dS^T Q.
//
// Layout: Q/K/V/O/dO are addressed in place inside the packed [B*S, 3*d] / [B*S, d]
// activations through 4-D TMA maps {head_dim, S, H, B}; no head split/merge copies.
//
// Structure of every kernel: warp 0 = TMA producer, warp 1 = MMA issuer (owns
// TMEM), warps 2..5 = one thread per tile row doing the softmax math on values
// read with tcgen05.ld.  Probabilities go back to the tensor core through a
// 128B-swizzled bf16 tile in shared memory.
//
// Determinism: dK/dV are accumulated in TMEM by the CTA that owns the key block,
// dQ by the CTA that owns the query block (second kernel), both in ascending block
// order; there are no atomics, so gradients are bit-identical run to run.
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

int ftk_make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t l0, uint64_t l1, uint64_t ld_elems, uint64_t s0_elems,
                       uint64_t s1_elems, uint32_t box_inner, uint32_t box_outer);

constexpr int AT_T = 128;           // tile rows (queries) == tile keys
constexpr int AT_THREADS = 192;
constexpr int AT_REGION = 16384;    // one [128 rows x 64 bf16] swizzled region

struct AttnArgs {
  int B, H, S;
  int causal;
  float sl2;    // scale * log2(e)
  float scale;
  __nv_bfloat16* o;
  long long o_bs, o_ss, o_hs;
  float* lse;
  const float* delta;
  __nv_bfloat16 *dq, *dk, *dv;
  long long dq_bs, dq_ss, dq_hs, dk_bs, dk_ss, dk_hs, dv_bs, dv_ss, dv_hs;
  int* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A (K-major) x B (K-major)^T with K = HD, operands stored as HD/64 regions.
template <int HD>
__device__ __forceinline__ void mma_kmajor(uint32_t d_tmem, uint32_t a_base, uint32_t b_base,
                                           uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const uint32_t off = (kk >> 2) * AT_REGION + (kk & 3) * 32;
    umma_bf16(d_tmem, make_smem_desc(a_base + off, 16, 1024), make_smem_desc(b_base + off, 16, 1024),
              idesc, kk != 0 ? 1u : 0u);
  }
}
// A = probabilities [128 x 128] K-major in two regions; B = [128 k-rows x HD] stored
// row-major per 64-column region (MN-major operand), K = 128.
__device__ __forceinline__ void mma_p_times_rows(uint32_t d_tmem, uint32_t p_base, uint32_t b_base,
                                                 uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < AT_T / 16; ++kk) {
    const uint32_t a_off = (kk >> 2) * AT_REGION + (kk & 3) * 32;
    umma_bf16(d_tmem, make_smem_desc(p_base + a_off, 16, 1024),
              make_smem_desc(b_base + kk * 2048, AT_REGION, 1024), idesc,
              (accumulate || kk != 0) ? 1u : 0u);
  }
}
// Write 32 fp32 values of one tile row as bf16 into the swizzled K-major tile.
__device__ __forceinline__ void store_row32_swizzled(uint8_t* tile, int row, int col0,
                                                     const float* v) {
  uint8_t* base = tile + (col0 >> 6) * AT_REGION + row * 128;
  const int j0 = (col0 & 63) >> 3;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint4 u;
    u.x = pack_bf16(v[8 * t + 0], v[8 * t + 1]);
    u.y = pack_bf16(v[8 * t + 2], v[8 * t + 3]);
    u.z = pack_bf16(v[8 * t + 4], v[8 * t + 5]);
    u.w = pack_bf16(v[8 * t + 6], v[8 * t + 7]);
    *reinterpret_cast<uint4*>(base + (((j0 + t) ^ (row & 7)) << 4)) = u;
  }
}
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar,
                                          int row0, int h, int b) {
#pragma unroll
  for (int c = 0; c < HD / 64; ++c) tma_load_4d(dst + c * AT_REGION, tm, bar, c * 64, row0, h, b);
}

// =============================================================================== forward
template <int HD>
struct FwdCfg {
  static constexpr int TILE = (HD / 64) * AT_REGION;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = TILE;
  static constexpr int OFF_V = OFF_K + 2 * TILE;
  static constexpr int OFF_P = OFF_V + 2 * TILE;
  static constexpr int OFF_BAR = OFF_P + 2 * AT_REGION;
  static constexpr int SMEM = OFF_BAR + 1024;
  static constexpr int TMEM_COLS = 256;
  static constexpr int TM_S = 0, TM_PV = 128;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, (HD == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  using C = FwdCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* pv_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  if ((smem_u32(smem) & 1023u) != 0u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, FT_ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(pv_full, 1);
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // heavy (late) query blocks first
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * AT_T;
  const int nkv_all = (p.S + AT_T - 1) / AT_T;
  const int nkv = p.causal ? min(qb + 1, nkv_all) : nkv_all;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, C::TILE);
      load_tile<HD>(smem + C::OFF_Q, &tmQ, q_full, q0, h, b);
    }
    for (int j = 0; j < nkv; ++j) {
      const int st = j & 1;
      if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&kv_full[st], 2 * C::TILE);
        load_tile<HD>(smem + C::OFF_K + st * C::TILE, &tmK, &kv_full[st], j * AT_T, h, b);
        load_tile<HD>(smem + C::OFF_V + st * C::TILE, &tmV, &kv_full[st], j * AT_T, h, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_pv = make_idesc_bf16(128, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + C::OFF_Q);
    const uint32_t p_addr = smem_u32(smem + C::OFF_P);
    bool ok = mbar_wait(q_full, 0, ctx, FT_ERR_WAIT_FULL);
    ok = ok && mbar_wait(&kv_full[0], 0, ctx, FT_ERR_WAIT_FULL);
    if (ok) {
      tc_fence_after();
      if (lane == 0) {
        mma_kmajor<HD>(tmem_base + C::TM_S, q_addr, smem_u32(smem + C::OFF_K), idesc_s);
        umma_commit(s_full);
      }
      __syncwarp();
      for (int j = 0; j < nkv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(p_ready, j & 1, ctx, FT_ERR_WAIT_SOFTMAX)) break;
        tc_fence_after();
        if (lane == 0) {
          mma_p_times_rows(tmem_base + C::TM_PV, p_addr, smem_u32(smem + C::OFF_V + st * C::TILE),
                           idesc_pv, false);
          umma_commit(pv_full);
          umma_commit(&kv_empty[st]);
        }
        __syncwarp();
        if (j + 1 < nkv) {
          const int sn = (j + 1) & 1;
          if (!mbar_wait(&kv_full[sn], ((j + 1) >> 1) & 1, ctx, FT_ERR_WAIT_FULL)) break;
          tc_fence_after();
          if (lane == 0) {
            mma_kmajor<HD>(tmem_base + C::TM_S, q_addr, smem_u32(smem + C::OFF_K + sn * C::TILE),
                           idesc_s);
            umma_commit(s_full);
          }
          __syncwarp();
        }
      }
    }
  } else {
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const uint32_t lane_sel = (uint32_t)(qd * 32) << 16;
    float m = -INFINITY, l = 0.f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    uint8_t* sP = smem + C::OFF_P;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * AT_T;
      const bool need_mask = (k0 + AT_T > p.S) || (p.causal && k0 + AT_T - 1 > q0);
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < AT_T; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + C::TM_S + c + lane_sel, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(r[i]);
          if (need_mask) {
            const int kc = k0 + c + i;
            if (kc >= p.S || (p.causal && kc > grow)) s = -INFINITY;
          }
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2((m - m_use) * p.sl2);
      const float moff = m_use * p.sl2;
      // The previous P tile is free: its PV MMA completed before the pv_full wait that
      // ended iteration j-1.
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < AT_T; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + C::TM_S + c + lane_sel, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(r[i]);
          float e = fast_exp2(s * p.sl2 - moff);
          if (need_mask) {
            const int kc = k0 + c + i;
            if (kc >= p.S || (p.causal && kc > grow)) e = 0.f;
          }
          pv[i] = e;
          rs += e;
        }
        store_row32_swizzled(sP, row, c, pv);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      l = l * alpha + rs;
      m = m_new;
      // accumulate this block's PV
      if (!mbar_wait(pv_full, j & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + C::TM_PV + c + lane_sel, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before();
    }
    if (ok && grow < p.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = p.o + (long long)b * p.o_bs + (long long)grow * p.o_ss + (long long)h * p.o_hs;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        uint4 u;
        u.x = pack_bf16(o[c + 0] * inv, o[c + 1] * inv);
        u.y = pack_bf16(o[c + 2] * inv, o[c + 3] * inv);
        u.z = pack_bf16(o[c + 4] * inv, o[c + 5] * inv);
        u.w = pack_bf16(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(op + c) = u;
      }
      if (p.lse)
        p.lse[((long long)b * p.H + h) * p.S + grow] =
            (l > 0.f) ? (m == -INFINITY ? 0.f : m) * p.sl2 + log2f(l) : -INFINITY;
    }
  }

  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// =============================================================================== delta
// delta[b,h,s] = sum_e dO * O ; one warp per (b, s, h) row.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                  float* __restrict__ delta, int B, int H, int S, int hd, long long bs,
                  long long ss, long long hs) {
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * S * H) return;
  const int h = (int)(w % H);
  const long long t = w / H;
  const int s = (int)(t % S);
  const int b = (int)(t / S);
  const long long off = (long long)b * bs + (long long)s * ss + (long long)h * hs;
  float acc = 0.f;
  if (lane * 8 < hd) {
    uint4 a = *reinterpret_cast<const uint4*>(o + off + lane * 8);
    uint4 g = *reinterpret_cast<const uint4*>(d_o + off + lane * 8);
    float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
    float2 g0 = unpack_bf16(g.x), g1 = unpack_bf16(g.y), g2 = unpack_bf16(g.z), g3 = unpack_bf16(g.w);
    acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y +
          a3.x * g3.x + a3.y * g3.y;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) delta[((long long)b * H + h) * S + s] = acc;
}

// =============================================================================== backward: dK, dV
template <int HD>
struct DkvCfg {
  static constexpr int TILE = (HD / 64) * AT_REGION;
  static constexpr int STAGES = (HD == 64) ? 2 : 1;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;                    // [STAGES]
  static constexpr int OFF_DO = OFF_Q + STAGES * TILE;      // [STAGES]
  static constexpr int OFF_PT = OFF_DO + STAGES * TILE;     // P^T  [keys x queries]
  static constexpr int OFF_DST = OFF_PT + 2 * AT_REGION;    // dS^T [keys x queries]
  static constexpr int OFF_STAT = OFF_DST + 2 * AT_REGION;  // [STAGES][2][128] floats
  static constexpr int OFF_BAR = OFF_STAT + STAGES * 2 * 128 * 4;
  static constexpr int SMEM = OFF_BAR + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_ST = 0, TM_DPT = 128, TM_DV = 256, TM_DK = 256 + HD;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const AttnArgs p) {
  using C = DkvCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* st_full = bars + 5;     // S^T and dP^T computed
  uint64_t* pds_ready = bars + 6;   // P^T and dS^T written to smem (128 arrivals)
  uint64_t* acc_done = bars + 7;    // dV/dK MMAs that read P^T/dS^T finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, FT_ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(pds_ready, 128);
    mbar_init(acc_done, 1);
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kb * AT_T;
  const int nq_all = (p.S + AT_T - 1) / AT_T;
  const int qb_first = p.causal ? kb : 0;
  const int nit = nq_all - qb_first;
  float* stat = reinterpret_cast<float*>(smem + C::OFF_STAT);

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_arrive_expect_tx(kv_full, 2 * C::TILE);
      load_tile<HD>(smem + C::OFF_K, &tmK, kv_full, k0, h, b);
      load_tile<HD>(smem + C::OFF_V, &tmV, kv_full, k0, h, b);
    }
    for (int it = 0; it < nit; ++it) {
      const int st = it % C::STAGES;
      const uint32_t ph = (it / C::STAGES) & 1;
      if (!mbar_wait(&qdo_empty[st], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) break;
      const int q0 = (qb_first + it) * AT_T;
      // per-query statistics for this block (plain loads, published by the arrive below)
      float* sl = stat + st * 256;
      const long long sbase = ((long long)b * p.H + h) * p.S;
      for (int i = lane; i < AT_T; i += 32) {
        const int gq = q0 + i;
        sl[i] = gq < p.S ? p.lse[sbase + gq] : INFINITY;
        sl[128 + i] = gq < p.S ? p.delta[sbase + gq] : 0.f;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_expect_tx(&qdo_full[st], 2 * C::TILE);
        load_tile<HD>(smem + C::OFF_Q + st * C::TILE, &tmQ, &qdo_full[st], q0, h, b);
        load_tile<HD>(smem + C::OFF_DO + st * C::TILE, &tmDO, &qdo_full[st], q0, h, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);
    const uint32_t k_addr = smem_u32(smem + C::OFF_K), v_addr = smem_u32(smem + C::OFF_V);
    const uint32_t pt_addr = smem_u32(smem + C::OFF_PT), dst_addr = smem_u32(smem + C::OFF_DST);
    bool ok = mbar_wait(kv_full, 0, ctx, FT_ERR_WAIT_FULL);
    if (ok && nit > 0) {
      ok = mbar_wait(&qdo_full[0], 0, ctx, FT_ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        if (lane == 0) {
          mma_kmajor<HD>(tmem_base + C::TM_ST, k_addr, smem_u32(smem + C::OFF_Q), idesc_s);
          mma_kmajor<HD>(tmem_base + C::TM_DPT, v_addr, smem_u32(smem + C::OFF_DO), idesc_s);
          umma_commit(st_full);
        }
        __syncwarp();
      }
      for (int it = 0; ok && it < nit; ++it) {
        const int st = it % C::STAGES;
        if (!mbar_wait(pds_ready, it & 1, ctx, FT_ERR_WAIT_SOFTMAX)) break;
        tc_fence_after();
        if (lane == 0) {
          mma_p_times_rows(tmem_base + C::TM_DV, pt_addr, smem_u32(smem + C::OFF_DO + st * C::TILE),
                           idesc_acc, it > 0);
          mma_p_times_rows(tmem_base + C::TM_DK, dst_addr, smem_u32(smem + C::OFF_Q + st * C::TILE),
                           idesc_acc, it > 0);
          umma_commit(acc_done);
          umma_commit(&qdo_empty[st]);
        }
        __syncwarp();
        if (it + 1 < nit) {
          const int sn = (it + 1) % C::STAGES;
          const uint32_t phn = ((it + 1) / C::STAGES) & 1;
          if (!mbar_wait(&qdo_full[sn], phn, ctx, FT_ERR_WAIT_FULL)) break;
          tc_fence_after();
          if (lane == 0) {
            mma_kmajor<HD>(tmem_base + C::TM_ST, k_addr, smem_u32(smem + C::OFF_Q + sn * C::TILE),
                           idesc_s);
            mma_kmajor<HD>(tmem_base + C::TM_DPT, v_addr, smem_u32(smem + C::OFF_DO + sn * C::TILE),
                           idesc_s);
            umma_commit(st_full);
          }
          __syncwarp();
        }
      }
    }
  } else {
    const int qd = warp & 3;
    const int row = qd * 32 + lane;  // key row of this thread
    const int gk = k0 + row;
    const uint32_t lane_sel = (uint32_t)(qd * 32) << 16;
    uint8_t* sPT = smem + C::OFF_PT;
    uint8_t* sDST = smem + C::OFF_DST;
    bool ok = true;
    for (int it = 0; it < nit && ok; ++it) {
      const int st = it % C::STAGES;
      const uint32_t ph = (it / C::STAGES) & 1;
      const int q0 = (qb_first + it) * AT_T;
      // statistics were written by the producer before its arrive on qdo_full
      if (!mbar_wait(&qdo_full[st], ph, ctx, FT_ERR_WAIT_FULL)) { ok = false; break; }
      if (!mbar_wait(st_full, it & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      // the previous P^T / dS^T tiles must have been consumed
      if (it > 0 && !mbar_wait(acc_done, (it - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      const float* sl = stat + st * 256;
      const bool need_mask = (q0 + AT_T > p.S) || (k0 + AT_T > p.S) || (p.causal && q0 < k0 + AT_T - 1);
#pragma unroll 1
      for (int c = 0; c < AT_T; c += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem_base + C::TM_ST + c + lane_sel, rs);
        tmem_ld32(tmem_base + C::TM_DPT + c + lane_sel, rd);
        tmem_ld_wait();
        float pv[32], dv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float lse = sl[c + i], dl = sl[128 + c + i];
          float e = fast_exp2(__uint_as_float(rs[i]) * p.sl2 - lse);
          if (need_mask) {
            const int gq = q0 + c + i;
            if (gq >= p.S || gk >= p.S || (p.causal && gk > gq)) e = 0.f;
          }
          pv[i] = e;
          dv[i] = e * (__uint_as_float(rd[i]) - dl);
        }
        store_row32_swizzled(sPT, row, c, pv);
        store_row32_swizzled(sDST, row, c, dv);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_ready);
    }
    if (ok && nit > 0) ok = mbar_wait(acc_done, (nit - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dvp = p.dv + (long long)b * p.dv_bs + (long long)gk * p.dv_ss + (long long)h * p.dv_hs;
      __nv_bfloat16* dkp = p.dk + (long long)b * p.dk_bs + (long long)gk * p.dk_ss + (long long)h * p.dk_hs;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t r1[32], r2[32];
        if (nit > 0) {
          tmem_ld32(tmem_base + C::TM_DV + c + lane_sel, r1);
          tmem_ld32(tmem_base + C::TM_DK + c + lane_sel, r2);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r1[i] = r2[i] = 0u;
        }
        if (gk < p.S) {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint4 u, w;
            u.x = pack_bf16(__uint_as_float(r1[8 * t + 0]), __uint_as_float(r1[8 * t + 1]));
            u.y = pack_bf16(__uint_as_float(r1[8 * t + 2]), __uint_as_float(r1[8 * t + 3]));
            u.z = pack_bf16(__uint_as_float(r1[8 * t + 4]), __uint_as_float(r1[8 * t + 5]));
            u.w = pack_bf16(__uint_as_float(r1[8 * t + 6]), __uint_as_float(r1[8 * t + 7]));
            w.x = pack_bf16(__uint_as_float(r2[8 * t + 0]) * p.scale, __uint_as_float(r2[8 * t + 1]) * p.scale);
            w.y = pack_bf16(__uint_as_float(r2[8 * t + 2]) * p.scale, __uint_as_float(r2[8 * t + 3]) * p.scale);
            w.z = pack_bf16(__uint_as_float(r2[8 * t + 4]) * p.scale, __uint_as_float(r2[8 * t + 5]) * p.scale);
            w.w = pack_bf16(__uint_as_float(r2[8 * t + 6]) * p.scale, __uint_as_float(r2[8 * t + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dvp + c + 8 * t) = u;
            *reinterpret_cast<uint4*>(dkp + c + 8 * t) = w;
          }
        }
      }
      tc_fence_before();
    }
  }

  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// =============================================================================== backward: dQ
template <int HD>
struct DqCfg {
  static constexpr int TILE = (HD / 64) * AT_REGION;
  static constexpr int STAGES = (HD == 64) ? 2 : 1;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;                 // [STAGES]
  static constexpr int OFF_V = OFF_K + STAGES * TILE;    // [STAGES]
  static constexpr int OFF_DS = OFF_V + STAGES * TILE;   // dS [queries x keys]
  static constexpr int OFF_BAR = OFF_DS + 2 * AT_REGION;
  static constexpr int SMEM = OFF_BAR + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_DP = 128, TM_DQ = 256;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const AttnArgs p) {
  using C = DqCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* ds_ready = bars + 6;
  uint64_t* acc_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, FT_ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(ds_ready, 128);
    mbar_init(acc_done, 1);
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * AT_T;
  const int nkv_all = (p.S + AT_T - 1) / AT_T;
  const int nkv = p.causal ? min(qb + 1, nkv_all) : nkv_all;

  if (warp == 0) {
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
  } else if (warp == 1) {
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + C::OFF_Q), do_addr = smem_u32(smem + C::OFF_DO);
    const uint32_t ds_addr = smem_u32(smem + C::OFF_DS);
    bool ok = mbar_wait(qdo_full, 0, ctx, FT_ERR_WAIT_FULL);
    ok = ok && mbar_wait(&kv_full[0], 0, ctx, FT_ERR_WAIT_FULL);
    if (ok) {
      tc_fence_after();
      if (lane == 0) {
        mma_kmajor<HD>(tmem_base + C::TM_S, q_addr, smem_u32(smem + C::OFF_K), idesc_s);
        mma_kmajor<HD>(tmem_base + C::TM_DP, do_addr, smem_u32(smem + C::OFF_V), idesc_s);
        umma_commit(s_full);
      }
      __syncwarp();
      for (int j = 0; j < nkv; ++j) {
        const int st = j % C::STAGES;
        if (!mbar_wait(ds_ready, j & 1, ctx, FT_ERR_WAIT_SOFTMAX)) break;
        tc_fence_after();
        if (lane == 0) {
          mma_p_times_rows(tmem_base + C::TM_DQ, ds_addr, smem_u32(smem + C::OFF_K + st * C::TILE),
                           idesc_acc, j > 0);
          umma_commit(acc_done);
          umma_commit(&kv_empty[st]);
        }
        __syncwarp();
        if (j + 1 < nkv) {
          const int sn = (j + 1) % C::STAGES;
          const uint32_t phn = ((j + 1) / C::STAGES) & 1;
          if (!mbar_wait(&kv_full[sn], phn, ctx, FT_ERR_WAIT_FULL)) break;
          tc_fence_after();
          if (lane == 0) {
            mma_kmajor<HD>(tmem_base + C::TM_S, q_addr, smem_u32(smem + C::OFF_K + sn * C::TILE), idesc_s);
            mma_kmajor<HD>(tmem_base + C::TM_DP, do_addr, smem_u32(smem + C::OFF_V + sn * C::TILE), idesc_s);
            umma_commit(s_full);
          }
          __syncwarp();
        }
      }
    }
  } else {
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const uint32_t lane_sel = (uint32_t)(qd * 32) << 16;
    const long long sbase = ((long long)b * p.H + h) * p.S;
    const float lse = grow < p.S ? p.lse[sbase + grow] : INFINITY;
    const float dl = grow < p.S ? p.delta[sbase + grow] : 0.f;
    uint8_t* sDS = smem + C::OFF_DS;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (j > 0 && !mbar_wait(acc_done, (j - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      const int k0 = j * AT_T;
      const bool need_mask = (k0 + AT_T > p.S) || (q0 + AT_T > p.S) || (p.causal && k0 + AT_T - 1 > q0);
#pragma unroll 1
      for (int c = 0; c < AT_T; c += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem_base + C::TM_S + c + lane_sel, rs);
        tmem_ld32(tmem_base + C::TM_DP + c + lane_sel, rd);
        tmem_ld_wait();
        float dv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = fast_exp2(__uint_as_float(rs[i]) * p.sl2 - lse);
          if (need_mask) {
            const int kc = k0 + c + i;
            if (kc >= p.S || grow >= p.S || (p.causal && kc > grow)) e = 0.f;
          }
          dv[i] = e * (__uint_as_float(rd[i]) - dl);
        }
        store_row32_swizzled(sDS, row, c, dv);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_ready);
    }
    if (ok) ok = mbar_wait(acc_done, (nkv - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dqp = p.dq + (long long)b * p.dq_bs + (long long)grow * p.dq_ss + (long long)h * p.dq_hs;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + C::TM_DQ + c + lane_sel, r);
        tmem_ld_wait();
        if (grow < p.S) {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[8 * t + 0]) * p.scale, __uint_as_float(r[8 * t + 1]) * p.scale);
            u.y = pack_bf16(__uint_as_float(r[8 * t + 2]) * p.scale, __uint_as_float(r[8 * t + 3]) * p.scale);
            u.z = pack_bf16(__uint_as_float(r[8 * t + 4]) * p.scale, __uint_as_float(r[8 * t + 5]) * p.scale);
            u.w = pack_bf16(__uint_as_float(r[8 * t + 6]) * p.scale, __uint_as_float(r[8 * t + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dqp + c + 8 * t) = u;
          }
        }
      }
      tc_fence_before();
    }
  }

  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// =============================================================================== host
static int make_map(CUtensorMap* m, const void* base, const FtkAttnDesc* a, long long bs,
                    long long ss, long long hs) {
  // dims {hd, S, H, B}; strides in elements
  typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                         CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                         CUtensorMapFloatOOBfill);
  static Fn enc = nullptr;
  if (!enc) {
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return -1;
    enc = reinterpret_cast<Fn>(fp);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (bs % 8) || (ss % 8) || (hs % 8)) return -4;
  cuuint64_t dims[4] = {(cuuint64_t)a->hd, (cuuint64_t)a->S, (cuuint64_t)a->H, (cuuint64_t)a->B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)(a->H > 1 ? hs : a->hd) * 2,
                           (cuuint64_t)(a->B > 1 ? bs : (long long)a->S * ss) * 2};
  cuuint32_t box[4] = {64, AT_T, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                   box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

static void fill_args(AttnArgs& p, const FtkAttnDesc* a) {
  p.B = a->B; p.H = a->H; p.S = a->S; p.causal = a->causal;
  p.scale = a->scale;
  p.sl2 = a->scale * 1.4426950408889634f;
  p.o = reinterpret_cast<__nv_bfloat16*>(a->o);
  p.o_bs = a->o_bs; p.o_ss = a->o_ss; p.o_hs = a->o_hs;
  p.lse = a->lse; p.delta = a->delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(a->dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(a->dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(a->dv);
  p.dq_bs = a->q_bs; p.dq_ss = a->q_ss; p.dq_hs = a->q_hs;
  p.dk_bs = a->k_bs; p.dk_ss = a->k_ss; p.dk_hs = a->k_hs;
  p.dv_bs = a->v_bs; p.dv_ss = a->v_ss; p.dv_hs = a->v_hs;
  p.status = ftk_status_word();
}

template <typename K>
static int set_smem(K kernel, int bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <int HD>
static int attn_fwd_launch(const FtkAttnDesc* a, cudaStream_t s) {
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, a->q, a, a->q_bs, a->q_ss, a->q_hs))) return rc;
  if ((rc = make_map(&tk, a->k, a, a->k_bs, a->k_ss, a->k_hs))) return rc;
  if ((rc = make_map(&tv, a->v, a, a->v_bs, a->v_ss, a->v_hs))) return rc;
  AttnArgs p;
  fill_args(p, a);
  if (!p.status) return -6;
  static bool attr = false;
  if (!attr) {
    if ((rc = set_smem(attn_fwd_kernel<HD>, FwdCfg<HD>::SMEM))) return rc;
    attr = true;
  }
  dim3 grid((a->S + AT_T - 1) / AT_T, a->H, a->B);
  attn_fwd_kernel<HD><<<grid, AT_THREADS, FwdCfg<HD>::SMEM, s>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
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
  attn_delta_kernel<<<(unsigned)((nrows + 7) / 8), 256, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(a->o), reinterpret_cast<const __nv_bfloat16*>(a->d_o),
      a->delta, a->B, a->H, a->S, a->hd, a->o_bs, a->o_ss, a->o_hs);
  dim3 grid((a->S + AT_T - 1) / AT_T, a->H, a->B);
  attn_bwd_dkv_kernel<HD><<<grid, AT_THREADS, DkvCfg<HD>::SMEM, s>>>(tq, tk, tv, tdo, p);
  attn_bwd_dq_kernel<HD><<<grid, AT_THREADS, DqCfg<HD>::SMEM, s>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_attn_fwd(const FtkAttnDesc* a, void* stream) {
  if (!a || a->B <= 0 || a->H <= 0 || a->S <= 0) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->hd == 64) return attn_fwd_launch<64>(a, s);
  if (a->hd == 128) return attn_fwd_launch<128>(a, s);
  return -5;
}
extern "C" int ftk_attn_bwd(const FtkAttnDesc* a, void* stream) {
  if (!a || a->B <= 0 || a->H <= 0 || a->S <= 0 || !a->delta || !a->lse) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->hd == 64) return attn_bwd_launch<64>(a, s);
  if (a->hd == 128) return attn_bwd_launch<128>(a, s);
  return -5;
}
