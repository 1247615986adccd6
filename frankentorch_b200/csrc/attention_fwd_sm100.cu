// Flash attention forward for sm_100a (tcgen05 / TMEM), head_dim 64 or 128.
//
// Semantics: ft-kernel-cpu/src/lib.rs:4572 sdpa_forward_f64 (blockwise QK^T -> stable online
// softmax -> PV, causal masks j > i); block-online rescaling as in the Metal attn_flash2
// shader (ft-kernel-metal/src/fused.rs:407).  Output O (bf16) and the log-sum-exp in the
// log2 domain of the scaled scores (fp32 [B, H, S]) for the recompute backward.
//
// One CTA owns 256 query rows (two 128-row tiles) of one (batch, head) and streams K and V
// blocks of 128 keys through one TMA ring of tile slots (K_j and V_j are separate slots, each
// released by the commit of the MMAs that read it).  12 warps:
//   warps 0-3  softmax group A (tile 0), warps 4-7 softmax group B (tile 1): one thread per
//              query row reads its whole 128-wide score row into registers with tcgen05.ld and
//              releases the TMEM score tile at once, so QK^T of the next block runs under the
//              exponentials of this one and the two groups alternate on the tensor core;
//   warp 8     TMA producer;  warp 9  issues S = Q K^T (owns TMEM);  warp 10 issues O += P V;
//              warp 11 only hands its registers to the softmax groups (setmaxnreg).
// The output accumulates in TMEM across all key blocks.  The running maximum is lazy: a row
// keeps its reference maximum until a block exceeds it by more than 2^8, and only then is the
// TMEM accumulator rescaled (tcgen05.ld / mul / tcgen05.st, voted per warp).  With head_dim 64
// the probabilities stay in tensor memory (tcgen05.st of packed bf16 pairs by the row's thread)
// and P V is issued with its A operand in TMEM; with head_dim 128 all 512 columns are taken by
// S and O, and P reaches the tensor core through a 128B-swizzled bf16 tile in shared memory.
#include "attn_common.cuh"

namespace ftk {

constexpr int F2_THREADS = 384;
constexpr float F2_LAZY = 8.0f;       // log2 headroom before the accumulator is rescaled

template <int HD>
struct Fwd2Cfg {
  static constexpr int TILE = (HD / 64) * AT_REGION;        // one [128 x HD] bf16 tile
  // head_dim 64 leaves 128 TMEM columns free: the probabilities go there (packed bf16, 64 columns
  // per tile) and P V reads its A operand from tensor memory.  A 128-row CTA tile keeps the
  // tensor core fed from shared memory at 128 B/clk, which is all the SM has: taking the P tile
  // out of shared memory (64 KB written + 64 KB read per key block) roughly halves that traffic.
  static constexpr bool TS = (HD == 64);
  static constexpr int NSLOT = (HD == 64) ? 8 : 3;          // K/V ring
  static constexpr int OFF_Q = 0;                           // 2 tiles
  static constexpr int OFF_KV = 2 * TILE;                   // [NSLOT]
  static constexpr int OFF_P = OFF_KV + NSLOT * TILE;       // 2 tiles of [128 x 128] bf16 (not TS)
  static constexpr int OFF_BAR = OFF_P + (TS ? 0 : 2 * 2 * AT_REGION);
  static constexpr int SMEM = OFF_BAR + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0;                            // S tile t at TM_S + 128 t
  static constexpr int TM_O = 256;                          // O tile t at TM_O + HD t
  static constexpr int TM_P = 256 + 2 * HD;                 // TS: P tile t at TM_P + 64 t
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

#ifdef FT_ATTN_TRACE
// Optional timeline of one CTA (development builds only): [role][iteration][point] clock64 values.
__device__ long long g_attn_trace[4 * 16 * 8 + 3 * 4096];
#define FT_TRACE(role, it, pt)                                                        \
  do {                                                                                \
    if (trace_cta && lane == 0 && (it) < 16) g_attn_trace[((role) * 16 + (it)) * 8 + (pt)] = clock64(); \
  } while (0)
#else
#define FT_TRACE(role, it, pt) do { } while (0)
#endif

template <int REGS>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}

template <int HD>
__global__ void __launch_bounds__(F2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  using C = Fwd2Cfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* q_full = bars;             // [1]
  uint64_t* kv_full = bars + 1;        // [8]
  uint64_t* kv_empty = bars + 9;       // [8]
  uint64_t* s_full = bars + 17;        // [2] per tile: scores in TMEM
  uint64_t* s_free = bars + 19;        // [2] per tile: scores copied to registers (one arrival per warp)
  uint64_t* p_ready = bars + 21;       // [2] per tile: probabilities in smem (one arrival per warp)
  uint64_t* pv_done = bars + 23;       // [2] per tile: PV finished (P tile free, O tile settled)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};
#ifdef FT_ATTN_TRACE
  const bool trace_cta = blockIdx.x == 0;
  const int cta_lin = blockIdx.x;
  if (threadIdx.x == 0 && cta_lin < 4096) {
    unsigned long long t0;
    unsigned smid;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    g_attn_trace[512 + cta_lin * 3 + 0] = (long long)t0;
    g_attn_trace[512 + cta_lin * 3 + 2] = smid;
  }
#endif

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, FT_ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::NSLOT; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);      // one arrival per warp of the group
      mbar_init(&p_ready[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    *abort_f = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Linear grid, heavy (late) query blocks first over the whole launch: every CTA of the block
  // with the most key blocks is scheduled before any lighter one (longest-first keeps the tail
  // of the launch short when the work per CTA varies 4:1 under a causal mask).
  const int n_hb = p.H * p.B;
  const int n_qb = (int)gridDim.x / n_hb;
  const int qb = n_qb - 1 - (int)blockIdx.x / n_hb;
  const int hb = (int)blockIdx.x % n_hb;
  const int h = hb % p.H, b = hb / p.H;
  const int q0 = qb * 2 * AT_T;
  const int nkv_all = (p.S + AT_T - 1) / AT_T;
  int nb[2];                                  // key blocks each tile needs
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * AT_T;
    nb[t] = (r0 >= p.S) ? 0 : (p.causal ? min(r0 / AT_T + 1, nkv_all) : nkv_all);
  }
  const int nkv = max(nb[0], nb[1]);

  if (warp >= 8) {
    reg_dec<40>();
    if (warp == 8) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_arrive_expect_tx(q_full, 2 * C::TILE);
        load_tile<HD>(smem + C::OFF_Q, &tmQ, q_full, q0, h, b);
        load_tile<HD>(smem + C::OFF_Q + C::TILE, &tmQ, q_full, q0 + AT_T, h, b);
      }
      for (int n = 0; n < 2 * nkv; ++n) {     // n = 2j: K_j, n = 2j + 1: V_j
        const int slot = n % C::NSLOT;
        const uint32_t ph = (n / C::NSLOT) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(&kv_full[slot], C::TILE);
          load_tile<HD>(smem + C::OFF_KV + slot * C::TILE, (n & 1) ? &tmV : &tmK, &kv_full[slot],
                        (n >> 1) * AT_T, h, b);
        }
        __syncwarp();
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------ MMA issuer 1: S = Q K^T
      // The issuing thread runs in step with the tensor pipe (an MMA is accepted when the one
      // before the previous has finished), so every wait, fence and descriptor step between
      // two MMAs is time the pipe idles.  Two issuers, one per product, overlap that overhead:
      // this warp owns the K slots, warp 10 the V slots (each slot has one releasing commit).
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t q_addr = smem_u32(smem + C::OFF_Q);
      const uint32_t kv_addr = smem_u32(smem + C::OFF_KV);
      bool ok = mbar_wait(q_full, 0, ctx, FT_ERR_WAIT_FULL);
      for (int jj = 0; ok && jj < nkv; ++jj) {
        FT_TRACE(2, jj, 0);
        const int n = 2 * jj, slot = n % C::NSLOT;
        if (!mbar_wait(&kv_full[slot], (n / C::NSLOT) & 1, ctx, FT_ERR_WAIT_FULL)) break;
        FT_TRACE(2, jj, 1);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (jj >= nb[t]) continue;
          // the score tile must have been copied to registers (block jj - 1)
          if (jj > 0 && !mbar_wait(&s_free[t], (jj - 1) & 1, ctx, FT_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          FT_TRACE(2, jj, 2 + t);
          tc_fence_after();
          if (lane == 0) {
            mma_kmajor<HD>(tmem_base + C::TM_S + 128 * t, q_addr + t * C::TILE,
                           kv_addr + slot * C::TILE, idesc_s);
            umma_commit(&s_full[t]);
          }
          __syncwarp();
        }
        if (!ok) break;
        if (lane == 0) umma_commit(&kv_empty[slot]);
        __syncwarp();
        FT_TRACE(2, jj, 4);
      }
    } else if (warp == 10) {
      // ------------------------------------------------------------ MMA issuer 2: O += P V
      const uint32_t idesc_pv = make_idesc_bf16(128, HD, 0, 1);
      const uint32_t p_addr = smem_u32(smem + C::OFF_P);
      const uint32_t kv_addr = smem_u32(smem + C::OFF_KV);
      bool ok = true;
      for (int j = 0; ok && j < nkv; ++j) {
        FT_TRACE(3, j, 0);
        const int n = 2 * j + 1, slot = n % C::NSLOT;
        if (!mbar_wait(&kv_full[slot], (n / C::NSLOT) & 1, ctx, FT_ERR_WAIT_FULL)) break;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= nb[t]) continue;
          if (!mbar_wait(&p_ready[t], j & 1, ctx, FT_ERR_WAIT_SOFTMAX)) { ok = false; break; }
          FT_TRACE(3, j, 1 + 2 * t);
          tc_fence_after();
          if (lane == 0) {
            if constexpr (C::TS)
              mma_ptmem_times_rows(tmem_base + C::TM_O + HD * t, tmem_base + C::TM_P + 64 * t,
                                   kv_addr + slot * C::TILE, idesc_pv, j > 0);
            else
              mma_p_times_rows(tmem_base + C::TM_O + HD * t, p_addr + t * 2 * AT_REGION,
                               kv_addr + slot * C::TILE, idesc_pv, j > 0);
            umma_commit(&pv_done[t]);
          }
          __syncwarp();
          FT_TRACE(3, j, 2 + 2 * t);
        }
        if (!ok) break;
        if (lane == 0) umma_commit(&kv_empty[slot]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------ softmax groups
    reg_inc<216>();
    const int t = warp >> 2;                 // tile of this group
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int grow = q0 + t * AT_T + row;
    const uint32_t lane_sel = (uint32_t)(qd * 32) << 16;
    const uint32_t s_tmem = tmem_base + C::TM_S + 128 * t + lane_sel;
    const uint32_t o_tmem = tmem_base + C::TM_O + HD * t + lane_sel;
    uint8_t* sP = smem + C::OFF_P + t * 2 * AT_REGION + row * 128;   // not TS
    const uint32_t p_tmem = tmem_base + C::TM_P + 64 * t + lane_sel;   // TS
    const int n_my = nb[t];
    float m2 = -INFINITY;                    // reference maximum, already times sl2
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_my; ++j) {
      FT_TRACE(t, j, 0);
      if (!mbar_wait(&s_full[t], j & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      FT_TRACE(t, j, 1);
      tc_fence_after();
      uint32_t r[128];
      tmem_ld32(s_tmem + 0, r + 0);
      tmem_ld32(s_tmem + 32, r + 32);
      tmem_ld32(s_tmem + 64, r + 64);
      tmem_ld32(s_tmem + 96, r + 96);
      tmem_ld_wait();
      FT_TRACE(t, j, 2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[t]);   // the next QK^T may overwrite the score tile now
      const int k0 = j * AT_T;
      const bool need_mask = (k0 + AT_T > p.S) || (p.causal && k0 + AT_T - 1 > q0 + t * AT_T);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kc = k0 + i;
          if (kc >= p.S || (p.causal && kc > grow)) r[i] = __float_as_uint(-INFINITY);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 8) {
        mx0 = max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        mx1 = max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        mx2 = max3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
        mx3 = max3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
      }
      const float bm2 = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.sl2;   // sl2 > 0
      FT_TRACE(t, j, 3);
      // lazy reference maximum: move it only when this block exceeds the headroom
      float alpha = 1.f;
      const bool move = (bm2 > m2 + F2_LAZY) || (m2 == -INFINITY && bm2 > -INFINITY);
      if (move) {
        alpha = (m2 == -INFINITY) ? 0.f : fast_exp2(m2 - bm2);
        m2 = bm2;
      }
      const float moff = (m2 == -INFINITY) ? 0.f : m2;
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
      // exponentials of elements [i0, i0 + 64): packed probabilities reuse the low registers
      auto exp_half = [&](int i0) {
#pragma unroll
        for (int i = i0; i < i0 + 64; i += 4) {
          const float e0 = fast_exp2(fmaf(__uint_as_float(r[i]), p.sl2, -moff));
          const float e1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), p.sl2, -moff));
          const float e2 = fast_exp2(fmaf(__uint_as_float(r[i + 2]), p.sl2, -moff));
          const float e3 = fast_exp2(fmaf(__uint_as_float(r[i + 3]), p.sl2, -moff));
          rs0 += e0; rs1 += e1; rs2 += e2; rs3 += e3;
          r[i >> 1] = pack_bf16(e0, e1);
          r[(i >> 1) + 1] = pack_bf16(e2, e3);
        }
      };
      // PV of the previous block must be finished before P is overwritten and before the
      // accumulator may be rescaled
      auto settle_previous = [&]() -> bool {
        if (j == 0) return true;
        if (!mbar_wait(&pv_done[t], (j - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL)) return false;
        if (__any_sync(0xffffffffu, move)) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD; c += 32) {
            uint32_t v[32];
            tmem_ld32(o_tmem + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(o_tmem + c, v);
          }
          tmem_st_wait();
          tc_fence_before();
        }
        return true;
      };
      if constexpr (C::TS) {
        // probabilities go to tensor memory, each half as soon as it is computed
        if (!settle_previous()) { ok = false; break; }
        FT_TRACE(t, j, 4);
        tc_fence_after();
        exp_half(0);
        tmem_st32(p_tmem, r);
        exp_half(64);
        tmem_st32(p_tmem + 32, r + 32);
        l = l * alpha + (rs0 + rs1) + (rs2 + rs3);
        FT_TRACE(t, j, 5);
        tmem_st_wait();
        tc_fence_before();
      } else {
        exp_half(0);
        exp_half(64);
        l = l * alpha + (rs0 + rs1) + (rs2 + rs3);
        FT_TRACE(t, j, 4);
        if (!settle_previous()) { ok = false; break; }
        FT_TRACE(t, j, 5);
#pragma unroll
        for (int c16 = 0; c16 < 16; ++c16) {     // 16 chunks of 8 bf16 (16 bytes)
          const uint4 u = make_uint4(r[4 * c16], r[4 * c16 + 1], r[4 * c16 + 2], r[4 * c16 + 3]);
          *reinterpret_cast<uint4*>(sP + (c16 >> 3) * AT_REGION + (((c16 & 7) ^ (row & 7)) << 4)) = u;
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
      FT_TRACE(t, j, 6);
    }
    if (ok && n_my > 0) ok = mbar_wait(&pv_done[t], (n_my - 1) & 1, ctx, FT_ERR_WAIT_TMEM_FULL);
    if (ok && n_my > 0) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = p.o + (long long)b * p.o_bs + (long long)grow * p.o_ss + (long long)h * p.o_hs;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(o_tmem + c, v);
        tmem_ld_wait();
        if (grow < p.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(v[i + 0]) * inv, __uint_as_float(v[i + 1]) * inv);
            u.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            u.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            u.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c + i) = u;
          }
        }
      }
      tc_fence_before();
      if (p.lse && grow < p.S)
        p.lse[((long long)b * p.H + h) * p.S + grow] = (l > 0.f) ? m2 + log2f(l) : -INFINITY;
    }
  }

  if (*abort_f) {
    for (int i = 0; i < 100; ++i) __nanosleep(10000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, C::TMEM_COLS);
#ifdef FT_ATTN_TRACE
  if (threadIdx.x == 0 && cta_lin < 4096) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    g_attn_trace[512 + cta_lin * 3 + 1] = (long long)t1;
  }
#endif
}

template <int HD>
static int attn_fwd2_launch(const FtkAttnDesc* a, cudaStream_t s) {
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
    if ((rc = set_smem(attn_fwd2_kernel<HD>, Fwd2Cfg<HD>::SMEM))) return rc;
    attr = true;
  }
  dim3 grid((unsigned)(((a->S + 2 * AT_T - 1) / (2 * AT_T)) * a->H * a->B));
  attn_fwd2_kernel<HD><<<grid, F2_THREADS, Fwd2Cfg<HD>::SMEM, s>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace ftk

using namespace ftk;

#ifdef FT_ATTN_TRACE
extern "C" int ftk_attn_trace_read(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_attn_trace, sizeof(long long) * n);
}
#endif

extern "C" int ftk_attn_fwd(const FtkAttnDesc* a, void* stream) {
  if (!a || a->B <= 0 || a->H <= 0 || a->S <= 0) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a->hd == 64) return attn_fwd2_launch<64>(a, s);
  if (a->hd == 128) return attn_fwd2_launch<128>(a, s);
  return -5;
}
