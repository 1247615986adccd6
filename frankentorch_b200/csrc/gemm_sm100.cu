// bf16 GEMM for sm_100a: TMA -> 128B-swizzled smem ring -> tcgen05.mma (fp32
// accumulators in TMEM, double buffered) -> tcgen05.ld epilogue.
//
//   D[l][M,N] = epi(alpha * A[l](M x K) * B[l](N x K)^T + bias[N]) (+ residual) (+ D)
//
// Both operands may be given K-major ("[rows, K]" row-major) or MN-major
// ("[K, rows]" row-major), so forward (x W^T), dgrad (dY W) and wgrad (dY^T x) of a
// Linear layer whose weight is [out, in] (reference: ft-kernel-cpu/src/lib.rs:17162
// linear_tensor_f64, :17226 linear_backward_f64) run without materialising a
// transpose.
//
// Determinism: within one launch K is reduced in ascending order by one CTA per output
// tile, so the result does not depend on the grid size.  Weight-gradient shapes (tiny
// output, very long K) use split-K: each split writes its fp32 partial tile to a
// workspace and a second kernel adds the partials in ascending split order - a fixed
// order again, so two runs give identical bits.
//
// One persistent CTA per SM, 10 warps: warp 0 issues TMA loads, warp 1 owns TMEM and
// issues the MMAs, warps 2..9 drain accumulators (warp w reads TMEM lane quarter w%4 and
// one half of the tile's columns).  Two accumulators let the epilogue of tile i overlap
// the mainloop of tile i+1.
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

constexpr int G_BM = 128;
constexpr int G_BK = 64;
constexpr int G_UMMA_K = 16;
constexpr int G_EPI_WARPS = 8;
constexpr int G_THREADS = 64 + 32 * G_EPI_WARPS;

struct GemmArgs {
  int M, N, K, L0, L1;
  int a_mn, b_mn;
  void* D;
  long long ldd, d_s0, d_s1;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  long long ldr, r_s0, r_s1;
  __nv_bfloat16* aux;  // optional bf16 copy of the pre-activation (same layout as D)
  float alpha;
  int epi;
  int out_fp32;
  int accumulate;
  int splits;          // >1: split-K, partial tiles go to `ws` as fp32 [split][M][N]
  float* ws;
  int* status;
};

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = G_BM * G_BK * 2;
  static constexpr int B_BYTES = BN * G_BK * 2;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 192 ? 5 : 6);
  static constexpr int ACC_STRIDE = (BN == 192) ? 256 : BN;  // TMEM columns between accumulators
  static constexpr int TMEM_COLS = (BN == 128) ? 256 : 512;  // power of two
  static constexpr int SMEM = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Epilogue activations use the hardware tanh (relative error ~2^-11, below bf16 rounding).
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanh_fast(u));
}
__device__ __forceinline__ float gelu_tanh_grad_fast(float x) {
  const float x2 = x * x;
  const float t = tanh_fast(0.7978845608028654f * (x + 0.044715f * x * x2));
  const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

// v[i] = f(v[i], rr[i]) for the 32 values of one row chunk; the switch is outside the loop.
__device__ __forceinline__ void apply_epi32(float* v, const float* rr, int epi) {
  switch (epi) {
    case FTK_EPI_GELU_TANH:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
      break;
    case FTK_EPI_GELU_ERF:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_erf_f(v[i]);
      break;
    case FTK_EPI_RELU:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = v[i] > 0.f ? v[i] : 0.f;
      break;
    case FTK_EPI_MUL_DGELU_TANH:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= gelu_tanh_grad_fast(rr[i]);
      break;
    case FTK_EPI_MUL_DGELU_ERF:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= gelu_erf_grad_f(rr[i]);
      break;
    case FTK_EPI_MUL_DRELU:
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = rr[i] > 0.f ? v[i] : 0.f;
      break;
    default:
      break;
  }
}

template <int BN>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_bf16_sm100_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB, const GemmArgs p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + Cfg::STAGES * Cfg::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES));
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::STAGES;
  uint64_t* tfull = bars + 2 * Cfg::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  int* abort_f = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx ctx{p.status, abort_f};

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::STAGES; ++i) {
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

  const int tiles_m = (p.M + G_BM - 1) / G_BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_mn = tiles_m * tiles_n;
  const int nbatch = p.L0 * p.L1;
  const int total = tiles_mn * nbatch * p.splits;  // work item = (split, batch, n tile, m tile)
  const int kblocks_all = (p.K + G_BK - 1) / G_BK;
  const int kb_per_split = (kblocks_all + p.splits - 1) / p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
    }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total; item += gridDim.x) {
      const int sp = item / (tiles_mn * nbatch);
      const int rem = item - sp * (tiles_mn * nbatch);
      const int l = rem / tiles_mn;
      const int t = rem - l * tiles_mn;
      const int m_t = t % tiles_m, n_t = t / tiles_m;
      const int l0 = l % p.L0, l1 = l / p.L0;
      const int kb0 = sp * kb_per_split;
      const int kb1 = min(kblocks_all, kb0 + kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[s], ph ^ 1u, ctx, FT_ERR_WAIT_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
          uint8_t* a_dst = sA + s * Cfg::A_BYTES;
          uint8_t* b_dst = sB + s * Cfg::B_BYTES;
          if (!p.a_mn) {
            tma_load_4d(a_dst, &tmA, &full[s], kb * G_BK, m_t * G_BM, l0, l1);
          } else {
#pragma unroll
            for (int c = 0; c < G_BM / 64; ++c)
              tma_load_4d(a_dst + c * (G_BK * 128), &tmA, &full[s], m_t * G_BM + c * 64, kb * G_BK,
                          l0, l1);
          }
          if (!p.b_mn) {
            tma_load_4d(b_dst, &tmB, &full[s], kb * G_BK, n_t * BN, l0, l1);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_4d(b_dst + c * (G_BK * 128), &tmB, &full[s], n_t * BN + c * 64, kb * G_BK,
                          l0, l1);
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
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_bf16(G_BM, BN, p.a_mn, p.b_mn);
    const uint32_t a_lbo = p.a_mn ? G_BK * 128 : 16, a_adv = p.a_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
    const uint32_t b_lbo = p.b_mn ? G_BK * 128 : 16, b_adv = p.b_mn ? G_UMMA_K * 128 : G_UMMA_K * 2;
    int s = 0;
    uint32_t ph = 0;
    int acc = 0;
    uint32_t acc_ph = 0;  // bit a = phase of accumulator a
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total; item += gridDim.x) {
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
          const uint32_t a_addr = smem_u32(sA + s * Cfg::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * Cfg::B_BYTES);
#pragma unroll
          for (int k = 0; k < G_BK / G_UMMA_K; ++k) {
            umma_bf16(d_tmem, make_smem_desc(a_addr + k * a_adv, a_lbo, 1024),
                      make_smem_desc(b_addr + k * b_adv, b_lbo, 1024), idesc,
                      (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (kb == kb1 - 1) umma_commit(&tfull[acc]);
        }
        __syncwarp();
        if (++s == Cfg::STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (kb1 <= kb0 && lane == 0) umma_commit(&tfull[acc]);  // empty split: nothing to wait for
      __syncwarp();
      acc_ph ^= (1u << acc);
      acc ^= 1;
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps)
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
    for (int item = blockIdx.x; item < total; item += gridDim.x) {
      const int sp = item / (tiles_mn * nbatch);
      const int rem = item - sp * (tiles_mn * nbatch);
      const int l = rem / tiles_mn;
      const int t = rem - l * tiles_mn;
      const int m_t = t % tiles_m, n_t = t / tiles_m;
      const int l0 = l % p.L0, l1 = l / p.L0;
      const bool empty_split = (sp * kb_per_split >= kblocks_all);
      if (!mbar_wait(&tfull[acc], (acc_ph >> acc) & 1u, ctx, FT_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const long long row = (long long)m_t * G_BM + row_in_tile;
      const long long d_off = l0 * p.d_s0 + l1 * p.d_s1 + row * p.ldd;
      const long long r_off = l0 * p.r_s0 + l1 * p.r_s1 + row * p.ldr;
      const bool need_r = p.resid != nullptr;
#pragma unroll 1
      for (int ci = c_begin; ci < c_end; ++ci) {
        const int c0 = ci * 32;
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * Cfg::ACC_STRIDE + c0 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        const int n0 = n_t * BN + c0;
        if (row < p.M && n0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = empty_split ? 0.f : __uint_as_float(r[i]) * p.alpha;
          const bool full_chunk = (n0 + 32 <= p.N);
          if (p.splits > 1) {
            // raw partial tile -> workspace [split][batch][M][N] (fp32)
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

// D (+)= sum over splits (ascending) of ws[split]; 4 outputs per thread.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ D, long long M, long long N,
                     long long ldd, int splits, int out_fp32, int accumulate) {
  const long long total4 = (M * N) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
    float4 s = reinterpret_cast<const float4*>(ws)[i];
    for (int k = 1; k < splits; ++k) {
      const float4 t = reinterpret_cast<const float4*>(ws + (long long)k * M * N)[i];
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    const long long e = i << 2;
    const long long r = e / N, c = e - r * N;
    if (out_fp32) {
      float* dp = reinterpret_cast<float*>(D) + r * ldd + c;
      if (accumulate) {
        const float4 o = *reinterpret_cast<float4*>(dp);
        s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
      }
      *reinterpret_cast<float4*>(dp) = s;
    } else {
      __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(D) + r * ldd + c;
      if (accumulate) {
        const uint2 o = *reinterpret_cast<uint2*>(dp);
        const float2 a = unpack_bf16(o.x), b = unpack_bf16(o.y);
        s.x += a.x; s.y += a.y; s.z += b.x; s.w += b.y;
      }
      uint2 o;
      o.x = pack_bf16(s.x, s.y);
      o.y = pack_bf16(s.z, s.w);
      *reinterpret_cast<uint2*>(dp) = o;
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 4-D bf16 tensor map {inner, outer, l0, l1} with 128B swizzle.
int ftk_make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t l0, uint64_t l1, uint64_t ld_elems, uint64_t s0_elems,
                       uint64_t s1_elems, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {inner, outer, l0, l1};
  uint64_t st1 = ld_elems * 2;
  uint64_t st2 = (l0 > 1 ? s0_elems : outer * ld_elems) * 2;
  uint64_t st3 = (l1 > 1 ? s1_elems : (l0 > 1 ? s0_elems * l0 : outer * ld_elems)) * 2;
  if (st2 == 0) st2 = 16;
  if (st3 == 0) st3 = 16;
  cuuint64_t strides[3] = {st1, st2, st3};
  cuuint32_t box[4] = {box_inner, box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a,
                       int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_sm100_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  long long items = (long long)((a.M + G_BM - 1) / G_BM) * ((a.N + BN - 1) / BN) * a.L0 * a.L1 * a.splits;
  int grid = (int)(items < max_ctas ? items : max_ctas);
  if (grid <= 0) return 0;
  gemm_bf16_sm100_kernel<BN><<<grid, G_THREADS, Cfg::SMEM, stream>>>(tmA, tmB, a);
  return (int)cudaGetLastError();
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_gemm_bf16(const FtkGemmDesc* g, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (!g || g->M <= 0 || g->N <= 0 || g->K <= 0) return -2;
  const int L0 = g->L0 > 0 ? g->L0 : 1, L1 = g->L1 > 0 ? g->L1 : 1;
  // alignment rules of the tiled TMA copies: 16-byte base, 16-byte strides.
  if ((reinterpret_cast<uintptr_t>(g->A) & 15) || (reinterpret_cast<uintptr_t>(g->B) & 15)) return -3;
  if ((g->lda % 8) || (g->ldb % 8)) return -4;
  if ((L0 > 1 && ((g->a_s0 % 8) || (g->b_s0 % 8))) || (L1 > 1 && ((g->a_s1 % 8) || (g->b_s1 % 8))))
    return -4;

  const int sms = g->max_ctas > 0 ? g->max_ctas : num_sms();
  const long long tiles_m = (g->M + G_BM - 1) / G_BM;
  // Tile choice: time ~ waves x per-tile cost.  Narrow tiles move more operand bytes per MMA
  // cycle (measured: a 128-wide tile costs ~0.86 of a 256-wide one for half the work).
  // Split-K (weight-gradient shapes: few output tiles, long reduction) is considered when the
  // epilogue is a plain store and the caller supplied a workspace.
  const int kblocks = (g->K + G_BK - 1) / G_BK;
  const bool splittable = g->epi == FTK_EPI_NONE && !g->bias && !g->resid && !g->aux && g->workspace &&
                          (g->N % 4 == 0) && (g->ldd % 4 == 0) && L0 * L1 == 1;
  auto cost = [&](int bn, int s) {
    const long long tiles = tiles_m * ((g->N + bn - 1) / bn) * L0 * L1;
    const long long waves = (tiles * s + sms - 1) / sms;
    const double w = bn == 256 ? 1.0 : (bn == 192 ? 0.80 : 0.86);
    return (double)waves * w / s + (s > 1 ? 0.08 + 0.01 * s : 0.0);
  };
  auto split_ok = [&](int s) {
    if (s == 1) return true;
    if (!splittable || g->split_k == 1 || kblocks / s < 8) return false;
    return (long long)s * g->M * g->N * 4 <= g->workspace_bytes;
  };
  static const int bn_opts[3] = {256, 192, 128};
  static const int s_opts[8] = {1, 2, 3, 4, 6, 8, 12, 16};
  int bn = g->force_bn, splits = 1;
  double best = 1e30;
  for (int bi = 0; bi < 3; ++bi) {
    if (g->force_bn && bn_opts[bi] != g->force_bn) continue;
    for (int si = 0; si < 8; ++si) {
      const int s = s_opts[si];
      if (g->split_k > 1 && s != g->split_k && s != 1) continue;
      if (!split_ok(s)) continue;
      const double c = cost(bn_opts[bi], s);
      if (c < best - 1e-9) {
        best = c;
        bn = bn_opts[bi];
        splits = s;
      }
    }
  }
  if (g->split_k > 1 && split_ok(g->split_k)) splits = g->split_k;
  if (bn != 128 && bn != 192 && bn != 256) return -5;

  CUtensorMap tmA, tmB;
  int rc;
  if (!g->a_mn)
    rc = ftk_make_tmap_bf16(&tmA, g->A, g->K, g->M, L0, L1, g->lda, g->a_s0, g->a_s1, G_BK, G_BM);
  else
    rc = ftk_make_tmap_bf16(&tmA, g->A, g->M, g->K, L0, L1, g->lda, g->a_s0, g->a_s1, 64, G_BK);
  if (rc) return 1000 + rc;
  if (!g->b_mn)
    rc = ftk_make_tmap_bf16(&tmB, g->B, g->K, g->N, L0, L1, g->ldb, g->b_s0, g->b_s1, G_BK, bn);
  else
    rc = ftk_make_tmap_bf16(&tmB, g->B, g->N, g->K, L0, L1, g->ldb, g->b_s0, g->b_s1, 64, G_BK);
  if (rc) return 2000 + rc;

  GemmArgs a;
  a.M = g->M; a.N = g->N; a.K = g->K; a.L0 = L0; a.L1 = L1;
  a.a_mn = g->a_mn ? 1 : 0; a.b_mn = g->b_mn ? 1 : 0;
  a.D = g->D; a.ldd = g->ldd; a.d_s0 = g->d_s0; a.d_s1 = g->d_s1;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(g->bias);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(g->resid);
  a.ldr = g->ldr; a.r_s0 = g->r_s0; a.r_s1 = g->r_s1;
  a.aux = reinterpret_cast<__nv_bfloat16*>(g->aux);
  a.alpha = g->alpha; a.epi = g->epi; a.out_fp32 = g->out_fp32; a.accumulate = g->accumulate;
  a.splits = splits;
  a.ws = reinterpret_cast<float*>(g->workspace);
  a.status = ftk_status_word();
  if (!a.status) return -6;
  rc = bn == 256 ? launch_gemm<256>(tmA, tmB, a, sms, stream)
                 : (bn == 192 ? launch_gemm<192>(tmA, tmB, a, sms, stream)
                              : launch_gemm<128>(tmA, tmB, a, sms, stream));
  if (rc || splits == 1) return rc;
  const long long total4 = ((long long)g->M * g->N) >> 2;
  long long blocks = (total4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a.ws, g->D, g->M, g->N, g->ldd, splits,
                                                            g->out_fp32, g->accumulate);
  return (int)cudaGetLastError();
}
