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
// the mainloop of tile i+1.  The device code, including the collective-fused forms
// (all-gather -> GEMM, GEMM -> reduce-scatter), lives in gemm_kernel.cuh; this file holds
// the split-K reduction and the host launchers.
#include "gemm2_kernel.cuh"
#include "gemm_group_kernel.cuh"

namespace ftk {

// D (+)= sum over splits (ascending) of ws[split]; 4 outputs per thread.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, void* __restrict__ D, long long M, long long N,
                     long long ldd, int splits, int out_fp32, int accumulate) {
  const long long total4 = (M * N) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += stride) {
    // all partials of the element are requested before the first add (one memory latency, not `splits`);
    // the adds stay in ascending split order
    constexpr int U = 8;
    float4 t[U];
#pragma unroll
    for (int k = 0; k < U; ++k)
      if (k < splits) t[k] = __ldcg(reinterpret_cast<const float4*>(ws + (long long)k * M * N) + i);
    float4 s = t[0];
#pragma unroll
    for (int k = 1; k < U; ++k)
      if (k < splits) { s.x += t[k].x; s.y += t[k].y; s.z += t[k].z; s.w += t[k].w; }
    for (int k0 = U; k0 < splits; k0 += U) {
#pragma unroll
      for (int k = 0; k < U; ++k)
        if (k0 + k < splits) t[k] = __ldcg(reinterpret_cast<const float4*>(ws + (long long)(k0 + k) * M * N) + i);
#pragma unroll
      for (int k = 0; k < U; ++k)
        if (k0 + k < splits) { s.x += t[k].x; s.y += t[k].y; s.z += t[k].z; s.w += t[k].w; }
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

__global__ void tick_i32_kernel(int* w) { *w += 1; }

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

static int num_sms() {
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!cache[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cache[dev] = n > 0 ? n : 148;
  }
  return cache[dev];
}

// cudaFuncSetAttribute applies to the current device only: remember per device what was set.
struct PerDeviceOnce {
  bool done[64] = {false};
  bool* slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return &done[dev];
  }
};

template <int BN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a,
                       int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static PerDeviceOnce once;
  bool* attr_set_p = once.slot();
  if (!*attr_set_p) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_sm100_kernel<BN, 0>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    *attr_set_p = true;
  }
  long long items = (long long)((a.M + G_BM - 1) / G_BM) * ((a.N + BN - 1) / BN) * a.L0 * a.L1 * a.splits;
  int grid = (int)(items < max_ctas ? items : max_ctas);
  if (grid <= 0) return 0;
  CommArgs none;
  memset(&none, 0, sizeof(none));
  gemm_bf16_sm100_kernel<BN, 0><<<grid, G_THREADS, Cfg::SMEM, stream>>>(tmA, tmB, tmA, a, none);
  return (int)cudaGetLastError();
}

// CTA-pair kernel: grid = 2 CTAs per cluster, at most sms / 2 clusters.
// Relative cost of a pair tile in the tile-choice model (a lone 128 x 256 tile = 1.0); the
// environment variable FT_GEMM_PAIR_COST overrides it (a large value disables the pair kernel).
static double pair_tile_cost() {
  static double c = -1.0;
  if (c < 0.0) {
    const char* e = getenv("FT_GEMM_PAIR_COST");
    c = (e && atof(e) > 0.0) ? atof(e) : 0.92;
  }
  return c;
}
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& a, int max_ctas,
                            cudaStream_t stream) {
  using Cfg = Gemm2Cfg;
  static PerDeviceOnce once;
  bool* attr_set_p = once.slot();
  if (!*attr_set_p) {
    cudaError_t e = cudaFuncSetAttribute(gemm2_bf16_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    *attr_set_p = true;
  }
  const long long items = (long long)((a.M + 255) / 256) * ((a.N + 255) / 256) * a.L0 * a.L1 * a.splits;
  long long pairs = max_ctas / 2;
  if (items < pairs) pairs = items;
  if (pairs <= 0) return 0;
  gemm2_bf16_sm100_kernel<<<(unsigned)(2 * pairs), G_THREADS, Cfg::SMEM, stream>>>(tmA, tmB, a);
  return (int)cudaGetLastError();
}

static int make_operand_maps(const FtkGemmDesc* g, int L0, int L1, int bn, CUtensorMap* tmA,
                             CUtensorMap* tmB) {
  int rc;
  if (!g->a_mn)
    rc = ftk_make_tmap_bf16(tmA, g->A, g->K, g->M, L0, L1, g->lda, g->a_s0, g->a_s1, G_BK, G_BM);
  else
    rc = ftk_make_tmap_bf16(tmA, g->A, g->M, g->K, L0, L1, g->lda, g->a_s0, g->a_s1, 64, G_BK);
  if (rc) return 1000 + rc;
  if (!g->b_mn)
    rc = ftk_make_tmap_bf16(tmB, g->B, g->K, g->N, L0, L1, g->ldb, g->b_s0, g->b_s1, G_BK, bn);
  else
    rc = ftk_make_tmap_bf16(tmB, g->B, g->N, g->K, L0, L1, g->ldb, g->b_s0, g->b_s1, 64, G_BK);
  if (rc) return 2000 + rc;
  return 0;
}

static void fill_gemm_args(GemmArgs& a, const FtkGemmDesc* g, int L0, int L1) {
  a.M = g->M; a.N = g->N; a.K = g->K; a.L0 = L0; a.L1 = L1;
  a.a_mn = g->a_mn ? 1 : 0; a.b_mn = g->b_mn ? 1 : 0;
  a.D = g->D; a.ldd = g->ldd; a.d_s0 = g->d_s0; a.d_s1 = g->d_s1;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(g->bias);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(g->resid);
  a.ldr = g->ldr; a.r_s0 = g->r_s0; a.r_s1 = g->r_s1;
  a.aux = reinterpret_cast<__nv_bfloat16*>(g->aux);
  a.alpha = g->alpha; a.epi = g->epi; a.out_fp32 = g->out_fp32; a.accumulate = g->accumulate;
  a.splits = 1;
  a.ws = reinterpret_cast<float*>(g->workspace);
  a.status = ftk_status_word();
  a.seg_counts = g->seg_counts;
  a.seg_rows = g->seg_rows;
}

}  // namespace ftk

using namespace ftk;

// flags[0..n) = *epoch with system-scope release stores (the flags may live on another GPU); launched
// behind the copy whose arrival they announce, on the same stream.
__global__ void set_flags_sys_kernel(int* flags, int n, const int* __restrict__ epoch) {
  const int e = *epoch;
  __threadfence_system();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags + i), "r"(e) : "memory");
}
extern "C" int ftk_set_flags_sys(int* flags, int n, const int* epoch, void* stream_v) {
  if (!flags || !epoch || n <= 0) return -2;
  // one warp: it must find room on an SM beside a resident GEMM CTA (the consumer that waits for these flags)
  set_flags_sys_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(flags, n, epoch);
  return (int)cudaGetLastError();
}
// One device-to-device copy on a stream (local or peer destination): the copy engines move it, no SM is used.
extern "C" int ftk_copy_async(void* dst, const void* src, long long bytes, void* stream_v) {
  if (!dst || !src || bytes <= 0) return -2;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice,
                              reinterpret_cast<cudaStream_t>(stream_v));
}

extern "C" int ftk_tick_i32(int* word, void* stream_v) {
  if (!word) return -2;
  tick_i32_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(word);
  return (int)cudaGetLastError();
}

// Argument checks and tile choice shared by the launcher and the plan query.  Returns 0 and
// (bn, splits), or a negative argument error.  bn == 512 stands for the CTA-pair kernel.
static int plan_gemm(const FtkGemmDesc* g, int* bn_out, int* splits_out) {
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
  if (g->seg_counts && g->seg_rows <= 0) return -2;
  const bool splittable = g->epi == FTK_EPI_NONE && !g->bias && !g->resid && !g->aux && g->workspace &&
                          (g->N % 4 == 0) && (g->ldd % 4 == 0) && L0 * L1 == 1 && !g->seg_counts;
  // Option 512 is the CTA-pair kernel: 256 x 256 tiles on sms / 2 clusters; per SM it does the
  // work of a 128 x 256 tile with a third less operand traffic.
  // The unit is the time of one 128 x 256 tile over all of K on one SM at the sustained rate (~6.9 ns per
  // unit of K).  A split costs the reduction kernel: s fp32 partials read, the output written (and read when
  // it accumulates) at ~4 TB/s plus a launch - 17 us for an [8192, 768] bf16 output with two splits, which is
  // why an activation-sized output is hardly ever worth splitting while a weight gradient is.
  const double unit_us = 6.93e-3 * (double)g->K;
  auto split_penalty = [&](int s) {
    if (s <= 1) return 0.0;
    const double mn = (double)g->M * (double)g->N;
    const double bytes = mn * 4.0 * s + mn * (g->out_fp32 ? 4.0 : 2.0) * (g->accumulate ? 2.0 : 1.0);
    return (bytes / 4.0e6 + 3.0) / unit_us;
  };
  auto cost = [&](int bn, int s) {
    if (bn == 512) {
      const long long tiles = ((g->M + 255) / 256) * ((g->N + 255) / 256) * L0 * L1;
      const long long waves = (tiles * s + sms / 2 - 1) / (sms / 2);
      // A pair tile has twice the epilogue of a single one and a longer pipeline fill, which a long K
      // amortises: measured against 128 x 192 tiles it costs ~1.0 at K = 768 and ~0.72 at K = 3072
      // (8192 x 768 x 2304: 37.5 vs 45.8 us, x 3072: 47.5 vs 53.0 us), and about a tenth more when B is given
      // [K, N] (8192 x 3072 x 768: 65.2 vs 54.3 us).  The base value is the K = 768 calibration.
      double kr = 768.0 * s / (double)g->K;
      if (kr > 1.5) kr = 1.5;
      static const bool k_scaled = !(getenv("FT_GEMM_PAIR_KSCALE") && atoi(getenv("FT_GEMM_PAIR_KSCALE")) == 0);
      const double c = k_scaled ? pair_tile_cost() * (0.608 + 0.392 * kr) * (g->b_mn ? 1.08 : 1.0) : pair_tile_cost();
      return (double)waves * c / s + split_penalty(s);
    }
    const long long tiles = tiles_m * ((g->N + bn - 1) / bn) * L0 * L1;
    const long long waves = (tiles * s + sms - 1) / sms;
    const double w = bn == 256 ? 1.0 : (bn == 192 ? 0.80 : 0.86);
    return (double)waves * w / s + split_penalty(s);
  };
  auto split_ok = [&](int s) {
    if (s == 1) return true;
    if (!splittable || g->split_k == 1 || kblocks / s < 8) return false;
    return (long long)s * g->M * g->N * 4 <= g->workspace_bytes;
  };
  static const int bn_opts[4] = {512, 256, 192, 128};
  static const int s_opts[8] = {1, 2, 3, 4, 6, 8, 12, 16};
  int bn = g->force_bn, splits = 1;
  double best = 1e30;
  for (int bi = 0; bi < 4; ++bi) {
    if (bn_opts[bi] == 512 && (sms < 2 || g->M < 256 || g->seg_counts)) continue;
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
  if (bn != 128 && bn != 192 && bn != 256 && bn != 512) return -5;
  *bn_out = bn;
  *splits_out = splits;
  return 0;
}

// Grouped launch: `n` (1..8) independent products with the same K and operand layouts, fp32 outputs with a plain
// store or accumulate epilogue, in one persistent kernel of 128 x 192 tiles (see gemm_group_kernel.cuh).
extern "C" int ftk_gemm_group_bf16(const FtkGemmDesc* descs, int n, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (!descs || n < 1 || n > GG_MAX) return -2;
  GroupArgs ga;
  GroupMaps maps;
  memset(&ga, 0, sizeof(ga));
  memset(&maps, 0, sizeof(maps));
  const FtkGemmDesc& g0 = descs[0];
  ga.n = n; ga.K = g0.K; ga.a_mn = g0.a_mn ? 1 : 0; ga.b_mn = g0.b_mn ? 1 : 0; ga.alpha = g0.alpha;
  ga.status = ftk_status_word();
  if (!ga.status) return -6;
  int total = 0;
  for (int p = 0; p < n; ++p) {
    const FtkGemmDesc* g = &descs[p];
    if (g->M <= 0 || g->N <= 0 || g->K != g0.K || (g->a_mn ? 1 : 0) != ga.a_mn || (g->b_mn ? 1 : 0) != ga.b_mn ||
        g->alpha != g0.alpha)
      return -2;
    if ((g->L0 > 1) || (g->L1 > 1) || !g->out_fp32 || g->epi != FTK_EPI_NONE || g->bias || g->resid || g->aux ||
        g->seg_counts || !g->D)
      return -7;
    if ((reinterpret_cast<uintptr_t>(g->A) & 15) || (reinterpret_cast<uintptr_t>(g->B) & 15)) return -3;
    if ((g->lda % 8) || (g->ldb % 8)) return -4;
    int rc = make_operand_maps(g, 1, 1, GG_BN, &maps.a[p], &maps.b[p]);
    if (rc) return rc;
    ga.M[p] = g->M; ga.N[p] = g->N;
    ga.D[p] = reinterpret_cast<float*>(g->D);
    ga.ldd[p] = g->ldd;
    ga.accumulate[p] = g->accumulate ? 1 : 0;
    total += ((g->M + G_BM - 1) / G_BM) * ((g->N + GG_BN - 1) / GG_BN);
    ga.tile_end[p] = total;
  }
  for (int p = n; p < GG_MAX; ++p) ga.tile_end[p] = total;
  using Cfg = GemmCfg<GG_BN>;
  static PerDeviceOnce once;
  bool* attr_set_p = once.slot();
  if (!*attr_set_p) {
    cudaError_t e = cudaFuncSetAttribute(gemm_group_bf16_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GG_SMEM);
    if (e != cudaSuccess) return (int)e;
    *attr_set_p = true;
  }
  const int sms = g0.max_ctas > 0 ? g0.max_ctas : num_sms();
  const int grid = total < sms ? total : sms;
  gemm_group_bf16_sm100_kernel<<<grid, G_THREADS, GG_SMEM, stream>>>(maps, ga);
  return (int)cudaGetLastError();
}

// Which kernel ftk_gemm_bf16 would launch for this problem: *bn = 128 / 192 / 256 (single-CTA tile
// 128 x bn) or 512 (CTA-pair kernel, 256 x 256 tiles); *splits = split-K factor.  Launches nothing.
extern "C" int ftk_gemm_plan(const FtkGemmDesc* g, int* bn, int* splits) {
  if (!bn || !splits) return -2;
  return plan_gemm(g, bn, splits);
}

extern "C" int ftk_gemm_bf16(const FtkGemmDesc* g, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  int bn = 0, splits = 1;
  int prc = plan_gemm(g, &bn, &splits);
  if (prc) return prc;
  const int L0 = g->L0 > 0 ? g->L0 : 1, L1 = g->L1 > 0 ? g->L1 : 1;
  const int sms = g->max_ctas > 0 ? g->max_ctas : num_sms();

  CUtensorMap tmA, tmB;
  int rc = make_operand_maps(g, L0, L1, bn == 512 ? 128 : bn, &tmA, &tmB);   // a pair stages 128 B rows per CTA
  if (rc) return rc;

  GemmArgs a;
  fill_gemm_args(a, g, L0, L1);
  a.splits = splits;
  if (!a.status) return -6;
  rc = bn == 512 ? launch_gemm_pair(tmA, tmB, a, sms, stream)
       : bn == 256 ? launch_gemm<256>(tmA, tmB, a, sms, stream)
                   : (bn == 192 ? launch_gemm<192>(tmA, tmB, a, sms, stream)
                                : launch_gemm<128>(tmA, tmB, a, sms, stream));
  if (rc || splits == 1) return rc;
  const long long total4 = ((long long)g->M * g->N) >> 2;
  long long blocks = (total4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaStream_t rs = g->reduce_stream ? reinterpret_cast<cudaStream_t>(g->reduce_stream) : stream;
  if (rs != stream) {
    // reduction on its own stream, ordered behind the GEMM (one event per device, re-recorded per call)
    static cudaEvent_t ev[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!ev[dev]) {
      cudaError_t e = cudaEventCreateWithFlags(&ev[dev], cudaEventDisableTiming);
      if (e != cudaSuccess) return (int)e;
    }
    cudaError_t e = cudaEventRecord(ev[dev], stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(rs, ev[dev], 0);
    if (e != cudaSuccess) return (int)e;
  }
  splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, rs>>>(a.ws, g->D, g->M, g->N, g->ldd, splits,
                                                         g->out_fp32, g->accumulate);
  return (int)cudaGetLastError();
}

// GEMM fused with all-gather of an operand or reduce-scatter of the output (see ftk_api.h).
extern "C" int ftk_gemm_comm_bf16(const FtkGemmDesc* g, const FtkCommDesc* cd, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (!g || !cd || g->M <= 0 || g->N <= 0 || g->K <= 0) return -2;
  if (cd->world < 1 || cd->world > FTK_MAX_RANKS || cd->rank < 0 || cd->rank >= cd->world) return -2;
  if (cd->mode < FTK_COMM_GATHER_A || cd->mode > FTK_COMM_SCATTER_D || !cd->epoch) return -2;
  if ((g->L0 > 1) || (g->L1 > 1)) return -2;
  if ((reinterpret_cast<uintptr_t>(g->A) & 15) || (reinterpret_cast<uintptr_t>(g->B) & 15)) return -3;
  if ((g->lda % 8) || (g->ldb % 8)) return -4;
  if (cd->chunk_rows <= 0 || cd->chunk_rows % G_BM) return -7;
  constexpr int BN = 256;
  const long long rows_total = (long long)cd->chunk_rows * cd->world;

  CommArgs c;
  memset(&c, 0, sizeof(c));
  c.mode = cd->mode; c.rank = cd->rank; c.world = cd->world; c.chunk_rows = cd->chunk_rows;
  c.epoch = cd->epoch;
  const int sms = g->max_ctas > 0 ? g->max_ctas : num_sms();
  // gathers: CTAs that only move data (default 20); reduce-scatter: every CTA reduces after its
  // GEMM tiles, dedicated CTAs are optional (default none)
  c.comm_ctas = cd->comm_ctas > 0 ? cd->comm_ctas : (cd->mode == FTK_COMM_SCATTER_D ? 0 : 20);
  if (cd->mode != FTK_COMM_SCATTER_D && (cd->push == 2 || cd->push == 3)) {
    c.comm_ctas = 0;    // 2: the shards arrive by copy engine; 3: the epilogue warps of every CTA push them
  } else if (cd->comm_ctas <= 0 && cd->mode != FTK_COMM_SCATTER_D && cd->push) {
    c.comm_ctas = 16;
  } else if (cd->comm_ctas <= 0 && cd->mode != FTK_COMM_SCATTER_D) {
    // Split the SMs between copying and computing in proportion to the work: a copy CTA keeps
    // 128 KB of peer loads in flight, which at NVLink latency under load is ~13 GB/s (measured
    // at 2 and 8 ranks), a compute CTA delivers its share of the sustained GEMM rate.
    const bool bk = cd->mode == FTK_COMM_GATHER_B && g->b_mn;
    const double row_bytes = 2.0 * (double)(bk ? g->N : g->K);
    const double remote = (double)(cd->world - 1) * (double)cd->chunk_rows * row_bytes;
    const double comm_work = remote / 13e9;
    const double gemm_work = 2.0 * (double)g->M * (double)g->N * (double)g->K / (1.4e15 / (double)sms);
    int cc = (int)(sms * comm_work / (comm_work + gemm_work) + 0.5);
    if (cc < 12) cc = 12;
    if (cc > 64) cc = 64;
    if (cd->world == 1) cc = 32;   // nothing to fetch: the copy CTAs only stage the own chunk
    c.comm_ctas = cc;
  }
  if (c.comm_ctas >= sms) return -7;

  if (cd->mode == FTK_COMM_SCATTER_D) {
    if (rows_total != g->M || (g->N % 8) || (g->ldd % 8) || (g->resid && (g->ldr % 8))) return -7;
    if (g->epi != FTK_EPI_NONE || g->aux) return -7;
    for (int r = 0; r < cd->world; ++r) {
      if (!cd->inbox[r] || !cd->arrive[r]) return -2;
      c.inbox[r] = reinterpret_cast<__nv_bfloat16*>(cd->inbox[r]);
      c.arrive[r] = cd->arrive[r];
    }
  } else {
    const bool ga = cd->mode == FTK_COMM_GATHER_A;
    // the staged operand must be contiguous [rows, K] so that a subtile is one byte range
    // (B given MN-major, i.e. [K, N] row-major, is sharded along K: dgrad with a sharded weight)
    const bool bk = !ga && g->b_mn;
    if (ga ? (g->a_mn || g->lda != g->K || rows_total != g->M)
           : (bk ? (g->ldb != g->N || rows_total != g->K) : (g->ldb != g->K || rows_total != g->N)))
      return -7;
    c.sub_bytes = (long long)G_BM * (bk ? g->N : g->K) * 2;
    if (c.sub_bytes > G_COPY_SLOT ? (c.sub_bytes % G_COPY_SLOT) : (c.sub_bytes % 16)) return -7;
    if (!cd->sub_flags) return -2;
    c.full = reinterpret_cast<uint8_t*>(const_cast<void*>(ga ? g->A : g->B));
    c.sub_flags = cd->sub_flags;
    c.ready_local = cd->push ? nullptr : cd->ready_local;
    c.push = cd->push == 3 ? 3 : (cd->push ? 1 : 0);
    for (int r = 0; r < cd->world; ++r) {
      if (cd->push) {
        // only the own shard is read; peers' staging buffers and flag arrays are written
        if (!cd->full_peer[r] || !cd->flags_peer[r] || (reinterpret_cast<uintptr_t>(cd->full_peer[r]) & 15)) return -2;
        c.full_peer[r] = reinterpret_cast<uint8_t*>(cd->full_peer[r]);
        c.flags_peer[r] = cd->flags_peer[r];
        if (r != cd->rank) continue;
      }
      if (!cd->src[r] || (reinterpret_cast<uintptr_t>(cd->src[r]) & 15)) return -3;
      c.src[r] = reinterpret_cast<const uint8_t*>(cd->src[r]);
      c.ready_peer[r] = cd->ready_peer[r];
      if (!cd->push && cd->ready_local && r != cd->rank && !cd->ready_peer[r]) return -2;
    }
    if (cd->push && (c.full_peer[cd->rank] != c.full || c.flags_peer[cd->rank] != c.sub_flags)) return -2;
  }

  CUtensorMap tmA, tmB;
  int rc = make_operand_maps(g, 1, 1, BN, &tmA, &tmB);
  if (rc) return rc;
  GemmArgs a;
  fill_gemm_args(a, g, 1, 1);
  if (!a.status) return -6;

  using Cfg = GemmCfg<BN>;
  constexpr int COMM_SMEM = Cfg::SMEM;
  static PerDeviceOnce once;
  bool* attr_set_p = once.slot();
  if (!*attr_set_p) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_sm100_kernel<BN, 1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, COMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    *attr_set_p = true;
  }
  const long long items = (long long)((a.M + G_BM - 1) / G_BM) * ((a.N + BN - 1) / BN);
  long long n_compute = sms - c.comm_ctas;
  if (items < n_compute) n_compute = items;
  const int grid = (int)n_compute + c.comm_ctas;   // all CTAs resident: one per SM
  // tiles inside this rank's own shard are read from the shard, not from the staging buffer
  CUtensorMap tmOwn = tmA;
  if (cd->mode == FTK_COMM_GATHER_A)
    rc = ftk_make_tmap_bf16(&tmOwn, cd->src[cd->rank], g->K, cd->chunk_rows, 1, 1, g->K, 0, 0, G_BK, G_BM);
  else if (cd->mode == FTK_COMM_GATHER_B && !g->b_mn && cd->chunk_rows >= BN)
    rc = ftk_make_tmap_bf16(&tmOwn, cd->src[cd->rank], g->K, cd->chunk_rows, 1, 1, g->K, 0, 0, G_BK, BN);
  if (rc) return 3000 + rc;
  gemm_bf16_sm100_kernel<BN, 1><<<grid, G_THREADS, COMM_SMEM, stream>>>(tmA, tmB, tmOwn, a, c);
  return (int)cudaGetLastError();
}
