// Shared pieces of the sm_100a attention kernels: argument block, tcgen05 MMA helpers for the
// two operand forms used by attention, the swizzled probability-tile store, TMA tile loads and
// the host-side tensor-map construction over packed [B, S, H, hd] activations.
#pragma once
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

// A (K-major) x B (K-major)^T with K = HD, operands stored as HD/64 regions.  The descriptors'
// low words are built once per call and stepped by constants (see desc_lo).
template <int HD>
__device__ __forceinline__ void mma_kmajor(uint32_t d_tmem, uint32_t a_base, uint32_t b_base,
                                           uint32_t idesc) {
  const uint32_t a_lo = desc_lo(a_base, 16), b_lo = desc_lo(b_base, 16);
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const uint32_t off = (uint32_t)(((kk >> 2) * AT_REGION + (kk & 3) * 32) >> 4);
    umma_bf16_lo(d_tmem, a_lo + off, b_lo + off, idesc, kk != 0 ? 1u : 0u);
  }
}
// A = probabilities [128 x 128] K-major in two regions; B = [128 k-rows x HD] stored
// row-major per 64-column region (MN-major operand), K = 128.
__device__ __forceinline__ void mma_p_times_rows(uint32_t d_tmem, uint32_t p_base, uint32_t b_base,
                                                 uint32_t idesc, bool accumulate) {
  const uint32_t a_lo = desc_lo(p_base, 16), b_lo = desc_lo(b_base, AT_REGION);
#pragma unroll
  for (int kk = 0; kk < AT_T / 16; ++kk) {
    const uint32_t a_off = (uint32_t)(((kk >> 2) * AT_REGION + (kk & 3) * 32) >> 4);
    umma_bf16_lo(d_tmem, a_lo + a_off, b_lo + (uint32_t)(kk * 128), idesc, (accumulate || kk != 0) ? 1u : 0u);
  }
}
// Same product with A = probabilities held in tensor memory: 128 lanes (rows) x 64 columns of
// packed bf16 pairs (K = 128), written by the row-owning threads with tcgen05.st.
__device__ __forceinline__ void mma_ptmem_times_rows(uint32_t d_tmem, uint32_t p_tmem, uint32_t b_base,
                                                     uint32_t idesc, bool accumulate) {
  const uint32_t b_lo = desc_lo(b_base, AT_REGION);
#pragma unroll
  for (int kk = 0; kk < AT_T / 16; ++kk) {
    umma_bf16_ts_lo(d_tmem, p_tmem + kk * 8, b_lo + (uint32_t)(kk * 128), idesc,
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


// ------------------------------------------------------------------------------- host helpers
static inline int make_map(CUtensorMap* m, const void* base, const FtkAttnDesc* a, long long bs,
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

static inline void fill_args(AttnArgs& p, const FtkAttnDesc* a) {
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
static inline int set_smem(K kernel, int bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}


}  // namespace ftk
