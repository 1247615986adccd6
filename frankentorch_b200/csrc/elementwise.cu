// Elementwise, embedding, optimizer and utility kernels (all HBM-bandwidth bound):
// GELU fwd/bwd (erf form is the reference default, ft-kernel-cpu/src/lib.rs:1924; the
// tanh form with the +-10 clamp is the Metal shader's, ft-kernel-metal/src/fused.rs:302),
// residual add (fused.rs:316), casts, replayable counter-based dropout
// (mask = rand > p scaled by 1/(1-p), ft-nn/src/lib.rs:2357), embedding gather and
// deterministic scatter-add, fused AdamW (ft-optim/src/lib.rs:1040-1054), the
// headless RGBA8 presenter (ft-kernel-metal/src/presentation.rs:224) and the 1-D
// im2col gather (fused.rs:262).  The runtime status word lives here too.
#include <cuda_fp16.h>
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

// ------------------------------------------------------------------------ status word
static int* g_status[64] = {nullptr};

}  // namespace ftk
using namespace ftk;

extern "C" int* ftk_status_word(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}
extern "C" int ftk_read_status(int reset) {
  int* p = ftk_status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -3;
  if (reset && v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

namespace ftk {

__device__ __forceinline__ void unpack8e(const uint4& u, float* f) {
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8e(const float* f) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  return u;
}
__device__ __forceinline__ float gelu_tanh_clamped(float x) {
  if (x >= 10.f) return x;
  if (x <= -10.f) return 0.f;
  return gelu_tanh_f(x);
}

// OP 0: gelu fwd, 1: gelu bwd (a = x, b = dy), 2: add
template <int OP>
__global__ void __launch_bounds__(256)
ew_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
               __nv_bfloat16* __restrict__ out, long long n, int tanh_form) {
  const long long nvec = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float fa[8], fb[8];
    unpack8e(reinterpret_cast<const uint4*>(a)[v], fa);
    if (OP != 0) unpack8e(reinterpret_cast<const uint4*>(b)[v], fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (OP == 0) fa[i] = tanh_form ? gelu_tanh_clamped(fa[i]) : gelu_erf_f(fa[i]);
      if (OP == 1) fa[i] = fb[i] * (tanh_form ? gelu_tanh_grad_f(fa[i]) : gelu_erf_grad_f(fa[i]));
      if (OP == 2) fa[i] += fb[i];
    }
    reinterpret_cast<uint4*>(out)[v] = pack8e(fa);
  }
  // tail
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = nvec << 3; i < n; ++i) {
      float x = __bfloat162float(a[i]), y = OP != 0 ? __bfloat162float(b[i]) : 0.f, r;
      if (OP == 0) r = tanh_form ? gelu_tanh_clamped(x) : gelu_erf_f(x);
      else if (OP == 1) r = y * (tanh_form ? gelu_tanh_grad_f(x) : gelu_erf_grad_f(x));
      else r = x + y;
      out[i] = __float2bfloat16(r);
    }
  }
}

__global__ void __launch_bounds__(256)
cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(x[i]);
}
__global__ void __launch_bounds__(256)
cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, long long n,
                     int accumulate) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = __bfloat162float(x[i]);
    y[i] = accumulate ? y[i] + v : v;
  }
}

// ------------------------------------------------------------------------ Philox dropout
__device__ __forceinline__ void philox_round(uint32_t* c, uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ void philox4x32(uint64_t seed, uint64_t ctr, uint32_t* out) {
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}
// Element i keeps its value (scaled) iff u_i > p where u_i comes from counter (offset + i/4).
__global__ void __launch_bounds__(256)
dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
               float p, unsigned long long seed, unsigned long long offset) {
  const float inv = 1.f / (1.f - p);
  const long long nq = (n + 3) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < nq; q += stride) {
    uint32_t r[4];
    philox4x32(seed, offset + (uint64_t)q, r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      long long idx = q * 4 + i;
      if (idx < n) {
        float u = (r[i] >> 8) * (1.0f / 16777216.0f);
        y[idx] = __float2bfloat16(u > p ? __bfloat162float(x[idx]) * inv : 0.f);
      }
    }
  }
}

// ------------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(128)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ wte,
                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, int S,
                     int d, long long vocab, int* status) {
  const int r = blockIdx.x;
  long long id = ids[r];
  // a token id outside the table: reported through the status word, row 0 is read instead
  if (!ft_index_ok(id, vocab, status)) id = 0;
  const uint4* te = reinterpret_cast<const uint4*>(wte + (size_t)id * d);
  const uint4* pe = wpe ? reinterpret_cast<const uint4*>(wpe + (size_t)(r % S) * d) : nullptr;
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)r * d);
  for (int v = threadIdx.x; v < (d >> 3); v += blockDim.x) {
    uint4 u = __ldg(te + v);
    if (pe) {
      float a[8], b[8];
      unpack8e(u, a);
      unpack8e(__ldg(pe + v), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += b[i];
      u = pack8e(a);
    }
    o[v] = u;
  }
}
// One CTA per sorted position; the CTA at the first position of a run of equal ids sums
// that run's rows in sorted (stable => ascending row) order, every other CTA exits.
__global__ void __launch_bounds__(128)
embedding_bwd_wte_kernel(const long long* __restrict__ sorted_ids, const int* __restrict__ order,
                         int rows, const __nv_bfloat16* __restrict__ dout,
                         float* __restrict__ dwte, int d, long long vocab, int* status) {
  const int b = blockIdx.x;
  const long long id = sorted_ids[b];
  if (b > 0 && sorted_ids[b - 1] == id) return;
  if (!ft_index_ok(id, vocab, status)) return;     // no table row to add into
  int e = b + 1;
  while (e < rows && sorted_ids[e] == id) ++e;
  for (int c = threadIdx.x * 2; c < d; c += blockDim.x * 2) {
    float s0 = 0.f, s1 = 0.f;
    for (int i = b; i < e; ++i) {
      float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(dout + (size_t)FT_IDX(order[i], rows, status) * d + c));
      s0 += v.x;
      s1 += v.y;
    }
    float* dst = dwte + (size_t)id * d + c;
    dst[0] += s0;
    dst[1] += s1;
  }
}
// The same scatter-add without a sort: one CTA per position i.  It first looks for an earlier position with the
// same token (then it has nothing to do: the first occurrence owns the row), otherwise it walks the later
// positions in ascending order, 1024 at a time, and adds the rows of those that carry its token: the sum of a
// table row is taken in ascending position order, exactly as after a stable sort, so both forms give the same
// bits.  The ids (64 KB for 8192 positions) stay in L2; chunks without a match cost one load and one block-wide
// vote.  No library sort, no atomics.
__global__ void __launch_bounds__(128)
embedding_bwd_wte_scan_kernel(const long long* __restrict__ ids, int rows, const __nv_bfloat16* __restrict__ dout,
                              float* __restrict__ dwte, int d, long long vocab, int* status) {
  constexpr int BLK = 1024;                               // positions looked at per vote: 8 loads in flight per thread
  __shared__ unsigned char match[BLK];
  __shared__ unsigned short list[BLK];
  __shared__ int n_list;
  const int i = blockIdx.x;
  const long long id = ids[i];
  if (!ft_index_ok(id, vocab, status)) return;            // no table row to add into
  for (int j0 = 0; j0 < i; j0 += BLK) {                   // an earlier occurrence owns this token's row
    long long v[BLK / 128];                               // all loads issued before the first compare
#pragma unroll
    for (int k = 0; k < BLK / 128; ++k) {
      const int j = j0 + threadIdx.x + 128 * k;
      v[k] = j < i ? __ldg(ids + j) : -1;
    }
    int any = 0;
#pragma unroll
    for (int k = 0; k < BLK / 128; ++k) any |= (v[k] == id) ? 1 : 0;
    if (__syncthreads_or(any)) return;
  }
  float acc[8];                                           // this thread's column pairs: c = 2 * (tid + 128 k)
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = 2 * (threadIdx.x + 128 * k);
    float2 v = make_float2(0.f, 0.f);
    if (c < d) v = unpack_bf16(*reinterpret_cast<const uint32_t*>(dout + (size_t)i * d + c));
    acc[2 * k] = v.x;
    acc[2 * k + 1] = v.y;
  }
  for (int j0 = i + 1; j0 < rows; j0 += BLK) {
    long long v[BLK / 128];
#pragma unroll
    for (int k = 0; k < BLK / 128; ++k) {
      const int j = j0 + threadIdx.x + 128 * k;
      v[k] = j < rows ? __ldg(ids + j) : -1;
    }
    unsigned char m[BLK / 128];
    int any = 0;
#pragma unroll
    for (int k = 0; k < BLK / 128; ++k) {
      m[k] = (v[k] == id) ? 1 : 0;
      any |= m[k];
    }
    if (!__syncthreads_or(any)) continue;                 // (also orders the previous block's reads of list[])
#pragma unroll
    for (int k = 0; k < BLK / 128; ++k) match[threadIdx.x + 128 * k] = m[k];
    __syncthreads();
    // warp 0 compacts the matching positions of the block into an ascending list: lane l owns positions
    // [32 l, 32 l + 32), a warp scan of the counts gives each lane its place
    if (threadIdx.x < 32) {
      int cnt = 0;
      for (int t = 0; t < 32; ++t) cnt += match[32 * threadIdx.x + t];
      int pos = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, pos, o);
        if ((int)threadIdx.x >= o) pos += up;
      }
      if (threadIdx.x == 31) n_list = pos;
      pos -= cnt;
      for (int t = 0; t < 32; ++t)
        if (match[32 * threadIdx.x + t]) list[pos++] = (unsigned short)(32 * threadIdx.x + t);
    }
    __syncthreads();
    const int n = n_list;
    for (int q0 = 0; q0 < n; q0 += 4) {                   // four rows in flight, added in ascending position order
      float2 v[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool on = q0 + u < n;
        const size_t r = on ? (size_t)(j0 + list[q0 + u]) : 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = 2 * (threadIdx.x + 128 * k);
          v[u][k] = (on && c < d) ? unpack_bf16(*reinterpret_cast<const uint32_t*>(dout + r * d + c))
                                  : make_float2(0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (q0 + u < n) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            acc[2 * k] += v[u][k].x;
            acc[2 * k + 1] += v[u][k].y;
          }
        }
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = 2 * (threadIdx.x + 128 * k);
    if (c < d) {
      float* dst = dwte + (size_t)id * d + c;
      dst[0] += acc[2 * k];
      dst[1] += acc[2 * k + 1];
    }
  }
}
// dwpe[s, :] += sum over batch (ascending b) of dout[b*S + s, :]
__global__ void __launch_bounds__(128)
embedding_bwd_wpe_kernel(const __nv_bfloat16* __restrict__ dout, float* __restrict__ dwpe, int rows,
                         int S, int d) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x * 2; c < d; c += blockDim.x * 2) {
    float s0 = 0.f, s1 = 0.f;
    for (int r = s; r < rows; r += S) {
      float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(dout + (size_t)r * d + c));
      s0 += v.x;
      s1 += v.y;
    }
    dwpe[(size_t)s * d + c] += s0;
    dwpe[(size_t)s * d + c + 1] += s1;
  }
}

// ------------------------------------------------------------------------ AdamW
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow,
             const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
             long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
             float gscale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float g = grad[i] * gscale;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float mh = mi / bc1, vh = vi / bc2;
    float p = master[i];
    p -= p * lr * wd + lr * mh / (sqrtf(vh) + eps);
    master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
  }
}

// Device-resident optimizer clock so a captured CUDA graph replays a correct step:
// hyper = {lr, bias_correction1, bias_correction2, grad_scale}; step is incremented here.
__global__ void adamw_tick_kernel(long long* __restrict__ step, float* __restrict__ hyper, double b1,
                                  double b2) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const long long s = *step + 1;
    *step = s;
    hyper[1] = (float)(1.0 - pow(b1, (double)s));
    hyper[2] = (float)(1.0 - pow(b2, (double)s));
  }
}
// hyper[3] = min(1, max_norm / (sqrt(sumsq) + 1e-6))  (clip_grad_norm_, ft-nn/src/lib.rs:740)
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm,
                                  float* __restrict__ hyper, float* __restrict__ norm_out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float nrm = sqrtf(*sumsq);
    if (norm_out) *norm_out = nrm;
    const float c = max_norm / (nrm + 1e-6f);
    hyper[3] = c < 1.f ? c : 1.f;
  }
}
__global__ void __launch_bounds__(256)
adamw_dev_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow,
                 const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
                 long long n, const float* __restrict__ hyper, float b1, float b2, float eps,
                 float wd) {
  const float lr = hyper[0], bc1 = hyper[1], bc2 = hyper[2], gscale = hyper[3];
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float g[4] = {g4.x, g4.y, g4.z, g4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gi = g[k] * gscale;
      mm[k] = b1 * mm[k] + (1.f - b1) * gi;
      vv[k] = b2 * vv[k] + (1.f - b2) * gi * gi;
      const float mh = mm[k] / bc1, vh = vv[k] / bc2;
      pp[k] -= pp[k] * lr * wd + lr * mh / (sqrtf(vh) + eps);
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    if (shadow) {
      uint2 o;
      o.x = pack_bf16(pp[0], pp[1]);
      o.y = pack_bf16(pp[2], pp[3]);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = n4 << 2; i < n; ++i) {
      const float gi = grad[i] * gscale;
      const float mi = b1 * m[i] + (1.f - b1) * gi;
      const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
      m[i] = mi;
      v[i] = vi;
      float p = master[i];
      p -= p * lr * wd + lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
      master[i] = p;
      if (shadow) shadow[i] = __float2bfloat16(p);
    }
  }
}
__global__ void __launch_bounds__(256) fill_f32_kernel(float* __restrict__ x, long long n, float v) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = v;
}

// ------------------------------------------------------------------------ presenter / im2col
template <bool HALF>
__global__ void present_rgba8_kernel(const unsigned char* __restrict__ src, void* __restrict__ dst,
                                     int width, int height, long long row_bytes) {
  const int x = blockIdx.x * blockDim.x + threadIdx.x;
  const int y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= width || y >= height) return;
  const uchar4 px = *reinterpret_cast<const uchar4*>(src + (size_t)y * row_bytes + (size_t)x * 4);
  const float k = 1.f / 255.f;
  const size_t o = (size_t)y * width + x;
  if (HALF) {
    __half2* d = reinterpret_cast<__half2*>(dst) + o * 2;
    d[0] = __floats2half2_rn(px.x * k, px.y * k);
    d[1] = __floats2half2_rn(px.z * k, px.w * k);
  } else {
    reinterpret_cast<float4*>(dst)[o] = make_float4(px.x * k, px.y * k, px.z * k, px.w * k);
  }
}
__global__ void im2col_1d_kernel(const float* __restrict__ x, float* __restrict__ y, int t_in,
                                 int cin, int k, int stride, int pad, int t_out) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;  // index into cin*k
  const int t = blockIdx.y * blockDim.y + threadIdx.y;
  if (col >= cin * k || t >= t_out) return;
  const int c = col / k, kk = col % k;
  const int ti = t * stride + kk - pad;
  y[(size_t)t * cin * k + col] = (ti >= 0 && ti < t_in) ? x[(size_t)ti * cin + c] : 0.f;
}

static inline int ew_grid(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  const long long cap = 148 * 16;
  return (int)(b > cap ? cap : b);
}

}  // namespace ftk

#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<const __nv_bfloat16*>(p)
#define BFW(p) reinterpret_cast<__nv_bfloat16*>(p)
static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int ftk_gelu_fwd(const void* x, void* y, long long n, int tanh_form, void* stream) {
  if (n <= 0 || !al16(x) || !al16(y)) return -2;
  ew_bf16_kernel<0><<<ew_grid(n >> 3, 256), 256, 0, STREAM(stream)>>>(BF(x), nullptr, BFW(y), n, tanh_form);
  return (int)cudaGetLastError();
}
extern "C" int ftk_gelu_bwd(const void* x, const void* dy, void* dx, long long n, int tanh_form,
                            void* stream) {
  if (n <= 0 || !al16(x) || !al16(dy) || !al16(dx)) return -2;
  ew_bf16_kernel<1><<<ew_grid(n >> 3, 256), 256, 0, STREAM(stream)>>>(BF(x), BF(dy), BFW(dx), n, tanh_form);
  return (int)cudaGetLastError();
}
extern "C" int ftk_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n <= 0 || !al16(a) || !al16(b) || !al16(out)) return -2;
  ew_bf16_kernel<2><<<ew_grid(n >> 3, 256), 256, 0, STREAM(stream)>>>(BF(a), BF(b), BFW(out), n, 0);
  return (int)cudaGetLastError();
}
extern "C" int ftk_cast_f32_to_bf16(const float* x, void* y, long long n, void* stream) {
  if (n <= 0) return -2;
  cast_f32_bf16_kernel<<<ew_grid(n, 256), 256, 0, STREAM(stream)>>>(x, BFW(y), n);
  return (int)cudaGetLastError();
}
extern "C" int ftk_cast_bf16_to_f32(const void* x, float* y, long long n, int accumulate,
                                    void* stream) {
  if (n <= 0) return -2;
  cast_bf16_f32_kernel<<<ew_grid(n, 256), 256, 0, STREAM(stream)>>>(BF(x), y, n, accumulate);
  return (int)cudaGetLastError();
}
extern "C" int ftk_dropout_bf16(const void* x, void* y, long long n, float p,
                                unsigned long long seed, unsigned long long offset, void* stream) {
  if (n <= 0 || !(p >= 0.f && p < 1.f)) return -2;
  dropout_kernel<<<ew_grid((n + 3) >> 2, 256), 256, 0, STREAM(stream)>>>(BF(x), BFW(y), n, p, seed, offset);
  return (int)cudaGetLastError();
}
extern "C" int ftk_embedding_fwd(const long long* ids, const void* wte, const void* wpe, void* out,
                                 int rows, int S, int d, long long vocab, void* stream) {
  if (rows <= 0 || d % 8 || S <= 0 || vocab <= 0) return -2;
  embedding_fwd_kernel<<<rows, 128, 0, STREAM(stream)>>>(ids, BF(wte), BF(wpe), BFW(out), S, d, vocab,
                                                         ftk_status_word());
  return (int)cudaGetLastError();
}
extern "C" int ftk_embedding_bwd(const long long* sorted_ids, const int* order, const void* dout,
                                 float* dwte, float* dwpe, int rows, int S, int d, long long vocab, void* stream) {
  if (rows <= 0 || d % 2 || (dwte && vocab <= 0)) return -2;
  if (dwte)
    embedding_bwd_wte_kernel<<<rows, 128, 0, STREAM(stream)>>>(sorted_ids, order, rows, BF(dout), dwte, d, vocab,
                                                               ftk_status_word());
  if (dwpe) embedding_bwd_wpe_kernel<<<S, 128, 0, STREAM(stream)>>>(BF(dout), dwpe, rows, S, d);
  return (int)cudaGetLastError();
}
// Sort-free form: `ids` in their original order (int64 [rows]); d <= 1024 (wider tables use the sorted form).
extern "C" int ftk_embedding_bwd_scan(const long long* ids, const void* dout, float* dwte, float* dwpe, int rows,
                                      int S, int d, long long vocab, void* stream) {
  if (rows <= 0 || d % 2 || d > 1024 || (dwte && vocab <= 0)) return -2;
  if (dwte)
    embedding_bwd_wte_scan_kernel<<<rows, 128, 0, STREAM(stream)>>>(ids, rows, BF(dout), dwte, d, vocab,
                                                                    ftk_status_word());
  if (dwpe) embedding_bwd_wpe_kernel<<<S, 128, 0, STREAM(stream)>>>(BF(dout), dwpe, rows, S, d);
  return (int)cudaGetLastError();
}
extern "C" int ftk_adamw(float* master, void* shadow, const float* grad, float* m, float* v,
                         long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                         float bc2, float gscale, void* stream) {
  if (n <= 0) return -2;
  adamw_kernel<<<ew_grid(n, 256), 256, 0, STREAM(stream)>>>(master, BFW(shadow), grad, m, v, n, lr,
                                                             b1, b2, eps, wd, bc1, bc2, gscale);
  return (int)cudaGetLastError();
}
extern "C" int ftk_present_rgba8(const unsigned char* src, void* dst, int width, int height,
                                 long long row_bytes, int dst_half, void* stream) {
  if (width <= 0 || height <= 0 || row_bytes < (long long)width * 4 || (row_bytes & 3)) return -2;
  dim3 b(32, 8), g((width + 31) / 32, (height + 7) / 8);
  if (dst_half)
    present_rgba8_kernel<true><<<g, b, 0, STREAM(stream)>>>(src, dst, width, height, row_bytes);
  else
    present_rgba8_kernel<false><<<g, b, 0, STREAM(stream)>>>(src, dst, width, height, row_bytes);
  return (int)cudaGetLastError();
}
extern "C" int ftk_im2col_1d(const float* x, float* y, int t_in, int cin, int k, int stride,
                             int pad, int t_out, void* stream) {
  if (t_in <= 0 || cin <= 0 || k <= 0 || t_out <= 0 || stride <= 0) return -2;
  dim3 b(32, 8), g((cin * k + 31) / 32, (t_out + 7) / 8);
  im2col_1d_kernel<<<g, b, 0, STREAM(stream)>>>(x, y, t_in, cin, k, stride, pad, t_out);
  return (int)cudaGetLastError();
}

extern "C" int ftk_adamw_tick(long long* step, float* hyper, double b1, double b2, void* stream) {
  adamw_tick_kernel<<<1, 32, 0, STREAM(stream)>>>(step, hyper, b1, b2);
  return (int)cudaGetLastError();
}
extern "C" int ftk_clip_scale(const float* sumsq, float max_norm, float* hyper, float* norm_out,
                              void* stream) {
  clip_scale_kernel<<<1, 32, 0, STREAM(stream)>>>(sumsq, max_norm, hyper, norm_out);
  return (int)cudaGetLastError();
}
extern "C" int ftk_adamw_dev(float* master, void* shadow, const float* grad, float* m, float* v,
                             long long n, const float* hyper, float b1, float b2, float eps,
                             float wd, void* stream) {
  if (n <= 0) return -2;
  if (!al16(master) || !al16(grad) || !al16(m) || !al16(v) || (shadow && (reinterpret_cast<uintptr_t>(shadow) & 7)))
    return -3;
  adamw_dev_kernel<<<ew_grid(n >> 2, 256), 256, 0, STREAM(stream)>>>(master, BFW(shadow), grad, m, v, n,
                                                                      hyper, b1, b2, eps, wd);
  return (int)cudaGetLastError();
}
// One thread stores the GPU's nanosecond timer: a time mark inside a stream (or a captured graph),
// for measuring how long a stream sat between two points without a host round trip.
__global__ void timestamp_kernel(unsigned long long* out) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *out = t;
}
extern "C" int ftk_timestamp(unsigned long long* out, void* stream) {
  if (!out) return -2;
  timestamp_kernel<<<1, 1, 0, STREAM(stream)>>>(out);
  return (int)cudaGetLastError();
}
extern "C" int ftk_fill_f32(float* x, long long n, float v, void* stream) {
  if (n <= 0) return -2;
  fill_f32_kernel<<<ew_grid(n, 256), 256, 0, STREAM(stream)>>>(x, n, v);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Bounded-wait self test: one thread waits for *flag >= want with a cycle budget and, when the
// budget runs out, records FT_ERR_WAIT_PEER in the status word and returns - the same protocol
// every peer wait of the multi-GPU kernels follows.  The host test points it at a flag that
// nothing sets and checks that the status word reports the timeout while the context stays usable.
__global__ void wait_probe_kernel(const int* flag, int want, long long budget_cycles, int* status,
                                  long long* waited_cycles) {
  const long long t0 = clock64();
  int v;
  bool ok = true;
  while (true) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= want) break;
    __nanosleep(256);
    if (clock64() - t0 > budget_cycles) {
      atomicCAS(status, 0, ftk::FT_ERR_WAIT_PEER | (int(blockIdx.x) << 8));
      ok = false;
      break;
    }
  }
  if (waited_cycles) *waited_cycles = ok ? 0 : clock64() - t0;
}

extern "C" int ftk_wait_probe(const int* flag, int want, long long budget_cycles, long long* waited_cycles,
                              void* stream) {
  int* status = ftk_status_word();
  if (!status || !flag || budget_cycles <= 0 || budget_cycles > 4000000000ll) return -2;
  wait_probe_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, want, budget_cycles, status,
                                                                         waited_cycles);
  return (int)cudaGetLastError();
}
