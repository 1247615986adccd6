// Mixture-of-experts routing and the two all-to-alls of expert parallelism, written as kernels
// that permute and move rows over NVLink peer memory in one pass (no staging copy, no library
// all-to-all).  The reference has no MoE layer; the primitives it is assembled from are top-k
// (ft-kernel-cpu/src/lib.rs:22808), row softmax (:18350), index_select and scatter_add.
//
//   route    : softmax over E expert logits, top-2 (ties -> lower index), gates renormalised
//              over the chosen pair.
//   slots    : position of every (token, k) among the rows its rank sends to that expert,
//              counted in (token, k) order by a block scan - deterministic; entries past the
//              per-source capacity are dropped (slot -1).
//   dispatch : row (token, k) -> recv[expert rank][expert local][source rank][slot][:], written
//              with peer stores and optionally scaled (backward sends gate * dOut); then the
//              senders raise one flag per destination, every rank waits (bounded) for all its
//              sources and zeroes the unused rows of its own buffer, so the expert GEMMs and
//              their weight gradients see exact zeros there.
//   combine  : out[token] = w0 * y[e0][slot0] + w1 * y[e1][slot1] (k = 0 first, then k = 1),
//              rows pulled from the expert ranks with peer loads after a ready handshake.
//
// Flags store the epoch (use count) of the call that set them and are never cleared.
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

constexpr long long MOE_WAIT_CYCLES = 4000000000ll;
constexpr int MOE_MAX_E = 64;

__device__ __forceinline__ int moe_ld_acq_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void moe_st_rel_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for *p >= want; on timeout records FT_ERR_WAIT_PEER and returns false.
__device__ __forceinline__ bool moe_wait(const int* p, int want, int* status) {
  const long long t0 = clock64();
  while (moe_ld_acq_sys(p) < want) {
    __nanosleep(128);
    if (clock64() - t0 > MOE_WAIT_CYCLES) {
      atomicCAS(status, 0, FT_ERR_WAIT_PEER | (int(blockIdx.x) << 8));
      return false;
    }
  }
  return true;
}

// ------------------------------------------------------------------ route
// One thread per token.  logits [T, ld] fp32 (first E columns), probs [T, E] fp32, idx [T, 2]
// int32, gate [T, 2] fp32.
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, float* __restrict__ probs, int* __restrict__ idx,
                 float* __restrict__ gate, int T, int E, int ld) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* lp = logits + (long long)t * ld;
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, lp[e]);
  if (!(mx > -INFINITY && mx < INFINITY)) mx = 0.f;     // non-finite guard
  float sum = 0.f;
  for (int e = 0; e < E; ++e) sum += __expf(lp[e] - mx);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  int i0 = 0, i1 = -1;
  float p0 = -1.f, p1 = -1.f;
  for (int e = 0; e < E; ++e) {
    const float pe = __expf(lp[e] - mx) * inv;
    probs[(long long)t * E + e] = pe;
    if (pe > p0) {
      p1 = p0; i1 = i0;
      p0 = pe; i0 = e;
    } else if (pe > p1) {
      p1 = pe; i1 = e;
    }
  }
  if (i1 < 0) { i1 = (i0 + 1) % E; p1 = 0.f; }
  const float s = p0 + p1;
  idx[2 * t] = i0;
  idx[2 * t + 1] = i1;
  gate[2 * t] = s > 0.f ? p0 / s : 0.5f;
  gate[2 * t + 1] = s > 0.f ? p1 / s : 0.5f;
}

// d_logits (bf16 [T, ld], columns >= E zeroed) from d_gate: g_k = p_k / (p_a + p_b),
// p = softmax(logits).
__global__ void __launch_bounds__(256)
moe_route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ idx,
                     const float* __restrict__ d_gate, __nv_bfloat16* __restrict__ d_logits, int T, int E,
                     int ld) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* pp = probs + (long long)t * E;
  const int a = idx[2 * t], b = idx[2 * t + 1];
  const float pa = pp[a], pb = pp[b], s = pa + pb;
  const float da = d_gate[2 * t], db = d_gate[2 * t + 1];
  float dpa = 0.f, dpb = 0.f;
  if (s > 0.f) {
    const float is2 = 1.f / (s * s);
    dpa = (da - db) * pb * is2;       // d g_a / d p_a = p_b / s^2, d g_b / d p_a = -p_b / s^2
    dpb = (db - da) * pa * is2;
  }
  const float dot = pa * dpa + pb * dpb;
  for (int e = 0; e < E; ++e) {
    const float dp = e == a ? dpa : (e == b ? dpb : 0.f);
    d_logits[(long long)t * ld + e] = __float2bfloat16(pp[e] * (dp - dot));
  }
  for (int e = E; e < ld; ++e) d_logits[(long long)t * ld + e] = __float2bfloat16(0.f);
}

// ------------------------------------------------------------------ slots
// grid = E CTAs of 1024 threads.  Entry j = 2 t + k; slot[j] = number of earlier entries routed
// to the same expert, or -1 when that number reaches `capacity`.  counts[e] = rows kept.
__global__ void __launch_bounds__(1024)
moe_slots_kernel(const int* __restrict__ idx, int* __restrict__ slot, int* __restrict__ counts,
                 int T, int capacity) {
  __shared__ int part[1024];
  const int e = blockIdx.x;
  const int n = 2 * T;
  const int per = (n + 1023) / 1024;
  const int j0 = threadIdx.x * per, j1 = min(n, j0 + per);
  int c = 0;
  for (int j = j0; j < j1; ++j) c += (idx[j] == e);
  part[threadIdx.x] = c;
  __syncthreads();
  // inclusive Hillis-Steele scan over 1024 partial counts (fixed order)
  for (int d = 1; d < 1024; d <<= 1) {
    const int v = threadIdx.x >= d ? part[threadIdx.x - d] : 0;
    __syncthreads();
    part[threadIdx.x] += v;
    __syncthreads();
  }
  int pos = part[threadIdx.x] - c;
  for (int j = j0; j < j1; ++j) {
    if (idx[j] == e) {
      slot[j] = pos < capacity ? pos : -1;
      ++pos;
    }
  }
  if (threadIdx.x == 1023) counts[e] = min(part[1023], capacity);
}

// ------------------------------------------------------------------ dispatch
struct MoeDispatchArgs {
  const __nv_bfloat16* x;      // [T, d] rows to send (token major)
  const int* idx;              // [T, 2]
  const int* slot;             // [T, 2]
  const float* scale;          // [T, 2] or null (1.0)
  const int* counts;           // [E] rows this rank sends to each expert
  __nv_bfloat16* recv[FTK_MAX_RANKS];   // recv buffer of every rank: [E_local][world][C][d]
  int* recv_counts[FTK_MAX_RANKS];      // [E_local][world] on every rank
  int* arrive[FTK_MAX_RANKS];           // [world] on every rank (one word per source)
  int* ticket;                 // local word, zero between launches
  const int* epoch;
  int T, d, E, e_local, capacity, rank, world;
  int* status;
};

__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const MoeDispatchArgs a) {
  __shared__ int s_last, s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int epoch = *a.epoch;
  const int vec = a.d >> 3;                       // 16-byte vectors per row
  // phase 1: permute + send
  for (long long j = (long long)blockIdx.x * wpb + warp; j < 2ll * a.T; j += (long long)gridDim.x * wpb) {
    const int sl = a.slot[j];
    if (sl < 0) continue;
    const int e = a.idx[j];
    const int dst = e / a.e_local, el = e - dst * a.e_local;
    const float sc = a.scale ? a.scale[j] : 1.f;
    const uint4* src = reinterpret_cast<const uint4*>(a.x + (j >> 1) * a.d);
    uint4* out = reinterpret_cast<uint4*>(
        a.recv[dst] + ((((long long)el * a.world + a.rank) * a.capacity + sl) * a.d));
    for (int v = lane; v < vec; v += 32) {
      uint4 u = src[v];
      if (a.scale) {
        float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z), f3 = unpack_bf16(u.w);
        u.x = pack_bf16(f0.x * sc, f0.y * sc);
        u.y = pack_bf16(f1.x * sc, f1.y * sc);
        u.z = pack_bf16(f2.x * sc, f2.y * sc);
        u.w = pack_bf16(f3.x * sc, f3.y * sc);
      }
      out[v] = u;
    }
  }
  // the last CTA to finish sending publishes counts and raises the arrival flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int tk = atomicAdd(a.ticket, 1);
    s_last = (tk == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
      const int dst = e / a.e_local, el = e - dst * a.e_local;
      a.recv_counts[dst][el * a.world + a.rank] = a.counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < a.world) moe_st_rel_sys(a.arrive[threadIdx.x] + a.rank, epoch);
    if (threadIdx.x == 0) *a.ticket = 0;
  }
  // phase 2: wait for every source, then zero the rows nobody wrote
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < a.world) {
    if (!moe_wait(a.arrive[a.rank] + threadIdx.x, epoch, a.status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int blocks = a.e_local * a.world;
  const int* rc = a.recv_counts[a.rank];
  __nv_bfloat16* mine = a.recv[a.rank];
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long r = (long long)blockIdx.x * wpb + warp; r < (long long)blocks * a.capacity;
       r += (long long)gridDim.x * wpb) {
    const int blk = (int)(r / a.capacity), sl = (int)(r - (long long)blk * a.capacity);
    if (sl < __ldcg(rc + blk)) continue;
    uint4* row = reinterpret_cast<uint4*>(mine + r * a.d);
    for (int v = lane; v < vec; v += 32) row[v] = z;
  }
}

// ------------------------------------------------------------------ combine
struct MoeCombineArgs {
  const __nv_bfloat16* y[FTK_MAX_RANKS];   // expert outputs of every rank: [E_local][world][C][d]
  int* ready[FTK_MAX_RANKS];               // [world] on every rank (one word per expert rank)
  const int* idx;                          // [T, 2]
  const int* slot;                         // [T, 2]
  const float* gate;                       // [T, 2] or null (weights 1)
  __nv_bfloat16* out;                      // [T, d]
  const __nv_bfloat16* resid;              // [T, d] or null, added last
  __nv_bfloat16* rows;                     // [T, 2, d] or null: the pulled rows, kept for backward
  const int* epoch;
  int T, d, e_local, capacity, rank, world;
  int* status;
};

__global__ void __launch_bounds__(256)
moe_combine_kernel(const MoeCombineArgs a) {
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int epoch = *a.epoch;
  // this rank's expert outputs were produced by earlier kernels of this stream: announce them
  if (blockIdx.x == 0 && (int)threadIdx.x < a.world) {
    __threadfence_system();
    moe_st_rel_sys(a.ready[threadIdx.x] + a.rank, epoch);
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < a.world) {
    if (!moe_wait(a.ready[a.rank] + threadIdx.x, epoch, a.status)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int vec = a.d >> 3;
  for (long long t = (long long)blockIdx.x * wpb + warp; t < a.T; t += (long long)gridDim.x * wpb) {
    const uint4* rp[2];
    float w[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int sl = a.slot[2 * t + k];
      const int e = a.idx[2 * t + k];
      const int src = e / a.e_local, el = e - src * a.e_local;
      rp[k] = sl < 0 ? nullptr
                     : reinterpret_cast<const uint4*>(
                           a.y[src] + ((((long long)el * a.world + a.rank) * a.capacity + sl) * a.d));
      w[k] = a.gate ? a.gate[2 * t + k] : 1.f;
    }
    for (int v = lane; v < vec; v += 32) {
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      const uint4 u0 = rp[0] ? __ldcg(rp[0] + v) : z;
      const uint4 u1 = rp[1] ? __ldcg(rp[1] + v) : z;
      if (a.rows) {
        reinterpret_cast<uint4*>(a.rows + (2 * t) * a.d)[v] = u0;
        reinterpret_cast<uint4*>(a.rows + (2 * t + 1) * a.d)[v] = u1;
      }
      const uint32_t* p0 = &u0.x;
      const uint32_t* p1 = &u1.x;
      uint4 rs = z;
      if (a.resid) rs = reinterpret_cast<const uint4*>(a.resid + t * a.d)[v];
      const uint32_t* pr = &rs.x;
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f0 = unpack_bf16(p0[i]), f1 = unpack_bf16(p1[i]), fr = unpack_bf16(pr[i]);
        // fixed order: k = 0, then k = 1, then the residual
        const float x0 = (w[0] * f0.x + w[1] * f1.x) + fr.x;
        const float x1 = (w[0] * f0.y + w[1] * f1.y) + fr.y;
        o[i] = pack_bf16(x0, x1);
      }
      if (a.out) reinterpret_cast<uint4*>(a.out + t * a.d)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// d_gate[t, k] = <g[t, :], rows[t, k, :]>; one warp per token.
__global__ void __launch_bounds__(256)
moe_gate_grad_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ rows,
                     float* __restrict__ d_gate, int T, int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float dot0 = 0.f, dot1 = 0.f;
  for (int v = lane; v < (d >> 3); v += 32) {
    const uint4 ug = reinterpret_cast<const uint4*>(g + t * d)[v];
    const uint4 u0 = reinterpret_cast<const uint4*>(rows + (2 * t) * d)[v];
    const uint4 u1 = reinterpret_cast<const uint4*>(rows + (2 * t + 1) * d)[v];
    const uint32_t *pg = &ug.x, *p0 = &u0.x, *p1 = &u1.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 fg = unpack_bf16(pg[i]), f0 = unpack_bf16(p0[i]), f1 = unpack_bf16(p1[i]);
      dot0 += fg.x * f0.x + fg.y * f0.y;
      dot1 += fg.x * f1.x + fg.y * f1.y;
    }
  }
#pragma unroll
  for (int dlt = 16; dlt > 0; dlt >>= 1) {
    dot0 += __shfl_xor_sync(0xffffffffu, dot0, dlt);
    dot1 += __shfl_xor_sync(0xffffffffu, dot1, dlt);
  }
  if (lane == 0) {
    d_gate[2 * t] = dot0;
    d_gate[2 * t + 1] = dot1;
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_moe_route(const float* logits, float* probs, int* idx, float* gate, int T, int E,
                             int ld, void* stream) {
  if (T <= 0 || E < 2 || E > MOE_MAX_E || ld < E) return -2;
  moe_route_kernel<<<(T + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, probs, idx,
                                                                                       gate, T, E, ld);
  return (int)cudaGetLastError();
}

extern "C" int ftk_moe_route_bwd(const float* probs, const int* idx, const float* d_gate, void* d_logits,
                                 int T, int E, int ld, void* stream) {
  if (T <= 0 || E < 2 || E > MOE_MAX_E || ld < E) return -2;
  moe_route_bwd_kernel<<<(T + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      probs, idx, d_gate, reinterpret_cast<__nv_bfloat16*>(d_logits), T, E, ld);
  return (int)cudaGetLastError();
}

extern "C" int ftk_moe_slots(const int* idx, int* slot, int* counts, int T, int E, int capacity,
                             void* stream) {
  if (T <= 0 || E < 1 || E > MOE_MAX_E || capacity <= 0) return -2;
  moe_slots_kernel<<<E, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(idx, slot, counts, T, capacity);
  return (int)cudaGetLastError();
}

extern "C" int ftk_moe_dispatch(const FtkMoeDesc* m, const void* x, const float* scale, void* const* recv,
                                int* const* recv_counts, int* const* arrive, void* stream) {
  if (!m || !x || m->world < 1 || m->world > FTK_MAX_RANKS || (m->d % 8) || m->E % m->world) return -2;
  MoeDispatchArgs a;
  a.x = reinterpret_cast<const __nv_bfloat16*>(x);
  a.idx = m->idx; a.slot = m->slot; a.scale = scale; a.counts = m->counts;
  for (int r = 0; r < m->world; ++r) {
    a.recv[r] = reinterpret_cast<__nv_bfloat16*>(recv[r]);
    a.recv_counts[r] = recv_counts[r];
    a.arrive[r] = arrive[r];
  }
  a.ticket = m->ticket; a.epoch = m->epoch;
  a.T = m->T; a.d = m->d; a.E = m->E; a.e_local = m->E / m->world; a.capacity = m->capacity;
  a.rank = m->rank; a.world = m->world;
  a.status = ftk_status_word();
  if (!a.status) return -6;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // both phases of the kernel need every CTA resident: 2 CTAs of 256 threads per SM
  moe_dispatch_kernel<<<2 * sms, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

extern "C" int ftk_moe_combine(const FtkMoeDesc* m, void* const* y, int* const* ready, const float* gate,
                               void* out, const void* resid, void* rows, void* stream) {
  if (!m || m->world < 1 || m->world > FTK_MAX_RANKS || (m->d % 8) || m->E % m->world) return -2;
  MoeCombineArgs a;
  for (int r = 0; r < m->world; ++r) {
    a.y[r] = reinterpret_cast<const __nv_bfloat16*>(y[r]);
    a.ready[r] = ready[r];
  }
  a.idx = m->idx; a.slot = m->slot; a.gate = gate;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
  a.rows = reinterpret_cast<__nv_bfloat16*>(rows);
  a.epoch = m->epoch;
  a.T = m->T; a.d = m->d; a.e_local = m->E / m->world; a.capacity = m->capacity;
  a.rank = m->rank; a.world = m->world;
  a.status = ftk_status_word();
  if (!a.status) return -6;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  moe_combine_kernel<<<4 * sms, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

extern "C" int ftk_moe_gate_grad(const void* g, const void* rows, float* d_gate, int T, int d, void* stream) {
  if (T <= 0 || (d % 8)) return -2;
  moe_gate_grad_kernel<<<(T + 7) / 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(g), reinterpret_cast<const __nv_bfloat16*>(rows), d_gate, T, d);
  return (int)cudaGetLastError();
}
