// Microbenchmarks of tcgen05.mma issue and execution rate on sm_100a (M = 128, cta_group::1, bf16).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -I frankentorch_b200/csrc -o mma_issue_rate benchmarks/mma_issue_rate.cu && ./mma_issue_rate
//
// Four experiments, each timing a stream of MMAs from one issuing thread per CTA with clock64:
//   minimal   descriptors loop-invariant, 16 MMAs unrolled: the rate of the tensor pipe itself
//   naive     both 64-bit descriptors rebuilt per instruction inside a rolled loop
//   stepped   descriptors stepped through a precomputed low word, with busy neighbour warps
//   neighbours  the minimal stream while eight other warps run ex2 / FMA / mbarrier / TMEM loops
// Every wait in these kernels is bounded by a cycle budget; operands are constant-filled shared
// memory, the results are discarded.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include "ft_sm100.cuh"
using namespace ftk;

namespace minimal {
// Cycles per tcgen05.mma with a minimal issue sequence: descriptors precomputed, 16 MMAs unrolled.
struct Res { long long issue, total; };

__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d), "l"(a), "l"(b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}

template <int N, int MODE, int NTHR>
__global__ void __launch_bounds__(128, 1) k(Res* out, int outer) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (warp == 0) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, MODE == 0 ? 0 : 1);
    const uint64_t a0 = make_smem_desc(smem_u32(smem), 16, 1024);
    const uint64_t b0 = MODE == 0 ? make_smem_desc(smem_u32(smem + 32768), 16, 1024)
                                  : make_smem_desc(smem_u32(smem + 32768), 16384, 1024);
    long long t0 = 0, t1 = 0, t2 = 0;
    uint32_t ph = 0;
    for (int rep = 0; rep < 3; ++rep) {
      __syncwarp();
      t0 = clock64();
      if (lane < NTHR) {   // NTHR = 1: one issuing thread
        for (int o = 0; o < outer; ++o) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int kk = i & 3;
            const uint32_t d = tm + ((i >> 2) & 1) * 256;
            const uint64_t bd = b0 + (MODE == 0 ? kk * 2 : kk * 128);
            if (MODE == 1) mma_ts(d, tm + 480 + kk * 8, bd, idesc);
            else mma_ss(d, a0 + kk * 2, bd, idesc);
          }
        }
        umma_commit(&bar);
      }
      __syncwarp();
      t1 = clock64();
      while (!mbar_try_wait(&bar, ph)) { if (clock64() - t1 > 200000000ll) break; }
      ph ^= 1;
      t2 = clock64();
    }
    if (lane == 0 && blockIdx.x == 0) { out->issue = t1 - t0; out->total = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

template <int N, int MODE>
void run(Res* d, const char* name) {
  cudaFuncSetAttribute(k<N, MODE, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  const int outer = 16;
  k<N, MODE, 1><<<148, 128, 96 * 1024>>>(d, outer);
  Res r; cudaError_t e = cudaMemcpy(&r, d, sizeof(r), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
  printf("%s N=%3d : issue %6.1f cyc/mma   total %6.1f cyc/mma  (ideal %d)\n", name, N, (double)r.issue / (16 * outer),
         (double)r.total / (16 * outer), N / 2);
}

int run() {
  Res* d; cudaMalloc(&d, sizeof(Res));
  run<64, 0>(d, "A smem K / B smem K ");
  run<128, 0>(d, "A smem K / B smem K ");
  run<256, 0>(d, "A smem K / B smem K ");
  run<64, 1>(d, "A tmem   / B smem MN");
  run<128, 1>(d, "A tmem   / B smem MN");
  run<256, 1>(d, "A tmem   / B smem MN");
  run<64, 2>(d, "A smem K / B smem MN");
  run<128, 2>(d, "A smem K / B smem MN");
  run<256, 2>(d, "A smem K / B smem MN");
  return 0;
}

}  // namespace minimal
namespace naive {
// Microbenchmark: cycles per tcgen05.mma (M=128, cta_group::1, bf16) for several N, operand
// sources and dependency patterns.  One CTA per SM slot requested; operands are zero-filled smem.

struct Res { long long issue, total; };

// mode: 0 = A smem K-major, B smem K-major (S-like); 1 = A tmem, B smem MN-major (PV-like);
//       2 = A smem K-major, B smem MN-major
// chain: 0 = all MMAs accumulate into one D; 1 = alternate two D tiles; 2 = groups of 4 then switch D
__global__ void __launch_bounds__(128, 1) k(Res* out, int N, int mode, int chain, int count) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (warp == 0) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, mode == 0 ? 0 : 1);
    const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32768);
    long long t0 = 0, t1 = 0, t2 = 0;
    uint32_t ph = 0;
    for (int rep = 0; rep < 3; ++rep) {
      __syncwarp();
      t0 = clock64();
      if (lane == 0) {
        for (int i = 0; i < count; ++i) {
          const int kk = i & 3;
          uint32_t d = tm;
          if (chain == 1) d += (i & 1) * 256;
          if (chain == 2) d += ((i >> 2) & 1) * 256;
          const uint64_t bdesc = mode == 0 ? make_smem_desc(b_addr + kk * 32, 16, 1024)
                                           : make_smem_desc(b_addr + kk * 2048, 16384, 1024);
          if (mode == 1) umma_bf16_ts(d, tm + 480 + kk * 8, bdesc, idesc, 1u);
          else umma_bf16(d, make_smem_desc(a_addr + kk * 32, 16, 1024), bdesc, idesc, 1u);
        }
        umma_commit(&bar);
      }
      __syncwarp();
      t1 = clock64();
      while (!mbar_try_wait(&bar, ph)) { if (clock64() - t1 > 200000000ll) break; }
      ph ^= 1;
      t2 = clock64();
    }
    if (lane == 0 && blockIdx.x == 0) { out->issue = t1 - t0; out->total = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, 512);
}

int run() {
  Res* d; cudaMalloc(&d, sizeof(Res));
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  const int count = 256;
  const char* mn[] = {"A smem K / B smem K ", "A tmem  / B smem MN ", "A smem K / B smem MN"};
  const char* cn[] = {"one D", "alt D", "4+4 D"};
  for (int ctas = 1; ctas <= 148; ctas += 147)
    for (int mode = 0; mode < 3; ++mode)
      for (int chain = 0; chain < 3; ++chain)
        for (int N = 64; N <= 256; N *= 2) {
          if (chain != 0 && N == 256 && false) continue;
          k<<<ctas, 128, 96 * 1024>>>(d, N, mode, chain, count);
          Res r; cudaError_t e = cudaMemcpy(&r, d, sizeof(r), cudaMemcpyDeviceToHost);
          if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
          printf("ctas %3d  %s  %s  N=%3d : issue %6.1f cyc/mma   total %6.1f cyc/mma  (ideal %d)\n", ctas, mn[mode],
                 cn[chain], N, (double)r.issue / count, (double)r.total / count, N / 2);
        }
  return 0;
}

}  // namespace naive
namespace stepped {
// MMA issue cost when descriptors change per instruction (as in attention), with and without
// busy neighbours on the issuing warp's scheduler.
struct Res { long long issue, total; float sink; };
__device__ __forceinline__ float ex2(float x) { float y; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// variant 0: slot-dependent descriptors via umma_bf16_lo; 1: same but issuing warp = warp 9 with elect
template <int N>
__global__ void __launch_bounds__(384, 1) k(Res* out, int outer, int imode, int issuer_warp, int* slots) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ volatile int done;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); done = 0; fence_mbar_init(); }
  if (warp == issuer_warp) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  float sink = 0.f;
  if (warp == issuer_warp) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, 0);
    const uint32_t q_addr = smem_u32(smem), kv_addr = smem_u32(smem + 32768);
    long long t0 = 0, t1 = 0, t2 = 0;
    uint32_t ph = 0;
    for (int rep = 0; rep < 3; ++rep) {
      __syncwarp();
      t0 = clock64();
      for (int o = 0; o < outer; ++o) {
        const int sl = slots[o & 7];          // runtime slot like the K/V ring
        if (lane == 0) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t a_lo = desc_lo(q_addr + t * 16384, 16), b_lo = desc_lo(kv_addr + sl * 16384, 16);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_bf16_lo(tm + 128 * t, a_lo + kk * 2, b_lo + kk * 2, idesc, kk != 0);
          }
        }
        __syncwarp();
      }
      if (lane == 0) umma_commit(&bar);
      __syncwarp();
      t1 = clock64();
      while (!mbar_try_wait(&bar, ph)) { if (clock64() - t1 > 200000000ll) break; }
      ph ^= 1;
      t2 = clock64();
    }
    done = 1;
    if (lane == 0 && blockIdx.x == 0) { out->issue = t1 - t0; out->total = t2 - t0; }
  } else if (warp < 8) {
    float x0 = lane * 0.001f, x1 = 0.5f, x2 = 0.25f, x3 = 0.125f;
    const long long tstart = clock64();
    for (int it = 0; it < 2000000; ++it) {
      if ((it & 15) == 0) { if (done) break; if (clock64() - tstart > 400000000ll) break; }
      if (imode == 1) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          x0 = ex2(fmaf(x0, 0.99f, -0.5f)) + x1; x1 = ex2(fmaf(x1, 0.98f, -0.25f)) + x2;
          x2 = ex2(fmaf(x2, 0.97f, -0.125f)) + x3; x3 = ex2(fmaf(x3, 0.96f, -0.0625f)) + x0;
        }
      } else if (imode == 2) {
#pragma unroll
        for (int u = 0; u < 16; ++u) { x0 = fmaf(x0, 0.99f, x1); x1 = fmaf(x1, 0.98f, x2); x2 = fmaf(x2, 0.97f, x3); x3 = fmaf(x3, 0.96f, x0); }
      } else break;
    }
    sink = x0 + x1 + x2 + x3;
  }
  if (sink == 123.456f && blockIdx.x == 0) out->sink = sink;
  tc_fence_before();
  __syncthreads();
  if (warp == issuer_warp) tmem_dealloc(tm, 512);
}

int run() {
  Res* d; cudaMalloc(&d, sizeof(Res));
  int h[8] = {0, 1, 2, 3, 4, 5, 6, 7}; int* ds; cudaMalloc(&ds, sizeof(h)); cudaMemcpy(ds, h, sizeof(h), cudaMemcpyHostToDevice);
  cudaFuncSetAttribute(k<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  const char* names[] = {"idle", "ex2+fma stream", "fma stream"};
  for (int iw = 9; iw <= 11; iw += 2)
    for (int im = 0; im < 3; ++im) {
      const int outer = 32;
      k<128><<<148, 384, 160 * 1024>>>(d, outer, im, iw, ds);
      Res r; cudaError_t e = cudaMemcpy(&r, d, sizeof(r), cudaMemcpyDeviceToHost);
      if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
      printf("N=128 SS, per-MMA descriptors, issuer warp %2d, neighbours: %-16s : issue %6.1f total %6.1f cyc/mma (ideal 64)\n", iw,
             names[im], (double)r.issue / (8 * outer), (double)r.total / (8 * outer));
    }
  return 0;
}

}  // namespace stepped
namespace neighbours {
// MMA rate under interference from other warps of the CTA (what an attention kernel's softmax
// warps do): ALU/MUFU streams, mbarrier polling, TMEM loads / stores.
struct Res { long long issue, total; float sink; };

__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d), "l"(a), "l"(b), "r"(idesc) : "memory");
}
__device__ __forceinline__ float ex2(float x) { float y; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

template <int N>
__global__ void __launch_bounds__(384, 1) k(Res* out, int outer, int imode, int nwarps_active) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar, never;
  __shared__ uint32_t slot;
  __shared__ volatile int done;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init(&never, 1); done = 0; fence_mbar_init(); }
  if (warp == 9) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  float sink = 0.f;
  if (warp == 9) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, 0);
    const uint64_t a0 = make_smem_desc(smem_u32(smem), 16, 1024);
    const uint64_t b0 = make_smem_desc(smem_u32(smem + 32768), 16, 1024);
    long long t0 = 0, t1 = 0, t2 = 0;
    uint32_t ph = 0;
    for (int rep = 0; rep < 3; ++rep) {
      __syncwarp();
      t0 = clock64();
      if (lane == 0) {
        for (int o = 0; o < outer; ++o) {
#pragma unroll
          for (int i = 0; i < 16; ++i) mma_ss(tm + ((i >> 2) & 1) * 128, a0 + (i & 3) * 2, b0 + (i & 3) * 2, idesc);
        }
        umma_commit(&bar);
      }
      __syncwarp();
      t1 = clock64();
      while (!mbar_try_wait(&bar, ph)) { if (clock64() - t1 > 200000000ll) break; }
      ph ^= 1;
      t2 = clock64();
    }
    done = 1;
    if (lane == 0 && blockIdx.x == 0) { out->issue = t1 - t0; out->total = t2 - t0; }
  } else if (warp < nwarps_active) {
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    float x0 = lane * 0.001f, x1 = 0.5f, x2 = 0.25f, x3 = 0.125f;
    uint32_t r[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = i;
    const long long tstart = clock64();
    for (int it = 0; it < 2000000; ++it) {
      if ((it & 15) == 0) { if (done) break; if (clock64() - tstart > 400000000ll) break; }
      if (imode == 1) {            // softmax-like math
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          x0 = ex2(fmaf(x0, 0.99f, -0.5f)) + x1; x1 = ex2(fmaf(x1, 0.98f, -0.25f)) + x2;
          x2 = ex2(fmaf(x2, 0.97f, -0.125f)) + x3; x3 = ex2(fmaf(x3, 0.96f, -0.0625f)) + x0;
        }
      } else if (imode == 2) {     // barrier polling
        if (mbar_try_wait(&never, 0)) x0 += 1.f;
      } else if (imode == 3) {     // TMEM loads (columns 256..383: not the accumulators)
        tmem_ld32(tm + 256 + lane_sel, r); tmem_ld32(tm + 288 + lane_sel, r); tmem_ld32(tm + 320 + lane_sel, r);
        tmem_ld32(tm + 352 + lane_sel, r); tmem_ld_wait();
        x0 += __uint_as_float(r[3]);
      } else if (imode == 4) {     // TMEM stores
        tmem_st32(tm + 384 + lane_sel, r); tmem_st32(tm + 416 + lane_sel, r); tmem_st_wait();
      } else if (imode == 5) {     // FMA-only stream
#pragma unroll
        for (int u = 0; u < 16; ++u) { x0 = fmaf(x0, 0.99f, x1); x1 = fmaf(x1, 0.98f, x2); x2 = fmaf(x2, 0.97f, x3); x3 = fmaf(x3, 0.96f, x0); }
      }
    }
    sink = x0 + x1 + x2 + x3;
  }
  if (sink == 123.456f && blockIdx.x == 0) out->sink = sink;
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tm, 512);
}

int run() {
  Res* d; cudaMalloc(&d, sizeof(Res));
  cudaFuncSetAttribute(k<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  cudaFuncSetAttribute(k<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
  const char* names[] = {"idle", "ex2+fma stream", "mbarrier polling", "tcgen05.ld", "tcgen05.st", "fma stream"};
  for (int nw = 8; nw >= 4; nw -= 4)
    for (int im = 0; im < 6; ++im) {
      const int outer = 16;
      k<128><<<148, 384, 96 * 1024>>>(d, outer, im, nw);
      Res r; cudaError_t e = cudaMemcpy(&r, d, sizeof(r), cudaMemcpyDeviceToHost);
      if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
      printf("N=128 SS, %d other warps: %-18s : %6.1f cyc/mma (ideal 64)\n", nw, names[im], (double)r.total / (16 * outer));
    }
  return 0;
}

}  // namespace neighbours

int main() {
  printf("== minimal issue sequence\n");
  if (minimal::run()) return 1;
  printf("== descriptors rebuilt per instruction (rolled loop)\n");
  if (naive::run()) return 1;
  printf("== descriptors stepped by a running low word, busy neighbours\n");
  if (stepped::run()) return 1;
  printf("== minimal stream under interference from eight other warps\n");
  if (neighbours::run()) return 1;
  return 0;
}
