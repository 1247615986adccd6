// Collectives through the NVSwitch multicast object (NVLS): every rank binds the same range of a
// symmetric allocation to one multicast address; a `multimem.st` to that address writes the value
// into every rank's copy with one egress transfer, and a `multimem.ld_reduce` returns the sum of
// all ranks' copies, added inside the switch.
//
//   nvls_allgather   each rank stores its chunk once (multimem.st, 16 bytes per thread) into slot
//                    `rank` of the gathered range on every GPU: egress bytes per rank are
//                    chunk, not (W-1) * chunk as with peer stores.
//   nvls_allreduce   two-shot, in place: rank r owns slice r of the range, loads the switch-side sum
//                    of the W copies of its slice (fp32, or bf16 pairs accumulated in fp32) and stores
//                    it back to every copy.  The order in which the switch adds the W values is the
//                    hardware's; it is the same on every run of the same topology, but it is not
//                    the ascending-rank order of the strict-mode kernels, so this kernel belongs to
//                    hardened mode only.
//
// Both kernels run the same two-barrier protocol over flags that live in the symmetric allocation
// and are written through ordinary peer (unicast) addresses with release stores:
//   enter : CTA 0 tells every peer "rank r entered call `seq`"; every CTA waits for the W entries
//           before it touches a peer's copy (the peers' earlier readers of the range are done and
//           their inputs are written: both were launched before their call `seq` in stream order).
//   leave : the last CTA to finish publishes "rank r finished call `seq`" on every peer and then
//           waits for the W finish flags, so that when the kernel has ended on a GPU all data for
//           that GPU has landed and later kernels on the stream may read it.
// Every wait is bounded; when the budget runs out the kernel records FT_ERR_WAIT_PEER, skips the
// data phase and returns.  Ranks must be on different GPUs (kernels that wait on one another
// cannot share one).  Tests of rank failure use the peer-store kernels instead: a process that
// dies while its memory is bound to a multicast object can fault its peers' GPUs.
//
// The reference has no collective of any kind (docs/planning/FEATURE_PARITY.md:176).
#include "ft_sm100.cuh"
#include "ftk_api.h"

extern "C" int* ftk_status_word(void);

namespace ftk {

#ifndef FT_PEER_WAIT_CYCLES
#define FT_PEER_WAIT_CYCLES 4000000000ll
#endif

struct NvlsArgs {
  char* mc;                                   // multicast address of the allocation
  char* local;                                // this rank's own mapping
  unsigned long long* flags[FTK_NVLS_MAX_RANKS];  // every rank's flag block [4][FTK_NVLS_MAX_RANKS] u64
  unsigned int* counter;                      // local device word, returns to zero
  int* status;
  int rank, world;
};

__device__ __forceinline__ void nv_st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long nv_ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 mm_ld_reduce_f32x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long* nv_flag(unsigned long long* base, int phase, int src) {
  return base + phase * FTK_NVLS_MAX_RANKS + src;
}

// Threads 0..W-1 each wait for one source's flag of `phase`; every thread learns whether all came.
__device__ __forceinline__ bool nv_wait_all(const NvlsArgs& a, int phase, unsigned long long seq) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < a.world) {
    const unsigned long long* p = nv_flag(a.flags[a.rank], phase, threadIdx.x);
    const long long t0 = clock64();
    while (nv_ld_acquire_sys(p) < seq) {
      if (clock64() - t0 > FT_PEER_WAIT_CYCLES) {
        atomicCAS(a.status, 0, FT_ERR_WAIT_PEER);
        ok_s = 0;
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  __syncthreads();
  return ok;
}

__device__ __forceinline__ bool nv_enter(const NvlsArgs& a, int phase, unsigned long long seq) {
  if (blockIdx.x == 0 && (int)threadIdx.x < a.world) {
    __threadfence_system();
    nv_st_release_sys(nv_flag(a.flags[threadIdx.x], phase, a.rank), seq);
  }
  return nv_wait_all(a, phase, seq);
}

// After a CTA's stores: the last CTA publishes the finish flag everywhere and waits for the peers'.
__device__ __forceinline__ void nv_leave(const NvlsArgs& a, int phase, unsigned long long seq) {
  __shared__ int last_s;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last_s = (atomicAdd(a.counter, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence_system();
  if ((int)threadIdx.x < a.world) nv_st_release_sys(nv_flag(a.flags[threadIdx.x], phase, a.rank), seq);
  if (threadIdx.x == 0) *a.counter = 0u;
  nv_wait_all(a, phase, seq);
}

__global__ void __launch_bounds__(256) nvls_allgather_kernel(NvlsArgs a, const uint4* __restrict__ src,
                                                             long long dst_off, long long n16,
                                                             unsigned long long seq) {
  const bool ok = nv_enter(a, 0, seq);
  if (ok) {
    char* dst = a.mc + dst_off + (long long)a.rank * n16 * 16;
    const long long stride = (long long)gridDim.x * blockDim.x;
    constexpr int U = 8;                              // loads in flight per thread
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n16; i0 += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < n16) v[u] = __ldcs(src + i0 + u * stride);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < n16) mm_st16(dst + (i0 + u * stride) * 16, v[u]);
    }
  }
  nv_leave(a, 1, seq);
}

template <bool kBf16>
__global__ void __launch_bounds__(256) nvls_allreduce_kernel(NvlsArgs a, long long off, long long n16,
                                                             unsigned long long seq) {
  const bool ok = nv_enter(a, 2, seq);
  if (ok) {
    const long long per = (n16 + a.world - 1) / a.world;
    const long long lo = per * a.rank;
    const long long hi = lo + per < n16 ? lo + per : n16;
    char* p = a.mc + off;
    const long long stride = (long long)gridDim.x * blockDim.x;
    constexpr int U = 4;                              // switch-side reductions in flight per thread
    for (long long i0 = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < hi; i0 += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) v[u] = kBf16 ? mm_ld_reduce_bf16x8(p + i * 16) : mm_ld_reduce_f32x4(p + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < hi) mm_st16(p + i * 16, v[u]);
      }
    }
  }
  nv_leave(a, 3, seq);
}

static int fill_args(const FtkNvlsComm* c, NvlsArgs* a) {
  if (!c || !c->mc || !c->local || !c->counter || c->world < 2 || c->world > FTK_NVLS_MAX_RANKS || c->rank < 0 ||
      c->rank >= c->world)
    return 1;
  a->mc = (char*)c->mc;
  a->local = (char*)c->local;
  for (int r = 0; r < c->world; ++r) {
    if (!c->flags[r]) return 1;
    a->flags[r] = (unsigned long long*)c->flags[r];
  }
  a->counter = c->counter;
  a->status = ftk_status_word();
  if (!a->status) return 1;
  a->rank = c->rank;
  a->world = c->world;
  return 0;
}

}  // namespace ftk

extern "C" {

// Every rank contributes `chunk_bytes` from `src` (any device memory of this rank); afterwards the range
// [dst_off, dst_off + world * chunk_bytes) of every rank's copy holds the W chunks in rank order.
int ftk_nvls_allgather(const FtkNvlsComm* c, const void* src, long long dst_off, long long chunk_bytes,
                       unsigned long long seq, int n_ctas, void* stream) {
  ftk::NvlsArgs a;
  if (ftk::fill_args(c, &a) || !src || ((uintptr_t)src & 15) || (dst_off & 15) || (chunk_bytes & 15) || chunk_bytes <= 0 ||
      seq == 0)
    return ftk::FT_ERR_BAD_ARG;
  if (n_ctas <= 0) n_ctas = 148;
  ftk::nvls_allgather_kernel<<<n_ctas, 256, 0, (cudaStream_t)stream>>>(a, (const uint4*)src, dst_off, chunk_bytes / 16, seq);
  return (int)cudaPeekAtLastError();
}

// In-place sum over ranks of `n_bytes` at byte offset `off` of the symmetric allocation (dtype 0: fp32, 1: bf16).
int ftk_nvls_allreduce(const FtkNvlsComm* c, long long off, long long n_bytes, int dtype, unsigned long long seq,
                       int n_ctas, void* stream) {
  ftk::NvlsArgs a;
  if (ftk::fill_args(c, &a) || (off & 15) || (n_bytes & 15) || n_bytes <= 0 || seq == 0 || dtype < 0 || dtype > 1)
    return ftk::FT_ERR_BAD_ARG;
  if (n_ctas <= 0) n_ctas = 148;
  if (dtype == 1)
    ftk::nvls_allreduce_kernel<true><<<n_ctas, 256, 0, (cudaStream_t)stream>>>(a, off, n_bytes / 16, seq);
  else
    ftk::nvls_allreduce_kernel<false><<<n_ctas, 256, 0, (cudaStream_t)stream>>>(a, off, n_bytes / 16, seq);
  return (int)cudaPeekAtLastError();
}

}  // extern "C"
