// Data-parallel optimizer step over NVLink peer memory, bucket by bucket: the gradient
// reduce-scatter (bf16 on the wire, fp32 sums) is fused with the mean scaling, the global-norm
// clipping and the sharded AdamW update, and the updated bf16 parameters are all-gathered by
// peer stores.  The host launches one bucket's kernels on a communication stream as soon as
// the backward pass has produced that bucket's last gradient, so the transfers run under the
// rest of the backward pass.
//
// Every rank (one process per GPU) maps every peer's inbox, parameter arena and flag block
// (CUDA IPC).  The flat parameter arena is cut into buckets [lo, hi) at fixed boundaries; each
// bucket is split into `world` equal shards of `shard` elements (a multiple of 8), rank r owns
// shard r of every bucket and keeps fp32 master / moments / reduced gradient for it only.
//
//   dp_push        (per bucket) reads this rank's fp32 gradients of the bucket, rounds them to
//                  the wire type and stores shard d into rank d's inbox, slot `rank`
//                  (16-byte peer stores, destinations visited in a rank-rotated order).  The
//                  last CTA to finish publishes "bucket b from rank r is in" on every peer.
//   dp_reduce      (per bucket) waits for the W arrival flags of the bucket, then adds the W
//                  inbox slots IN RANK ORDER (0..W-1) in fp32, scales by 1/W and writes the
//                  reduced fp32 shard; per-CTA sums of squares go to a scratch array.
//   dp_norm        one warp: adds the per-CTA partials in index order, publishes this rank's
//                  sum of squares to every peer, waits for all W values and adds them in rank
//                  order -> global gradient norm -> clip factor.  A rank whose earlier wait
//                  failed publishes a poison value instead, so every rank skips the update.
//   dp_update      AdamW on the fp32 master shards of buckets [b0, b1) (math of
//                  ft-optim/src/lib.rs:1040-1054) and peer stores of the updated bf16 values
//                  into every rank's parameter arena; the last CTA publishes "parameters of
//                  [b0, b1) from rank r are written".  The arithmetic is skipped when no update
//                  is pending (first step, or a poisoned step); the flag is published regardless,
//                  so the waits of a step never depend on whether the previous one was healthy.
//   dp_wait_params waits until every peer has published the parameters of a bucket range.
//
// The update may be deferred: dp_norm, which ends a step, stores the hyper-parameters of that
// step (learning rate, bias corrections, clip factor) next to a `pending` word, and the host
// launches dp_update for each bucket at the start of the NEXT step on the communication stream,
// in forward order, while the forward pass waits bucket by bucket (an event for the local part,
// dp_wait_params for the peers' parts).  The all-gather then runs under the forward pass.
//
// Waiting kernels only ever wait for kernels that were launched earlier on the same stream or
// that run on other GPUs, never for a later launch on this GPU.  Flags hold the sequence number
// of the step that set them (a device word the host advances once per step, so a captured CUDA
// graph replays correctly) and are never cleared.  Every wait on a peer flag is bounded: when
// the budget runs out the kernel records FT_ERR_WAIT_PEER in the status word, clears the step's
// `ok` word and returns; the host raises (strict mode) or falls back to NCCL (hardened mode).
// Plain acquire loads on peer-visible memory.  Optionally (params_mc) the parameter arenas are
// bound to one NVSwitch multicast address and dp_update broadcasts each updated bf16 value with a
// single multimem.st (egress bytes per rank: its shard once, not W-1 times); everything else,
// flags included, stays on ordinary peer stores.  Jobs that must survive a rank's exit run
// without it: a process that dies bound to a multicast object can fault its peers' GPUs.
//
// The reference has no distributed training (docs/planning/FEATURE_PARITY.md:176); the sums'
// fixed order carries its determinism contract (ft-autograd/src/lib.rs:20794-20819) across GPUs.
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

constexpr int DP_MAX_RANKS = FTK_DP_MAX_RANKS;
constexpr int DP_MAX_BUCKETS = FTK_DP_MAX_BUCKETS;
// ~2 s at 1.9 GHz: peers are released by the same host barrier, steady-state skew is far smaller
#ifndef FT_PEER_WAIT_CYCLES
#define FT_PEER_WAIT_CYCLES 4000000000ll
#endif
constexpr float DP_POISON = -1.0f;   // a sum of squares is never negative

struct DpPeers {
  void* inbox[DP_MAX_RANKS];               // each rank's inbox (wire type), see dp_push
  __nv_bfloat16* params[DP_MAX_RANKS];     // each rank's flat bf16 parameter arena
  unsigned long long* flags[DP_MAX_RANKS]; // each rank's flag block: [3][DP_MAX_BUCKETS][DP_MAX_RANKS] u64
  float* slots[DP_MAX_RANKS];              // each rank's sumsq slots: [DP_MAX_RANKS] fp32
  const FtkDpBucket* buckets;              // local device table
  __nv_bfloat16* params_mc;                // multicast address of the parameter arenas (NVLS), or null
  int rank, world, n_buckets;
};

__device__ __forceinline__ unsigned long long* flag_at(unsigned long long* base, int phase, int bucket, int src) {
  return base + ((long long)phase * DP_MAX_BUCKETS + bucket) * DP_MAX_RANKS + src;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Wait until flag >= want; false (and a status code) when the budget runs out.
__device__ __forceinline__ bool wait_flag(const unsigned long long* p, unsigned long long want,
                                          int* status, long long budget) {
  const long long t0 = clock64();
  while (ld_acquire_sys(p) < want) {
    if (clock64() - t0 > budget) {
      atomicCAS(status, 0, FT_ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(200);
  }
  return true;
}
// Threads 0..W-1 of the CTA each wait for one source's flag; returns (to every thread) whether all came.
__device__ __forceinline__ bool wait_all_sources(const DpPeers& P, int phase, int bucket,
                                                 unsigned long long want, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < P.world) {
    if (!wait_flag(flag_at(P.flags[P.rank], phase, bucket, threadIdx.x), want, status, FT_PEER_WAIT_CYCLES))
      ok_s = 0;
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  __syncthreads();
  return ok;
}
// Called by every CTA after its stores: the last one to arrive publishes (phase, bucket, rank) = seq
// on every peer.  `counter` is a local device word that returns to zero.
__device__ __forceinline__ void last_cta_publishes(const DpPeers& P, unsigned int* counter, int phase,
                                                   int bucket, unsigned long long seq) {
  __shared__ int last_s;
  __threadfence_system();           // this thread's peer stores are visible system-wide ...
  __syncthreads();                  // ... for every thread of the CTA
  if (threadIdx.x == 0) {
    __threadfence_system();
    last_s = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (last_s) {
    __threadfence_system();
    if ((int)threadIdx.x < P.world) st_release_sys(flag_at(P.flags[threadIdx.x], phase, bucket, P.rank), seq);
    if (threadIdx.x == 0) *counter = 0u;
  }
}

__device__ __forceinline__ void store_wire8(__nv_bfloat16* dst, const float4& a, const float4& b) {
  uint4 o;
  o.x = pack_bf16(a.x, a.y);
  o.y = pack_bf16(a.z, a.w);
  o.z = pack_bf16(b.x, b.y);
  o.w = pack_bf16(b.z, b.w);
  *reinterpret_cast<uint4*>(dst) = o;
}
__device__ __forceinline__ void store_wire8(float* dst, const float4& a, const float4& b) {
  reinterpret_cast<float4*>(dst)[0] = a;
  reinterpret_cast<float4*>(dst)[1] = b;
}
__device__ __forceinline__ void load_wire8(const __nv_bfloat16* src, float (&f)[8]) {
  const uint4 w = __ldcg(reinterpret_cast<const uint4*>(src));
  const float2 f0 = unpack_bf16(w.x), f1 = unpack_bf16(w.y), f2 = unpack_bf16(w.z), f3 = unpack_bf16(w.w);
  f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y; f[4] = f2.x; f[5] = f2.y; f[6] = f3.x; f[7] = f3.y;
}
__device__ __forceinline__ void load_wire8(const float* src, float (&f)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
  const float4 b = __ldcg(reinterpret_cast<const float4*>(src) + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// ----------------------------------------------------------------------------------- push
// Inbox layout on rank d (wire type): for bucket b the W slots start at W * off_b; slot s holds
// shard d of rank s's gradients of that bucket.
template <typename WireT>
__global__ void __launch_bounds__(256)
dp_push_kernel(DpPeers P, int b, const float* __restrict__ grads, unsigned int* counters,
               const long long* __restrict__ seq_ptr) {
  const FtkDpBucket bk = P.buckets[b];
  const unsigned long long seq = (unsigned long long)*seq_ptr;
  const long long vps = bk.shard >> 3;                       // 8-element vectors per shard
  const long long total = vps * P.world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int j = (int)(i / vps);
    const long long v = i - (long long)j * vps;
    const int d = (P.rank + 1 + j) % P.world;                // ranks start on different destinations
    const long long e = bk.lo + (long long)d * bk.shard + v * 8;
    if (e >= bk.hi) continue;                                // a short last shard (bucket ends are 8-aligned)
    const float4 a = __ldcs(reinterpret_cast<const float4*>(grads + e));
    const float4 c = __ldcs(reinterpret_cast<const float4*>(grads + e) + 1);
    WireT* dst = reinterpret_cast<WireT*>(P.inbox[d]) + (long long)P.world * bk.off +
                 (long long)P.rank * bk.shard + v * 8;
    store_wire8(dst, a, c);
  }
  last_cta_publishes(P, counters + b, 0, b, seq);
}

// ----------------------------------------------------------------------------------- reduce
template <typename WireT>
__global__ void __launch_bounds__(256)
dp_reduce_kernel(DpPeers P, int b, float* __restrict__ gshard, float* __restrict__ partial_sumsq,
                 int partial_stride, const long long* __restrict__ seq_ptr, int* ok_word, int* status) {
  __shared__ float red[32];
  const FtkDpBucket bk = P.buckets[b];
  const unsigned long long seq = (unsigned long long)*seq_ptr;
  const bool live = wait_all_sources(P, 0, b, seq, status);
  if (!live && threadIdx.x == 0) *ok_word = 0;
  float ss = 0.f;
  if (live) {
    const long long mine = bk.lo + (long long)P.rank * bk.shard;
    long long n_valid = bk.hi - mine;                         // elements of this rank's shard inside the bucket
    n_valid = n_valid < 0 ? 0 : (n_valid > bk.shard ? bk.shard : n_valid);
    const long long nv = n_valid >> 3;
    const float inv_w = 1.f / (float)P.world;
    const WireT* inbox = reinterpret_cast<const WireT*>(P.inbox[P.rank]) + (long long)P.world * bk.off;
    float* out = gshard + bk.off;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
      float acc[8], f[8];
      load_wire8(inbox + i * 8, acc);
      for (int s = 1; s < P.world; ++s) {                     // fixed rank order: replayable bits
        load_wire8(inbox + (long long)s * bk.shard + i * 8, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += f[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        acc[k] *= inv_w;
        ss += acc[k] * acc[k];
      }
      reinterpret_cast<float4*>(out + i * 8)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(out + i * 8)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
  // fixed-tree block reduction of the sum of squares
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) partial_sumsq[(long long)b * partial_stride + blockIdx.x] = t;
  }
  // the bucket's row of partials has room for the largest grid; entries beyond this launch's grid
  // must read as zero whatever an earlier, wider launch left there
  if (blockIdx.x == 0)
    for (int i = gridDim.x + threadIdx.x; i < partial_stride; i += blockDim.x)
      partial_sumsq[(long long)b * partial_stride + i] = 0.f;
}

// ----------------------------------------------------------------------------------- norm
// ok_word: 1 at the start of a step; any failed wait clears it.  After this kernel it is 1 only if
// every rank's reduces succeeded and every rank's sum of squares arrived.
__global__ void __launch_bounds__(32)
dp_norm_kernel(DpPeers P, const float* __restrict__ partial_sumsq, int n_partial, float max_norm,
               float* __restrict__ hyper, float* __restrict__ norm_out,
               const long long* __restrict__ seq_ptr, int* ok_word, int* status, int* pending,
               float* __restrict__ hyper_pending, const float* __restrict__ extra_sumsq) {
  const unsigned long long seq = (unsigned long long)*seq_ptr;
  float s = 0.f;
  if (threadIdx.x == 0) {
    for (int i = 0; i < n_partial; ++i) s += partial_sumsq[i];   // index order
    // squared norm of this rank's own (not replicated) gradients, e.g. tensor-parallel shards or
    // local experts: the global norm covers every parameter of the job, wherever it lives
    if (extra_sumsq) s += *extra_sumsq;
    if (*ok_word == 0) s = DP_POISON;
  }
  s = __shfl_sync(0xffffffffu, s, 0);
  // thread r publishes to rank r and then signals rank r: its release store orders the slot write
  if ((int)threadIdx.x < P.world) {
    P.slots[threadIdx.x][P.rank] = s;
    __threadfence_system();
    st_release_sys(flag_at(P.flags[threadIdx.x], 1, 0, P.rank), seq);
  }
  __syncwarp();
  bool ok = true;
  if ((int)threadIdx.x < P.world)
    ok = wait_flag(flag_at(P.flags[P.rank], 1, 0, threadIdx.x), seq, status, FT_PEER_WAIT_CYCLES);
  ok = __all_sync(0xffffffffu, ok);
  if (threadIdx.x == 0) {
    float tot = 0.f;
    if (ok)
      for (int r = 0; r < P.world; ++r) {
        const float v = reinterpret_cast<volatile float*>(P.slots[P.rank])[r];
        if (v < 0.f) ok = false;                      // a peer's step is poisoned: nobody updates
        tot += v;
      }
    const float nrm = ok ? sqrtf(tot) : 0.f;
    if (norm_out) *norm_out = nrm;
    float c = 1.f;
    if (max_norm > 0.f) {
      c = max_norm / (nrm + 1e-6f);
      if (c > 1.f) c = 1.f;
    }
    hyper[3] = ok ? c : 0.f;
    *ok_word = ok ? 1 : 0;
    // what the (possibly deferred) update of this step's gradients will use
    hyper_pending[0] = hyper[0];
    hyper_pending[1] = hyper[1];
    hyper_pending[2] = hyper[2];
    hyper_pending[3] = ok ? c : 0.f;
    *pending = ok ? 1 : 0;
  }
}

// ----------------------------------------------------------------------------------- update + all-gather
__global__ void __launch_bounds__(256)
dp_update_kernel(DpPeers P, int b0, int b1, float* __restrict__ master, float* __restrict__ m,
                 float* __restrict__ v, const float* __restrict__ gshard, const float* __restrict__ hyper,
                 float b1c, float b2c, float eps, float wd, unsigned int* counters,
                 const long long* __restrict__ seq_ptr, const int* __restrict__ pending) {
  // with nothing pending (first step, or a poisoned step) master, moments and parameters stay
  // exactly as they were; the flag below is published all the same
  const bool live = *pending != 0;
  const unsigned long long seq = (unsigned long long)*seq_ptr;
  const float lr = hyper[0], bc1 = hyper[1], bc2 = hyper[2], gscale = hyper[3];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int b = b0; live && b < b1; ++b) {
    const FtkDpBucket bk = P.buckets[b];
    const long long mine = bk.lo + (long long)P.rank * bk.shard;
    long long n_valid = bk.hi - mine;
    n_valid = n_valid < 0 ? 0 : (n_valid > bk.shard ? bk.shard : n_valid);
    const long long n4 = n_valid >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      const long long li = (bk.off >> 2) + i;               // index into the local shard arrays (float4)
      const float4 g4 = reinterpret_cast<const float4*>(gshard)[li];
      float4 m4 = reinterpret_cast<float4*>(m)[li];
      float4 v4 = reinterpret_cast<float4*>(v)[li];
      float4 p4 = reinterpret_cast<float4*>(master)[li];
      float g[4] = {g4.x, g4.y, g4.z, g4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w};
      float vv[4] = {v4.x, v4.y, v4.z, v4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gi = g[k] * gscale;
        mm[k] = b1c * mm[k] + (1.f - b1c) * gi;
        vv[k] = b2c * vv[k] + (1.f - b2c) * gi * gi;
        const float mh = mm[k] / bc1, vh = vv[k] / bc2;
        pp[k] -= pp[k] * lr * wd + lr * mh / (sqrtf(vh) + eps);
      }
      reinterpret_cast<float4*>(m)[li] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(v)[li] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      reinterpret_cast<float4*>(master)[li] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      uint2 o;
      o.x = pack_bf16(pp[0], pp[1]);
      o.y = pack_bf16(pp[2], pp[3]);
      if (P.params_mc) {
        // all-gather through the switch: one multimem store lands in every rank's parameter arena
        asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(
                         reinterpret_cast<uint2*>(P.params_mc + mine) + i),
                     "r"(o.x), "r"(o.y)
                     : "memory");
      } else {
        for (int j = 0; j < P.world; ++j) {   // all-gather: store into every rank's parameter arena
          const int r = (P.rank + j) % P.world;
          reinterpret_cast<uint2*>(P.params[r] + mine)[i] = o;
        }
      }
    }
  }
  last_cta_publishes(P, counters + DP_MAX_BUCKETS + b0, 2, b0, seq);
}

// Waits until every peer has published the parameters of the bucket range that starts at `b0`.
__global__ void __launch_bounds__(32)
dp_wait_params_kernel(DpPeers P, int b0, const long long* __restrict__ seq_ptr, int* ok_word, int* status) {
  const unsigned long long seq = (unsigned long long)*seq_ptr;
  bool ok = true;
  if ((int)threadIdx.x < P.world)
    ok = wait_flag(flag_at(P.flags[P.rank], 2, b0, threadIdx.x), seq, status, FT_PEER_WAIT_CYCLES);
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && threadIdx.x == 0) *ok_word = 0;
}

__global__ void dp_begin_step_kernel(long long* seq, int* ok_word) {
  *seq += 1;
  *ok_word = 1;
}
__global__ void dp_clear_pending_kernel(int* pending) { *pending = 0; }

}  // namespace ftk

using namespace ftk;

// ------------------------------------------------------------------------------------- IPC helpers
extern "C" int ftk_ipc_alloc(long long bytes, void** ptr_out, unsigned char* handle_out /*64*/) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return (int)e;
  }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return (int)e;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle_out, &h, 64);
  *ptr_out = p;
  return 0;
}
extern "C" int ftk_ipc_open(const unsigned char* handle, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return (int)cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int ftk_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int ftk_ipc_free(void* ptr) { return (int)cudaFree(ptr); }

// ------------------------------------------------------------------------------------- launchers
static int fill_peers(const FtkDpComm* c, DpPeers* P) {
  if (!c || c->world < 1 || c->world > DP_MAX_RANKS || c->rank < 0 || c->rank >= c->world ||
      c->n_buckets < 1 || c->n_buckets > DP_MAX_BUCKETS || !c->buckets || c->n_ctas < 1)
    return -2;
  for (int r = 0; r < c->world; ++r) {
    P->inbox[r] = c->inbox[r];
    P->params[r] = reinterpret_cast<__nv_bfloat16*>(c->params[r]);
    P->flags[r] = reinterpret_cast<unsigned long long*>(c->flags[r]);
    P->slots[r] = reinterpret_cast<float*>(c->slots[r]);
  }
  P->buckets = c->buckets;
  P->params_mc = reinterpret_cast<__nv_bfloat16*>(c->params_mc);
  P->rank = c->rank;
  P->world = c->world;
  P->n_buckets = c->n_buckets;
  return 0;
}

extern "C" int ftk_dp_begin_step(const FtkDpComm* c, void* stream) {
  if (!c || !c->seq || !c->ok_word) return -2;
  dp_begin_step_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(c->seq, c->ok_word);
  return (int)cudaPeekAtLastError();
}

// Push this rank's gradients of bucket b to the owners and reduce the shard this rank owns.
extern "C" int ftk_dp_bucket_reduce(const FtkDpComm* c, int b, const float* grads, int n_ctas, void* stream) {
  DpPeers P;
  int rc = fill_peers(c, &P);
  if (rc) return rc;
  if (b < 0 || b >= c->n_buckets || !grads || n_ctas < 1 || n_ctas > c->n_ctas) return -2;
  int* status = ftk_status_word();
  if (!status) return -6;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (c->wire_fp32) {
    dp_push_kernel<float><<<n_ctas, 256, 0, s>>>(P, b, grads, c->counters, c->seq);
    dp_reduce_kernel<float><<<n_ctas, 256, 0, s>>>(P, b, c->gshard, c->partial, c->n_ctas, c->seq, c->ok_word,
                                                   status);
  } else {
    dp_push_kernel<__nv_bfloat16><<<n_ctas, 256, 0, s>>>(P, b, grads, c->counters, c->seq);
    dp_reduce_kernel<__nv_bfloat16><<<n_ctas, 256, 0, s>>>(P, b, c->gshard, c->partial, c->n_ctas, c->seq,
                                                           c->ok_word, status);
  }
  return (int)cudaPeekAtLastError();
}

extern "C" int ftk_dp_norm(const FtkDpComm* c, float max_norm, float* hyper, float* norm_out,
                           const float* extra_sumsq, void* stream) {
  DpPeers P;
  int rc = fill_peers(c, &P);
  if (rc) return rc;
  int* status = ftk_status_word();
  if (!status) return -6;
  if (!c->pending || !c->hyper_pending) return -2;
  dp_norm_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      P, c->partial, c->n_buckets * c->n_ctas, max_norm, hyper, norm_out, c->seq, c->ok_word, status, c->pending,
      c->hyper_pending, extra_sumsq);
  return (int)cudaPeekAtLastError();
}

// Applies the pending update (hyper-parameters stored by the last ftk_dp_norm) to buckets [b0, b1).
extern "C" int ftk_dp_update(const FtkDpComm* c, int b0, int b1, float* master, float* m, float* v,
                             float beta1, float beta2, float eps, float wd, int n_ctas, void* stream) {
  DpPeers P;
  int rc = fill_peers(c, &P);
  if (rc) return rc;
  if (b0 < 0 || b1 > c->n_buckets || b0 >= b1 || n_ctas < 1 || !c->pending || !c->hyper_pending) return -2;
  dp_update_kernel<<<n_ctas, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      P, b0, b1, master, m, v, c->gshard, c->hyper_pending, beta1, beta2, eps, wd, c->counters, c->seq,
      c->pending);
  return (int)cudaPeekAtLastError();
}

extern "C" int ftk_dp_clear_pending(const FtkDpComm* c, void* stream) {
  if (!c || !c->pending) return -2;
  dp_clear_pending_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(c->pending);
  return (int)cudaPeekAtLastError();
}

extern "C" int ftk_dp_wait_params(const FtkDpComm* c, int b0, void* stream) {
  DpPeers P;
  int rc = fill_peers(c, &P);
  if (rc) return rc;
  if (b0 < 0 || b0 >= c->n_buckets) return -2;
  int* status = ftk_status_word();
  if (!status) return -6;
  dp_wait_params_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(P, b0, c->seq, c->ok_word, status);
  return (int)cudaPeekAtLastError();
}
