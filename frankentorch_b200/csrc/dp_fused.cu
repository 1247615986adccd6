// Data-parallel optimizer step over NVLink peer memory: gradient reduce-scatter fused with
// the mean scaling, global-norm clipping and the sharded AdamW update, followed by the
// parameter all-gather written straight into every peer's parameter buffer.
//
// Every rank (one process per GPU) maps the flat gradient and parameter arenas of all peers
// (CUDA IPC).  Rank r owns shard r of the flat arena:
//
//   dp_reduce_shard      waits until every peer's gradients of this step are complete, then
//                        for each element of its shard loads the W peer values with plain
//                        P2P loads IN RANK ORDER (0..W-1), adds them in fp32 in that order
//                        (bit-identical on every run), scales by 1/W and keeps the result in
//                        a local fp32 shard buffer; per-CTA sums of squares go to a scratch.
//   dp_norm_exchange     one CTA: adds the per-CTA partials in index order, publishes the
//                        shard's sum of squares to every peer, waits for all W values and
//                        adds them in rank order -> global gradient norm -> clip factor.
//   dp_adamw_allgather   AdamW on the fp32 master shard (math of ft-optim/src/lib.rs:1040-1054)
//                        and P2P stores of the updated bf16 values into every rank's
//                        parameter arena; then signals "parameters written".
//   dp_wait_params       waits until every peer has written its shard into this rank's
//                        parameters (which also means every peer is done reading this rank's
//                        gradients, so the next backward may overwrite them).
//
// Flags are monotonically increasing step numbers read from the device-resident step counter,
// so a captured CUDA graph replays correctly.  Every wait on a peer flag is bounded: when the
// budget runs out the kernel records FT_ERR_WAIT_PEER in the status word and returns, and the
// host raises (strict mode) or falls back to NCCL (hardened mode).  Waits use plain acquire
// loads on peer-visible memory; no multimem / NVLS object is bound, so a peer that exits
// between steps cannot fault the other GPUs.
#include "ft_sm100.cuh"
#include "ftk_api.h"

namespace ftk {

constexpr int DP_MAX_RANKS = 16;
// ~2 s at 1.9 GHz: peers are released by the same host barrier, steady-state skew is far smaller
#ifndef FT_PEER_WAIT_CYCLES
#define FT_PEER_WAIT_CYCLES 4000000000ll
#endif

struct DpPeers {
  const float* grads[DP_MAX_RANKS];        // each rank's flat fp32 gradient arena
  __nv_bfloat16* params[DP_MAX_RANKS];     // each rank's flat bf16 parameter arena
  unsigned long long* flags[DP_MAX_RANKS]; // each rank's flag block: [3][DP_MAX_RANKS] u64
  float* slots[DP_MAX_RANKS];              // each rank's sumsq slots: [DP_MAX_RANKS] fp32
  int rank, world;
};

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
                                          int* status) {
  const long long t0 = clock64();
  while (ld_acquire_sys(p) < want) {
    if (clock64() - t0 > FT_PEER_WAIT_CYCLES) {
      atomicCAS(status, 0, FT_ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(200);
  }
  return true;
}
// One thread per peer signals (phase, my rank) = step on every rank, then waits for all
// peers' signals on its own flag block.  Returns false on timeout.  Called by one CTA.
__device__ bool signal_and_wait_all(const DpPeers& P, int phase, unsigned long long step, int* status,
                                    bool do_signal, bool do_wait) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (do_signal) {
    __threadfence_system();
    if ((int)threadIdx.x < P.world)
      st_release_sys(P.flags[threadIdx.x] + phase * DP_MAX_RANKS + P.rank, step);
  }
  if (do_wait && (int)threadIdx.x < P.world) {
    if (!wait_flag(P.flags[P.rank] + phase * DP_MAX_RANKS + threadIdx.x, step, status)) ok_s = 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// ----------------------------------------------------------------------------------- reduce
// grid: any; CTA 0 performs the start barrier and releases the others through `gate`.
__global__ void __launch_bounds__(256)
dp_reduce_shard_kernel(DpPeers P, float* __restrict__ gshard, float* __restrict__ partial_sumsq,
                       long long shard_len, const long long* __restrict__ step_ptr,
                       unsigned long long* __restrict__ gate, int* status) {
  __shared__ float red[33];
  const unsigned long long step = (unsigned long long)*step_ptr;
  // ---- start barrier: everyone's gradients of this step are complete
  if (blockIdx.x == 0) {
    const bool ok = signal_and_wait_all(P, 0, step, status, true, true);
    if (threadIdx.x == 0) st_release_sys(gate, ok ? step : ~0ull);
  }
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    unsigned long long g;
    while ((g = ld_acquire_sys(gate)) < step) {
      if (clock64() - t0 > 2 * FT_PEER_WAIT_CYCLES) {
        atomicCAS(status, 0, FT_ERR_WAIT_PEER);
        g = ~0ull;
        break;
      }
      __nanosleep(100);
    }
    red[32] = (g == ~0ull) ? -1.f : 1.f;
  }
  __syncthreads();
  const bool live = red[32] > 0.f;
  __syncthreads();
  float ss = 0.f;
  if (live) {
    const long long base = (long long)P.rank * shard_len;
    const float inv_w = 1.f / (float)P.world;
    const long long n4 = shard_len >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      float4 acc = reinterpret_cast<const float4*>(P.grads[0] + base)[i];
      for (int r = 1; r < P.world; ++r) {   // fixed rank order: replayable bits
        const float4 v = reinterpret_cast<const float4*>(P.grads[r] + base)[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      acc.x *= inv_w; acc.y *= inv_w; acc.z *= inv_w; acc.w *= inv_w;
      reinterpret_cast<float4*>(gshard)[i] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
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
    if (threadIdx.x == 0) partial_sumsq[blockIdx.x] = t;
  }
}

// ----------------------------------------------------------------------------------- norm
__global__ void __launch_bounds__(32)
dp_norm_exchange_kernel(DpPeers P, const float* __restrict__ partial_sumsq, int n_partial,
                        float max_norm, float* __restrict__ hyper, float* __restrict__ norm_out,
                        const long long* __restrict__ step_ptr, int* status) {
  const unsigned long long step = (unsigned long long)*step_ptr;
  float s = 0.f;
  if (threadIdx.x == 0)
    for (int i = 0; i < n_partial; ++i) s += partial_sumsq[i];   // index order
  s = __shfl_sync(0xffffffffu, s, 0);
  // thread r publishes to rank r and later signals rank r: its release store orders the slot write
  if ((int)threadIdx.x < P.world) P.slots[threadIdx.x][P.rank] = s;
  __syncwarp();
  const bool ok = signal_and_wait_all(P, 1, step, status, true, true);
  if (threadIdx.x == 0) {
    float tot = 0.f;
    if (ok)
      for (int r = 0; r < P.world; ++r) tot += reinterpret_cast<volatile float*>(P.slots[P.rank])[r];
    const float nrm = sqrtf(tot);
    if (norm_out) *norm_out = nrm;
    float c = 1.f;
    if (max_norm > 0.f) {
      c = max_norm / (nrm + 1e-6f);
      if (c > 1.f) c = 1.f;
    }
    hyper[3] = ok ? c : 0.f;   // a failed exchange turns the update into pure weight decay
  }
}

// ----------------------------------------------------------------------------------- update + all-gather
__global__ void __launch_bounds__(256)
dp_adamw_allgather_kernel(DpPeers P, float* __restrict__ master, float* __restrict__ m,
                          float* __restrict__ v, const float* __restrict__ gshard, long long shard_len,
                          const float* __restrict__ hyper, float b1, float b2, float eps, float wd) {
  const float lr = hyper[0], bc1 = hyper[1], bc2 = hyper[2], gscale = hyper[3];
  const long long base = (long long)P.rank * shard_len;
  const long long n4 = shard_len >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 g4 = reinterpret_cast<const float4*>(gshard)[i];
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
    uint2 o;
    o.x = pack_bf16(pp[0], pp[1]);
    o.y = pack_bf16(pp[2], pp[3]);
    for (int r = 0; r < P.world; ++r)   // all-gather: store into every rank's parameter arena
      reinterpret_cast<uint2*>(P.params[r] + base)[i] = o;
  }
}

// Signals "my shard is written everywhere" and waits for every peer's signal.
__global__ void __launch_bounds__(32)
dp_finish_kernel(DpPeers P, const long long* __restrict__ step_ptr, int* status) {
  const unsigned long long step = (unsigned long long)*step_ptr;
  signal_and_wait_all(P, 2, step, status, true, true);
}

struct DpState {
  DpPeers peers;
  unsigned long long* gate;   // local
  float* partial;             // local, DP_REDUCE_CTAS floats
};

}  // namespace ftk

using namespace ftk;

// ------------------------------------------------------------------------------------- IPC helpers
extern "C" int ftk_ipc_alloc(long long bytes, void** ptr_out, unsigned char* handle_out /*64*/) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
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
// `desc`: world pointers each for grads, params, flags, slots (this rank's view of every peer).
extern "C" int ftk_dp_step(const void* const* grads, void* const* params, void* const* flags,
                           void* const* slots, int rank, int world, float* gshard, float* partial,
                           int n_partial, unsigned long long* gate, float* master, float* m, float* v,
                           long long shard_len, const long long* step_ptr, float* hyper,
                           float* norm_out, float max_norm, float b1, float b2, float eps, float wd,
                           void* stream) {
  if (world < 1 || world > DP_MAX_RANKS || rank < 0 || rank >= world || (shard_len & 3) || n_partial < 1)
    return -2;
  DpPeers P;
  for (int r = 0; r < world; ++r) {
    P.grads[r] = reinterpret_cast<const float*>(grads[r]);
    P.params[r] = reinterpret_cast<__nv_bfloat16*>(params[r]);
    P.flags[r] = reinterpret_cast<unsigned long long*>(flags[r]);
    P.slots[r] = reinterpret_cast<float*>(slots[r]);
  }
  P.rank = rank;
  P.world = world;
  int* status = ftk_status_word();
  if (!status) return -6;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dp_reduce_shard_kernel<<<n_partial, 256, 0, s>>>(P, gshard, partial, shard_len, step_ptr, gate, status);
  dp_norm_exchange_kernel<<<1, 32, 0, s>>>(P, partial, n_partial, max_norm, hyper, norm_out, step_ptr, status);
  dp_adamw_allgather_kernel<<<n_partial, 256, 0, s>>>(P, master, m, v, gshard, shard_len, hyper, b1, b2, eps, wd);
  dp_finish_kernel<<<1, 32, 0, s>>>(P, step_ptr, status);
  return (int)cudaGetLastError();
}
