// ftk_colsum_bf16_noalloc: the bias-gradient column sum with its scratch memory in a
// file-scope device array, for callers that cannot allocate (see ftk_noalloc.h).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "ftk_noalloc.h"

namespace {

constexpr int kRowsPerBlock = 64;   // rows summed by one thread before the cross-block pass
constexpr int kMaxDevices = 64;
constexpr long long kMaxGridY = 65535;

// Scratch for the per-row-block partial sums.  In host code this name is only a stand-in
// for the symbol; its device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_colsum_scratch[FTK_COLSUM_NOALLOC_MAX_FLOATS];

std::mutex g_mu;
float* g_scratch_addr[kMaxDevices] = {nullptr};

__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

// partial[blk][c] = sum of x[r, c] over the 64 rows of block blk (ascending r)
__global__ void __launch_bounds__(128)
colsum_partial_noalloc(const __nv_bfloat16* __restrict__ x, float* __restrict__ partial, int rows,
                       int cols, long long ld) {
  const int c = (blockIdx.x * 128 + threadIdx.x) * 2;
  const int blk = blockIdx.y;
  if (c >= cols) return;
  const int r0 = blk * kRowsPerBlock;
  const int r1 = min(rows, r0 + kRowsPerBlock);
  float s0 = 0.f, s1 = 0.f;
  for (int r = r0; r < r1; ++r) {
    const float2 v = bf16x2_to_float2(*reinterpret_cast<const uint32_t*>(x + (size_t)r * ld + c));
    s0 += v.x;
    s1 += v.y;
  }
  partial[(size_t)blk * cols + c] = s0;
  if (c + 1 < cols) partial[(size_t)blk * cols + c + 1] = s1;
}
// out[c] (+)= partial[0][c] + partial[1][c] + ...  (ascending blk)
__global__ void colsum_final_noalloc(const float* __restrict__ partial, float* __restrict__ out,
                                     int cols, int nblk, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int b = 0; b < nblk; ++b) s += partial[(size_t)b * cols + c];
  out[c] = accumulate ? out[c] + s : s;
}

// Once per device, with that device current: resolve the scratch array's device address.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch) != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_scratch_addr[dev] = p;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int ftk_colsum_bf16_noalloc(const void* x, float* out, int rows, int cols, long long ld,
                                       int accumulate, void* stream) {
  if (!x || !out || rows <= 0 || cols <= 0 || (cols % 2) || (ld % 2) || ld < cols)
    return FTK_NOALLOC_ERR_BAD_ARG;
  // the kernel reads x as 32-bit bf16 pairs and out as fp32 words: a pointer that is not 4-byte
  // aligned (a bf16 view that starts at an odd element) would fault on the device, so refuse it here
  if ((reinterpret_cast<uintptr_t>(x) & 3u) || (reinterpret_cast<uintptr_t>(out) & 3u))
    return FTK_NOALLOC_ERR_BAD_ARG;
  const long long nblk = ((long long)rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (nblk * (long long)cols > (long long)FTK_COLSUM_NOALLOC_MAX_FLOATS)
    return FTK_NOALLOC_ERR_TOO_LARGE;
  if (nblk > kMaxGridY) return FTK_NOALLOC_ERR_TOO_LARGE;   // row blocks ride on grid.y
  float* scratch = scratch_for_current_device();
  if (!scratch) return FTK_NOALLOC_ERR_SETUP;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((cols / 2 + 127) / 128), (unsigned)nblk);
  colsum_partial_noalloc<<<grid, 128, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch, rows,
                                              cols, ld);
  // a first launch that was refused must not be followed by a kernel that folds stale scratch into out
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return (int)e;
  colsum_final_noalloc<<<(cols + 255) / 256, 256, 0, s>>>(scratch, out, cols, (int)nblk, accumulate);
  return (int)cudaPeekAtLastError();
}

extern "C" const char* ftk_noalloc_strerror(int code) {
  switch (code) {
    case FTK_NOALLOC_OK: return "ok";
    case FTK_NOALLOC_ERR_BAD_ARG:
      return "ftk_colsum_bf16_noalloc: bad argument (null pointer, non-positive extent, odd cols or ld, ld < cols, "
             "or x / out not 4-byte aligned)";
    case FTK_NOALLOC_ERR_TOO_LARGE:
      return "ftk_colsum_bf16_noalloc: ceil(rows/64)*cols exceeds the built-in scratch of 1048576 floats (4 MiB); "
             "or ceil(rows/64) exceeds 65535 row blocks; use ftk_colsum_bf16 with a caller-provided scratch buffer "
             "for larger problems";
    case FTK_NOALLOC_ERR_SETUP:
      return "ftk_colsum_bf16_noalloc: could not resolve the device address of the built-in scratch array";
    default: return "ftk_colsum_bf16_noalloc: CUDA error (see cudaGetErrorString)";
  }
}
