// Column-sum entry point that performs no device allocation.
//
// This entry point has no counterpart in the reference project; it exists for
// callers of this library that are not allowed to allocate device memory.
//
// Who that is: a host that has already handed all of the GPU's memory to its own
// arena (an inference server or a framework that reserves HBM up front), a
// latency-bound loop that must not call cudaMalloc/cudaFree because those calls
// may synchronise the device and take unbounded time, and plug-in style callers
// that only ever receive buffers from their host application.  The regular
// ftk_colsum_bf16 needs a caller-provided scratch buffer for its per-row-block
// partial sums; such callers have nowhere to get one from.  Here the scratch is a
// fixed array inside the library image instead.
//
// What it computes: out[c] (+)= sum over rows r of x[r, c] for a bf16 [rows, cols]
// matrix with row stride `ld`, in fp32, in a fixed summation order (row blocks of 64
// summed in ascending row order, then the block partials in ascending order), so a call
// returns the same bits every time; ftk_colsum_bf16 blocks its rows differently, so the
// two entry points agree to fp32 rounding, not bit for bit.
//
// Limits and rules:
//   * scratch capacity is FTK_COLSUM_NOALLOC_MAX_FLOATS floats (4 MiB), held by every
//     GPU that loads the library until the process exits;
//     ceil(rows / 64) * cols must not exceed it, otherwise the call returns
//     FTK_NOALLOC_ERR_TOO_LARGE and launches nothing
//     (ftk_noalloc_strerror() gives the message); ceil(rows / 64) itself must not exceed
//     65535 (the row blocks are one grid dimension), same error;
//   * x and out must be 4-byte aligned (x is read as pairs of bf16, out as fp32 words): a
//     bf16 view that starts at an odd element is refused with FTK_NOALLOC_ERR_BAD_ARG
//     before anything is launched, because on the device it would be a misaligned access;
//   * the first call on each device looks up the scratch array's device address
//     (cudaGetSymbolAddress) and caches it; make that first call before starting
//     any stream capture on that device;
//   * all calls on a device share the one scratch array and it keeps the previous
//     call's partial sums: the kernel overwrites every partial it later reads, so
//     nothing needs clearing, but two calls whose kernels overlap on the GPU (for
//     example on different streams) race on it - serialise them;
//   * the call allocates nothing: no cudaMalloc/cudaFree, no allocating library
//     routine; the caller passes the input and the output.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define FTK_COLSUM_NOALLOC_MAX_FLOATS (1 << 20)

enum {
  FTK_NOALLOC_OK = 0,
  FTK_NOALLOC_ERR_BAD_ARG = -2,      // null pointer, non-positive extent, odd cols/ld, x/out not 4-byte aligned
  FTK_NOALLOC_ERR_TOO_LARGE = -20,   // ceil(rows/64)*cols exceeds the scratch capacity, or > 65535 row blocks
  FTK_NOALLOC_ERR_SETUP = -21,       // the scratch symbol's address could not be resolved
};

// x: bf16 [rows, cols], row stride ld (elements); out: fp32 [cols]; accumulate != 0 adds to out.
int ftk_colsum_bf16_noalloc(const void* x, float* out, int rows, int cols, long long ld,
                            int accumulate, void* stream);
const char* ftk_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
