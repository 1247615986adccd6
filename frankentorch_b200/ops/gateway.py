"""Generic CUDA compute gateway: compile a kernel from source at run time, bind buffers, launch
a validated grid, wait for completion.

API parity with the reference's Metal compute gateway (ft-kernel-metal/src/compute.rs:56-405:
``Gateway`` / ``Library`` / ``Pipeline`` / ``SharedBuffer`` / ``Grid`` / ``MathMode`` and the typed
errors ``SizeOverflow``, ``BufferTooLarge``, zero-extent grid, zero-length buffer), re-targeted to
NVRTC + the CUDA driver API for sm_100a:

* ``Gateway.open()``                  - the current CUDA device
* ``gateway.library(source)``         - NVRTC compile, IEEE-faithful by default
  (``MathMode.Safe``: no ``--use_fast_math``, fused multiply-add contraction off);
  ``library_with(source, MathMode.Fast)`` opts into fast math (compute.rs:69-81)
* ``library.pipeline(name)``          - a ``__global__`` function by name
* ``gateway.buffer_f32 / buffer_u32 / buffer_zeroed`` - device buffers with host read-back
  (``read_f32`` / ``read_u32`` / ``read_u8``)
* ``gateway.dispatch(pipeline, buffers, grid)`` - every buffer is passed as one pointer argument
  in order; synchronous like the reference's ``wait_until_completed`` (compute.rs:371-405)

Pure validation (``Grid.validate``, buffer size checks) needs no GPU and mirrors
compute.rs:112-200.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

USIZE_MAX = (1 << 64) - 1


class GatewayError(RuntimeError):
    """``Error::Kernel`` of the reference: compile / lookup / launch failures and bad arguments."""


class SizeOverflow(GatewayError):
    def __init__(self, what: str):
        super().__init__(f"size overflow computing {what}")
        self.what = what


class BufferTooLarge(GatewayError):
    def __init__(self, requested: int, maximum: int):
        super().__init__(f"buffer of {requested} bytes exceeds the device maximum {maximum}")
        self.requested, self.maximum = requested, maximum


class MathMode(enum.Enum):
    Safe = "safe"     # IEEE-faithful, the default (compute.rs:69-75)
    Fast = "fast"


def _checked_product(values: Sequence[int], what: str) -> int:
    p = 1
    for v in values:
        p *= int(v)
        if p > USIZE_MAX:
            raise SizeOverflow(what)
    return p


def checked_byte_len(elements: int, element_bytes: int, what: str) -> int:
    n = int(elements) * int(element_bytes)
    if n > USIZE_MAX:
        raise SizeOverflow(what)
    return n


def validate_buffer_size(nbytes: int, maximum: int) -> None:
    if nbytes == 0:
        raise GatewayError("zero-length buffer")
    if nbytes > maximum:
        raise BufferTooLarge(nbytes, maximum)


@dataclass(frozen=True)
class Grid:
    """Thread-block counts and threads per block, three extents each (compute.rs:83-110)."""
    threadgroups: Tuple[int, int, int]
    threads_per_threadgroup: Tuple[int, int, int]

    @staticmethod
    def linear(groups: int, threads: int) -> "Grid":
        return Grid((groups, 1, 1), (threads, 1, 1))

    @staticmethod
    def grid_2d(gx: int, gy: int, tx: int, ty: int) -> "Grid":
        return Grid((gx, gy, 1), (tx, ty, 1))

    def threadgroup_count(self) -> int:
        return _checked_product(self.threadgroups, "threadgroup count")

    def threads_per_threadgroup_count(self) -> int:
        return _checked_product(self.threads_per_threadgroup, "threads-per-threadgroup count")

    def validate(self) -> None:
        if any(int(n) == 0 for n in (*self.threadgroups, *self.threads_per_threadgroup)):
            raise GatewayError(f"grid has a zero extent: threadgroups {list(self.threadgroups)}, "
                               f"threads {list(self.threads_per_threadgroup)}")
        if any(int(n) < 0 for n in (*self.threadgroups, *self.threads_per_threadgroup)):
            raise GatewayError("grid has a negative extent")
        _checked_product((self.threadgroup_count(), self.threads_per_threadgroup_count()), "dispatch thread count")


def _drv():
    from cuda.bindings import driver, nvrtc
    return driver, nvrtc


def _ck(res, what: str):
    driver, nvrtc = _drv()
    err = res[0]
    ok = (driver.CUresult.CUDA_SUCCESS, nvrtc.nvrtcResult.NVRTC_SUCCESS)
    if err not in ok:
        raise GatewayError(f"{what}: {err!r}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


class SharedBuffer:
    """Device memory owned by the gateway, readable back to the host."""

    def __init__(self, gw: "Gateway", nbytes: int):
        driver, _ = _drv()
        validate_buffer_size(nbytes, gw.max_buffer_length())
        self._gw = gw
        self.nbytes = int(nbytes)
        self.ptr = int(_ck(driver.cuMemAlloc(self.nbytes), "cuMemAlloc"))
        self._freed = False

    def len_bytes(self) -> int:
        return self.nbytes

    def _upload(self, arr: np.ndarray) -> None:
        driver, _ = _drv()
        arr = np.ascontiguousarray(arr)
        _ck(driver.cuMemcpyHtoD(self.ptr, arr.ctypes.data, arr.nbytes), "cuMemcpyHtoD")

    def _read(self, out: np.ndarray) -> None:
        driver, _ = _drv()
        if out.nbytes > self.nbytes:
            raise GatewayError(f"read of {out.nbytes} bytes from a buffer of {self.nbytes}")
        _ck(driver.cuMemcpyDtoH(out.ctypes.data, self.ptr, out.nbytes), "cuMemcpyDtoH")

    def read_f32(self, out: np.ndarray) -> None:
        self._read(out.view(np.float32) if out.dtype != np.float32 else out)

    def read_u32(self, out: np.ndarray) -> None:
        self._read(out.view(np.uint32) if out.dtype != np.uint32 else out)

    def read_u8(self, out: np.ndarray) -> None:
        self._read(out.view(np.uint8) if out.dtype != np.uint8 else out)

    def free(self) -> None:
        if not self._freed:
            driver, _ = _drv()
            driver.cuMemFree(self.ptr)
            self._freed = True

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Pipeline:
    def __init__(self, lib: "Library", name: str, fn, max_threads: int):
        self.library, self.name, self.fn = lib, name, fn
        self._max_threads = max_threads

    def max_threads_per_threadgroup(self) -> int:
        return self._max_threads

    def thread_execution_width(self) -> int:
        return 32


class Library:
    def __init__(self, gw: "Gateway", module, mode: MathMode):
        self.gateway, self.module, self.mode = gw, module, mode

    def pipeline(self, name: str) -> Pipeline:
        driver, _ = _drv()
        res = driver.cuModuleGetFunction(self.module, name.encode())
        if res[0] != driver.CUresult.CUDA_SUCCESS:
            raise GatewayError(f"kernel '{name}' not found in the library: {res[0]!r}")
        fn = res[1]
        mx = _ck(driver.cuFuncGetAttribute(driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, fn),
                 "cuFuncGetAttribute")
        return Pipeline(self, name, fn, int(mx))


class Gateway:
    """The current CUDA device as a compile-and-dispatch target."""

    def __init__(self, device_index: int = 0):
        driver, _ = _drv()
        _ck(driver.cuInit(0), "cuInit")
        self.device = _ck(driver.cuDeviceGet(device_index), "cuDeviceGet")
        self.ctx = _ck(driver.cuDevicePrimaryCtxRetain(self.device), "cuDevicePrimaryCtxRetain")
        _ck(driver.cuCtxSetCurrent(self.ctx), "cuCtxSetCurrent")
        A = driver.CUdevice_attribute
        self._major = int(_ck(driver.cuDeviceGetAttribute(A.CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, self.device), "attr"))
        self._minor = int(_ck(driver.cuDeviceGetAttribute(A.CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, self.device), "attr"))
        self._smem = int(_ck(driver.cuDeviceGetAttribute(A.CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN, self.device), "attr"))
        self._total = int(_ck(driver.cuDeviceTotalMem(self.device), "cuDeviceTotalMem"))

    @staticmethod
    def open(device_index: int = 0) -> "Gateway":
        try:
            return Gateway(device_index)
        except GatewayError:
            raise
        except Exception as e:   # no driver / no device
            raise GatewayError(f"no CUDA device available: {e}") from e

    def device_name(self) -> str:
        driver, _ = _drv()
        name = _ck(driver.cuDeviceGetName(128, self.device), "cuDeviceGetName")
        return bytes(name).split(b"\0")[0].decode()

    def has_unified_memory(self) -> bool:
        return False          # discrete HBM; buffers are read back explicitly

    def max_threadgroup_memory(self) -> int:
        return self._smem

    def max_buffer_length(self) -> int:
        return self._total

    def library(self, source: str) -> Library:
        return self.library_with(source, MathMode.Safe)

    def library_with(self, source: str, mode: MathMode) -> Library:
        driver, nvrtc = _drv()
        prog = _ck(nvrtc.nvrtcCreateProgram(source.encode(), b"gateway.cu", 0, [], []), "nvrtcCreateProgram")
        arch = f"sm_{self._major}{self._minor}" + ("a" if self._major >= 9 else "")
        opts = [f"--gpu-architecture={arch}".encode(), b"--std=c++17"]
        opts += [b"--use_fast_math"] if mode is MathMode.Fast else [b"--fmad=false"]
        res = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if res[0] != nvrtc.nvrtcResult.NVRTC_SUCCESS:
            n = _ck(nvrtc.nvrtcGetProgramLogSize(prog), "nvrtcGetProgramLogSize")
            log = b" " * int(n)
            nvrtc.nvrtcGetProgramLog(prog, log)
            nvrtc.nvrtcDestroyProgram(prog)
            raise GatewayError("kernel source failed to compile:\n" + log.decode(errors="replace"))
        n = _ck(nvrtc.nvrtcGetCUBINSize(prog), "nvrtcGetCUBINSize")
        cubin = b" " * int(n)
        _ck(nvrtc.nvrtcGetCUBIN(prog, cubin), "nvrtcGetCUBIN")
        nvrtc.nvrtcDestroyProgram(prog)
        module = _ck(driver.cuModuleLoadData(np.frombuffer(cubin, dtype=np.uint8).ctypes.data), "cuModuleLoadData")
        lib = Library(self, module, mode)
        lib._cubin = cubin
        return lib

    def buffer_f32(self, data) -> SharedBuffer:
        arr = np.asarray(data, dtype=np.float32)
        b = SharedBuffer(self, checked_byte_len(arr.size, 4, "f32 buffer"))
        b._upload(arr)
        return b

    def buffer_u32(self, data) -> SharedBuffer:
        arr = np.asarray(data, dtype=np.uint32)
        b = SharedBuffer(self, checked_byte_len(arr.size, 4, "u32 buffer"))
        b._upload(arr)
        return b

    def buffer_zeroed(self, nbytes: int) -> SharedBuffer:
        driver, _ = _drv()
        b = SharedBuffer(self, nbytes)
        _ck(driver.cuMemsetD8(b.ptr, 0, b.nbytes), "cuMemsetD8")
        return b

    def dispatch(self, pipeline: Pipeline, buffers: List[SharedBuffer], grid: Grid) -> None:
        """Launch ``pipeline`` over ``grid`` with ``buffers`` as pointer arguments and wait for it."""
        driver, _ = _drv()
        grid.validate()
        want, mx = grid.threads_per_threadgroup_count(), pipeline.max_threads_per_threadgroup()
        if want > mx:
            raise GatewayError(f"kernel '{pipeline.name}': {want} threads/threadgroup exceeds the pipeline maximum {mx}")
        gx, gy, gz = (int(v) for v in grid.threadgroups)
        if gx > 2147483647 or gy > 65535 or gz > 65535:
            raise SizeOverflow("threadgroup extent")
        ptrs = [C.c_void_p(b.ptr) for b in buffers]
        argv = (C.c_void_p * max(len(ptrs), 1))(*[C.addressof(p) for p in ptrs])
        tx, ty, tz = (int(v) for v in grid.threads_per_threadgroup)
        _ck(driver.cuLaunchKernel(pipeline.fn, gx, gy, gz, tx, ty, tz, 0, 0, C.addressof(argv), 0), "cuLaunchKernel")
        res = driver.cuCtxSynchronize()
        if res[0] != driver.CUresult.CUDA_SUCCESS:
            raise GatewayError(f"kernel '{pipeline.name}' did not complete: {res[0]!r}")
