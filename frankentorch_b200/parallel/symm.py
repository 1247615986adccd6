"""Peer-visible ("symmetric") device buffers for one-process-per-GPU jobs on one node.

Each rank allocates a buffer with ``cudaMalloc`` inside the kernel library, exports a CUDA IPC
handle, exchanges handles through the process group and maps every peer's buffer.  Kernels
then receive the table of peer base pointers and issue plain loads / stores over
NVLink (no TMA multicast, no multimem objects).  Buffers are exposed to PyTorch as ordinary
tensors through ``__cuda_array_interface__``.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib


class _RawCuda:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _bind(lib):
    lib.ftk_ipc_alloc.argtypes = [C.c_longlong, C.POINTER(C.c_void_p), C.c_char_p]
    lib.ftk_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.ftk_ipc_close.argtypes = [C.c_void_p]
    lib.ftk_ipc_free.argtypes = [C.c_void_p]
    for f in (lib.ftk_ipc_alloc, lib.ftk_ipc_open, lib.ftk_ipc_close, lib.ftk_ipc_free):
        f.restype = C.c_int
    return lib


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``, each mapped into every process."""

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup], device: torch.device):
        self.lib = _bind(_lib.load())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        torch.cuda.set_device(device)
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        rc = self.lib.ftk_ipc_alloc(self.nbytes, C.byref(ptr), handle)
        if rc != 0:
            raise RuntimeError(f"ftk_ipc_alloc({self.nbytes}) failed with CUDA error {rc}")
        self.local_ptr = int(ptr.value)
        self.peer_ptrs: List[int] = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        self._opened: List[int] = []
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                p = C.c_void_p()
                rc = self.lib.ftk_ipc_open(h, C.byref(p))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed with CUDA error {rc}")
                self.peer_ptrs[r] = int(p.value)
                self._opened.append(int(p.value))
            dist.barrier(group=group)
        self._holder = _RawCuda(self.local_ptr, self.nbytes)
        self.bytes = torch.as_tensor(self._holder, device=device)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        t = self.bytes[byte_offset:].view(dtype)
        return t if numel is None else t[:numel]

    def peer_table(self, byte_offset: int = 0):
        """ctypes array of ``void*``: this rank's view of every rank's buffer (+ offset)."""
        arr = (C.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.peer_ptrs[r] + byte_offset
        return arr

    def close(self) -> None:
        """Unmap the peers' buffers and, once every rank has done so (a barrier of the group), free this
        rank's own allocation.  Collective over the group; tensors handed out by :meth:`tensor` are dead
        afterwards.  A buffer that is never closed lives until the process ends."""
        if self.local_ptr == 0:
            return
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self.lib.ftk_ipc_close(p)
        self._opened = []
        if self.world > 1 and self.group is not None and dist.is_initialized():
            dist.barrier(group=self.group)          # nobody maps this rank's memory any more
        self.bytes = None
        self._holder = None
        self.lib.ftk_ipc_free(self.local_ptr)
        self.local_ptr = 0
        self.peer_ptrs = [0] * self.world
