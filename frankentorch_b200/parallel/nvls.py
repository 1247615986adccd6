"""Collectives through the NVSwitch multicast object (NVLS) on one node.

:class:`MulticastBuffer` is a symmetric allocation (the same size on every rank of a group) that
is also bound to one multicast address: PyTorch's symmetric-memory allocator does the driver
work (``cuMemCreate`` + handle exchange + ``cuMulticastCreate`` / bind); the kernels are this
package's own (``csrc/nvls.cu``: ``multimem.st`` all-gather, ``multimem.ld_reduce`` +
``multimem.st`` two-shot all-reduce, with bounded two-barrier protocols over release / acquire
flags).  ``mc_ptr`` is 0 where the GPUs or the driver offer no multicast; callers then keep
to the peer-store kernels (``parallel/symm.py``, ``parallel/data_parallel.py``).

The switch adds the W values of a ``multimem.ld_reduce`` in an order of its own: the all-reduce
is stable run to run on one topology but not bit-identical with the ascending-rank sums of the
strict-mode kernels, so it is offered to hardened mode only.  The all-gather is pure data movement
and is bit-exact.  Rank-failure tests never run on these buffers (a process that dies while its
memory is bound to a multicast object can fault the peers' GPUs).

The reference has no multi-device code (docs/planning/FEATURE_PARITY.md:176).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as K

MAX_RANKS = 16
FLAG_BYTES = 4 * MAX_RANKS * 8


class NvlsUnavailable(RuntimeError):
    """The group's GPUs (or the driver) expose no multicast object."""


class _Comm(C.Structure):
    _fields_ = [("mc", C.c_void_p), ("local", C.c_void_p), ("flags", C.c_void_p * MAX_RANKS),
                ("counter", C.c_void_p), ("rank", C.c_int), ("world", C.c_int)]


def _bind(lib):
    lib.ftk_nvls_allgather.argtypes = [C.POINTER(_Comm), C.c_void_p, C.c_longlong, C.c_longlong, C.c_ulonglong,
                                       C.c_int, C.c_void_p]
    lib.ftk_nvls_allreduce.argtypes = [C.POINTER(_Comm), C.c_longlong, C.c_longlong, C.c_int, C.c_ulonglong,
                                       C.c_int, C.c_void_p]
    lib.ftk_nvls_allgather.restype = lib.ftk_nvls_allreduce.restype = C.c_int
    return lib


class MulticastBuffer:
    """``nbytes`` on every rank of ``group``, peer-mapped and bound to one multicast address."""

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup], device: torch.device):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.device = device
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if not 2 <= self.world <= MAX_RANKS:
            raise NvlsUnavailable(f"multicast buffers serve 2..{MAX_RANKS} ranks, not {self.world}")
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.flag_off = self.nbytes
        torch.cuda.set_device(device)
        self._t = symm.empty(self.nbytes + FLAG_BYTES, dtype=torch.uint8, device=device)
        self._hdl = symm.rendezvous(self._t, self.group)
        self.mc_ptr = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        self.peer_ptrs: List[int] = [int(p) for p in self._hdl.buffer_ptrs]
        self.local_ptr = self.peer_ptrs[self.rank]
        self._t.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)
        self.bytes = self._t[:self.nbytes]

    @property
    def has_multicast(self) -> bool:
        return self.mc_ptr != 0

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        t = self.bytes[byte_offset:].view(dtype)
        return t if numel is None else t[:numel]

    def peer_table(self, byte_offset: int = 0):
        arr = (C.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.peer_ptrs[r] + byte_offset
        return arr


class NvlsCollectives:
    """All-gather and all-reduce kernels over one :class:`MulticastBuffer`."""

    def __init__(self, buf: MulticastBuffer, n_ctas: int = 148):
        if not buf.has_multicast:
            raise NvlsUnavailable("the symmetric allocation has no multicast address on this system")
        self.buf, self.n_ctas = buf, int(n_ctas)
        self.lib = _bind(_lib.load())
        self._counter = torch.zeros(4, dtype=torch.int32, device=buf.device)
        self.seq = 0
        c = _Comm()
        c.mc, c.local = buf.mc_ptr, buf.local_ptr
        for r in range(buf.world):
            c.flags[r] = buf.peer_ptrs[r] + buf.flag_off
        c.counter, c.rank, c.world = self._counter.data_ptr(), buf.rank, buf.world
        self._c = c

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.buf.device).cuda_stream)

    def all_gather(self, src: torch.Tensor, dst_byte_offset: int = 0) -> torch.Tensor:
        """Every rank's ``src`` (contiguous, a multiple of 16 bytes) lands in rank order at
        ``dst_byte_offset`` of every rank's buffer; returns the gathered view ``[world, *src.shape]``."""
        if not src.is_contiguous():
            raise ValueError("all_gather needs a contiguous source")
        nb = src.numel() * src.element_size()
        if nb % 16 or dst_byte_offset % 16 or dst_byte_offset + nb * self.buf.world > self.buf.nbytes:
            raise ValueError("chunk must be a multiple of 16 bytes and fit the buffer")
        self.seq += 1
        rc = self.lib.ftk_nvls_allgather(C.byref(self._c), src.data_ptr(), dst_byte_offset, nb, self.seq, self.n_ctas,
                                         self._stream())
        K._chk(rc, "nvls_allgather")
        return self.buf.tensor(src.dtype, src.numel() * self.buf.world, dst_byte_offset).view(
            self.buf.world, *src.shape)

    def all_reduce_(self, byte_offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Sum over ranks, in place, of ``numel`` elements (fp32 or bf16) at ``byte_offset`` of the buffer."""
        code = {torch.float32: 0, torch.bfloat16: 1}.get(dtype)
        if code is None:
            raise ValueError("all_reduce_ takes fp32 or bf16")
        nb = numel * (4 if code == 0 else 2)
        if nb % 16 or byte_offset % 16 or byte_offset + nb > self.buf.nbytes:
            raise ValueError("range must be a multiple of 16 bytes and fit the buffer")
        self.seq += 1
        rc = self.lib.ftk_nvls_allreduce(C.byref(self._c), byte_offset, nb, code, self.seq, self.n_ctas, self._stream())
        K._chk(rc, "nvls_allreduce")
        return self.buf.tensor(dtype, numel, byte_offset)
