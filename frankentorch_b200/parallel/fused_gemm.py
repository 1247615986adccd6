"""GEMMs fused with their collective over NVLink peer memory (one kernel per op).

Three forms of the tcgen05 GEMM kernel (``csrc/gemm_kernel.cuh``), each one launch in which a
few CTAs move data between GPUs while the rest multiply:

* :meth:`FusedCollectives.allgather_a_gemm`  - all-gather of row-sharded activations feeding
  the A operand (tensor-parallel column-parallel Linear with sequence parallelism);
* :meth:`FusedCollectives.allgather_b_gemm`  - all-gather of a row-sharded weight feeding the
  B operand (ZeRO-3 parameter gather fused into the first GEMM that consumes it), forward
  (``x W^T``) and dgrad (``dy W``, weight sharded along the reduction dimension);
  Both gathers have two forms: the *pull* form (staging buffer in ordinary local memory; copy CTAs
  fetch the peers' shards) and the *push* form (staging buffer in symmetric memory, passed as a
  :class:`SymmTensor`: every rank delivers its own shard into all peers' staging buffers in the
  order the consumers need them, and consumers poll flags in their own memory only).  The push
  form has three transports (``FT_GATHER_TRANSPORT``): ``ew`` lets the epilogue warps of EVERY CTA
  store the shard into the peers' buffers while they wait for their accumulators (no SM is set aside,
  all of them issue peer stores); ``sm`` (default) moves the shards with copy CTAs inside the GEMM kernel; ``ce`` enqueues the deliveries as device-to-device copies on
  other streams, each followed by a one-warp kernel that sets the arrival flags at the consumer,
  so the copy engines move the bytes and all SMs multiply.  Measured on two GPUs the hand-over
  between the copy engines and that kernel costs tens of microseconds per delivery, which makes
  ``ce`` the slowest of the three forms there; it is kept as an option for large chunks;
* :meth:`FusedCollectives.gemm_reduce_scatter` - the epilogue stores bf16 partial tiles into the
  owning rank's inbox and the owner adds them in ascending rank order (row-parallel Linear,
  ZeRO-3 weight-gradient reduce-scatter).

The reference has no distributed layer at all (FEATURE_PARITY.md:176); the Linear math is
ft-nn/src/lib.rs:1076-1100 and ft-kernel-cpu/src/lib.rs:17162-17302.

Protocol state: every flag word stores the *epoch* (use count) of the call that set it, so
flag arrays are never cleared and can be shared by calls of different shapes.  The epoch lives
in device memory and is advanced by a one-thread kernel before each launch, which keeps the
sequence replayable inside a CUDA graph.  Shard buffers and inboxes that change between calls
must alternate between two slots: a rank can run at most one collective ahead of its slowest
peer, because every collective needs a contribution of every rank.  The same rule covers the
push form's staging buffers (:meth:`FusedCollectives.staging` hands out such pairs): a peer
writes into this rank's buffer, so the buffer a call receives into must not be read by the
call before it nor by anything launched after that call.
"""
from __future__ import annotations

import os

import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as K
from ..ops._lib import (COMM_GATHER_A, COMM_GATHER_B, COMM_SCATTER_D, FtkCommDesc, FtkGemmDesc)
from .symm import SymmetricBuffer

TILE_M = 128
TILE_N = 256


class SymmTensor:
    """A tensor inside a :class:`SymmetricBuffer` together with its address on every rank."""

    def __init__(self, buf: SymmetricBuffer, shape: Sequence[int], dtype: torch.dtype, byte_offset: int = 0):
        n = 1
        for s in shape:
            n *= int(s)
        self.buf = buf
        self.t = buf.tensor(dtype, n, byte_offset).view(*shape)
        self.peer_ptrs: List[int] = [p + byte_offset for p in buf.peer_ptrs]

    @staticmethod
    def alloc(shape: Sequence[int], dtype: torch.dtype, group, device) -> "SymmTensor":
        n = 1
        for s in shape:
            n *= int(s)
        buf = SymmetricBuffer(n * torch.empty((), dtype=dtype).element_size(), group, device)
        return SymmTensor(buf, shape, dtype)


class FusedCollectives:
    """Flag storage, inboxes and launch helpers for the collective-fused GEMMs of one group."""

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, *,
                 max_gather_bytes: int = 1 << 30, max_inbox_elems: int = 0, max_chunk_tiles: int = 4096,
                 comm_ctas: int = 0):
        self.group, self.device = group, device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        if comm_ctas == 0 and "FT_COMM_CTAS" in os.environ:
            from ..utils.config import env_flag
            comm_ctas = int(env_flag("FT_COMM_CTAS"))
        self.comm_ctas = comm_ctas
        self.lib = _lib.load()
        # local words: [0] epoch, then one flag per 32 KiB piece of a gathered operand
        self.local = torch.zeros(64 + max_gather_bytes // 32768 + 1024, dtype=torch.int32, device=device)
        self.epoch = self.local[0:1]
        self.sub_flags = self.local[64:]
        # symmetric words: ready[world] | arrive[3][max_chunk_tiles][world]
        self.max_chunk_tiles = max_chunk_tiles
        words = 64 + 3 * max_chunk_tiles * self.world
        self.flags = SymmetricBuffer(words * 4, group, device)
        self.flags.bytes.zero_()
        # push-form gathers: the per-piece flags are written by the peers
        self.gflags = SymmetricBuffer(self.sub_flags.numel() * 4, group, device)
        self.gflags.bytes.zero_()
        self.max_inbox_elems = max_inbox_elems
        self.inbox = None
        if max_inbox_elems:
            # three slots of [world][chunk_rows][N] bf16, see begin_step()
            self.inbox = SymmetricBuffer(3 * max_inbox_elems * 2, group, device)
        self._slot = 0
        self._first = True
        self.transport = os.environ.get("FT_GATHER_TRANSPORT", "sm")
        # copy-engine transport: copies per (chunk, destination) and streams the destinations are dealt to.  Every
        # copy -> flag kernel -> copy hand-over between the copy engines and the SMs on one stream costs ~10 us, so
        # few, large copies on alternating streams beat many small ones in one queue.
        self.ce_parts = 1
        self.comm_streams = [torch.cuda.Stream(device=device)
                             for _ in range(max(1, int(os.environ.get("FT_GATHER_CE_STREAMS", "2"))))]
        torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=group)

    # ------------------------------------------------------------------ helpers
    def begin_step(self) -> None:
        """Call at the start of every training step (also while a CUDA graph is being captured).

        Consecutive reduce-scatters must not share an inbox slot.  The first one of a step takes
        slot 2 and the rest alternate between 0 and 1, so the rule also holds across the step
        boundary when one captured step is replayed, whatever the number of calls per step.
        """
        self._first = True
        self._slot = 0

    def _next_slot(self) -> int:
        if self._first:
            self._first = False
            return 2
        s = self._slot
        self._slot ^= 1
        return s

    def _tick(self) -> None:
        K._chk(self.lib.ftk_tick_i32(self.epoch.data_ptr(), K._stream()), "ftk_tick_i32")

    def _comm(self, mode: int, chunk_rows: int) -> FtkCommDesc:
        c = FtkCommDesc()
        c.mode, c.rank, c.world = mode, self.rank, self.world
        c.comm_ctas, c.chunk_rows = self.comm_ctas, chunk_rows
        c.epoch = self.epoch.data_ptr()
        return c

    @staticmethod
    def _gemm_desc(a, b, out, *, a_mn=False, b_mn=False, bias=None, resid=None, aux=None, epi=K.EPI_NONE,
                   alpha=1.0, accumulate=False, M=None, N=None, K_=None) -> FtkGemmDesc:
        g = FtkGemmDesc()
        g.M, g.N, g.K, g.L0, g.L1 = M, N, K_, 1, 1
        g.a_mn, g.b_mn = int(a_mn), int(b_mn)
        g.A, g.lda = a.data_ptr(), a.stride(0)
        g.B, g.ldb = b.data_ptr(), b.stride(0)
        g.D, g.ldd = out.data_ptr(), out.stride(0)
        g.bias = None if bias is None else bias.data_ptr()
        if resid is not None:
            g.resid, g.ldr = resid.data_ptr(), resid.stride(0)
        if aux is not None:
            g.aux = aux.data_ptr()
        g.alpha, g.epi = float(alpha), int(epi)
        g.out_fp32 = 1 if out.dtype == torch.float32 else 0
        g.accumulate = int(accumulate)
        return g

    def staging(self, shape: Sequence[int], slots: int = 2) -> List[SymmTensor]:
        """``slots`` symmetric bf16 staging buffers for the push-form gathers (alternate them call by call)."""
        return [SymmTensor.alloc(shape, torch.bfloat16, self.group, self.device) for _ in range(slots)]

    def _gather(self, c: FtkCommDesc, shard: SymmTensor, handshake: bool, full=None) -> None:
        for r in range(self.world):
            c.src[r] = shard.peer_ptrs[r]
        if isinstance(full, SymmTensor):
            row_bytes = shard.t.shape[1] * 2
            n_flags = c.chunk_rows // TILE_M * self.world * max(1, TILE_M * row_bytes // 32768)
            if n_flags > self.sub_flags.numel():
                raise K.KernelError("gathered operand needs more flag words than were allocated")
            c.push = {"ce": 2, "ew": 3}.get(self.transport, 1)
            c.sub_flags = self.gflags.local_ptr
            for r in range(self.world):
                c.full_peer[r] = full.peer_ptrs[r]
                c.flags_peer[r] = self.gflags.peer_ptrs[r]
            return
        # one flag word per copied piece (at most 32 KiB) of the gathered operand
        row_bytes = shard.t.shape[1] * 2
        sub = TILE_M * row_bytes
        n_flags = c.chunk_rows // TILE_M * self.world * max(1, sub // 32768)
        if n_flags > self.sub_flags.numel():
            raise K.KernelError("gathered operand needs more flag words than were allocated")
        c.sub_flags = self.sub_flags.data_ptr()
        if handshake and self.world > 1:
            c.ready_local = self.flags.local_ptr
            for r in range(self.world):
                c.ready_peer[r] = self.flags.peer_ptrs[r] + 4 * self.rank

    def _ce_deliver(self, shard: SymmTensor, full: SymmTensor, own_last: bool):
        """Copy-engine transport of the push form: on the communication stream, behind everything the launching
        stream has queued so far (the shard is final, the epoch is ticked), copy this rank's shard into every
        rank's staging buffer - destinations in the order they will need it, each chunk in ``ce_parts`` copies -
        and set the arrival flags of each part at its consumer.  Returns the events the launching stream must
        wait for after the GEMM (the shard may then be rewritten, the own staged copy is complete)."""
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        for cs in self.comm_streams:
            cs.wait_event(ev)
        rows, cols = shard.t.shape
        row_bytes = cols * 2
        piece = min(TILE_M * row_bytes, 32768)
        chunk_bytes = rows * row_bytes
        ppc = chunk_bytes // piece
        W, r = self.world, self.rank
        if own_last:
            dests = [(r - 1 - d) % W for d in range(W - 1)] + [r]
        else:
            dests = [r] + [(r - d) % W for d in range(1, W)]
        parts = min(self.ce_parts, ppc)
        bounds = [ppc * k // parts for k in range(parts + 1)]
        src, lib = shard.peer_ptrs[r], self.lib
        for n, dest in enumerate(dests):
            raw = C.c_void_p(self.comm_streams[n % len(self.comm_streams)].cuda_stream)
            for k in range(parts):
                p0, p1 = bounds[k], bounds[k + 1]
                K._chk(lib.ftk_copy_async(full.peer_ptrs[dest] + r * chunk_bytes + p0 * piece, src + p0 * piece,
                                          (p1 - p0) * piece, raw), "ftk_copy_async")
                K._chk(lib.ftk_set_flags_sys(self.gflags.peer_ptrs[dest] + 4 * (r * ppc + p0), p1 - p0,
                                             self.epoch.data_ptr(), raw), "ftk_set_flags_sys")
        done = []
        for cs in self.comm_streams:
            e = torch.cuda.Event()
            e.record(cs)
            done.append(e)
        return done

    # ------------------------------------------------------------------ all-gather -> GEMM (A)
    def allgather_a_gemm(self, x_shard: SymmTensor, w: torch.Tensor, x_full: torch.Tensor, *,
                         b_mn: bool = False, bias=None, epi=K.EPI_NONE, resid=None, aux=None, out=None,
                         handshake: bool = True) -> torch.Tensor:
        """``out = epi(allgather(x_shard) @ op(w) + bias)``; ``x_full`` receives the gathered rows.

        ``x_shard.t`` is ``[rows / world, K]`` in symmetric memory, ``x_full`` ``[rows, K]`` local
        scratch (contiguous) or, for the push form, a :class:`SymmTensor` of that shape; ``w`` is
        ``[N, K]`` or, with ``b_mn``, ``[K, N]``.
        """
        full_sym = x_full if isinstance(x_full, SymmTensor) else None
        if full_sym is not None:
            x_full = full_sym.t
        ms, k = x_shard.t.shape
        m = ms * self.world
        n = w.shape[1] if b_mn else w.shape[0]
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
        g = self._gemm_desc(x_full, w, out, b_mn=b_mn, bias=bias, resid=resid, aux=aux, epi=epi, M=m, N=n, K_=k)
        c = self._comm(COMM_GATHER_A, ms)
        self._gather(c, x_shard, handshake, full_sym)
        self._tick()
        done = self._ce_deliver(x_shard, full_sym, own_last=True) if c.push == 2 else None
        K._chk(self.lib.ftk_gemm_comm_bf16(C.byref(g), C.byref(c), K._stream()), "ftk_gemm_comm_bf16(gather A)")
        for e in done or ():
            torch.cuda.current_stream(self.device).wait_event(e)
        return out

    # ------------------------------------------------------------------ all-gather -> GEMM (B)
    def allgather_b_gemm(self, x: torch.Tensor, w_shard: SymmTensor, w_full: torch.Tensor, *,
                         dgrad: bool = False, bias=None, epi=K.EPI_NONE, resid=None, aux=None, out=None,
                         handshake: bool = False) -> torch.Tensor:
        """Forward ``x @ W^T`` or (``dgrad``) ``x @ W`` with ``W = allgather(w_shard)`` ``[out, in]``.

        The weight is sharded by output rows.  ``w_full`` ``[out, in]`` is local scratch that holds
        the gathered weight afterwards (a later GEMM of the same layer may reuse it).
        """
        full_sym = w_full if isinstance(w_full, SymmTensor) else None
        if full_sym is not None:
            w_full = full_sym.t
        rows_s, cols = w_shard.t.shape
        rows = rows_s * self.world
        m = x.shape[0]
        n, k = (cols, rows) if dgrad else (rows, cols)
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
        g = self._gemm_desc(x, w_full, out, b_mn=dgrad, bias=bias, resid=resid, aux=aux, epi=epi, M=m, N=n, K_=k)
        c = self._comm(COMM_GATHER_B, rows_s)
        self._gather(c, w_shard, handshake, full_sym)
        self._tick()
        done = self._ce_deliver(w_shard, full_sym, own_last=False) if c.push == 2 else None
        K._chk(self.lib.ftk_gemm_comm_bf16(C.byref(g), C.byref(c), K._stream()), "ftk_gemm_comm_bf16(gather B)")
        for e in done or ():
            torch.cuda.current_stream(self.device).wait_event(e)
        return out

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_reduce_scatter(self, a: torch.Tensor, b: torch.Tensor, out_shard: torch.Tensor, *,
                            a_mn: bool = False, b_mn: bool = False, bias=None, resid=None,
                            accumulate: bool = False, alpha: float = 1.0) -> torch.Tensor:
        """``out_shard = rows[rank] of sum_over_ranks(a @ op(b)) (+ bias) (+ resid) (+ out_shard)``.

        The full product is ``[M, N]`` with ``M = world * out_shard.shape[0]``; partial tiles cross
        NVLink as bf16 and are added in ascending rank order in fp32.
        """
        m = a.shape[1] if a_mn else a.shape[0]
        k = a.shape[0] if a_mn else a.shape[1]
        n = b.shape[1] if b_mn else b.shape[0]
        ms = out_shard.shape[0]
        if ms * self.world != m or out_shard.shape[1] != n:
            raise K.KernelError(f"reduce-scatter output {tuple(out_shard.shape)} does not match [{m}/{self.world}, {n}]")
        tiles = (ms // TILE_M) * ((n + TILE_N - 1) // TILE_N)
        if self.inbox is None or self.world * ms * n > self.max_inbox_elems or tiles > self.max_chunk_tiles:
            raise K.KernelError("inbox / flag storage too small for this reduce-scatter")
        g = self._gemm_desc(a, b, out_shard, a_mn=a_mn, b_mn=b_mn, bias=bias, resid=resid, alpha=alpha,
                            accumulate=accumulate, M=m, N=n, K_=k)
        c = self._comm(COMM_SCATTER_D, ms)
        slot = self._next_slot()
        for r in range(self.world):
            c.inbox[r] = self.inbox.peer_ptrs[r] + slot * self.max_inbox_elems * 2
            c.arrive[r] = self.flags.peer_ptrs[r] + 4 * (64 + slot * self.max_chunk_tiles * self.world)
        self._tick()
        K._chk(self.lib.ftk_gemm_comm_bf16(C.byref(g), C.byref(c), K._stream()), "ftk_gemm_comm_bf16(scatter)")
        return out_shard
