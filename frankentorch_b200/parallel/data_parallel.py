"""Data parallelism (ZeRO-1 style): the gradient reduce-scatter is fused with the sharded AdamW
update and the parameter all-gather, bucket by bucket, through in-kernel NVLink peer accesses,
and runs under the backward pass.

``FusedDataParallel`` cuts the flat parameter arena into buckets at parameter boundaries.  The
tape tells it whenever a rule has written a parameter gradient in place; when the last gradient
of a bucket is in, that bucket's push + ordered reduce (``csrc/dp_fused.cu``) is launched on a
communication stream behind an event, while the main stream continues with the backward pass.
Gradients cross NVLink as bf16 and are summed in fp32 in ascending rank order, so results are
bit-identical run to run (and between eager execution and CUDA-graph replay: the step number
lives in device memory and the cross-stream dependencies are captured with the graph).  After
the last bucket: global gradient norm (one scalar exchange).  AdamW on the owned shards and the
peer stores of the updated bf16 parameters into every rank's arena follow at once, or - the
default - at the start of the next step, bucket by bucket under the forward pass.

``NcclDataParallel`` is the stock path - NCCL all-reduce of the flat gradient followed by the
single-GPU fused AdamW - kept as the baseline and as the hardened-mode fallback.

The reference has no distributed training at all (docs/planning/FEATURE_PARITY.md:176); the
single-process optimizer semantics that must be preserved are those of AdamW,
ft-optim/src/lib.rs:800-1085.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as K
from .symm import SymmetricBuffer

DP_MAX_RANKS = 16
DP_MAX_BUCKETS = 64
DEFAULT_BUCKET_ELEMS = 16 * 1024 * 1024      # ~32 MB of bf16 on the wire per bucket
# Grid sizes.  The GEMMs of the backward pass fill every SM's shared memory, so a communication kernel
# that becomes ready while one runs is not co-resident with it: it takes the SMs between two compute
# kernels (or next to the row kernels).  What it costs the step is therefore its own duration, and wide
# grids that finish quickly beat narrow ones that "stay out of the way" (measured at 2 GPUs, GPT-2
# small: 12 / 48 / 148 / 296 CTAs per bucket kernel -> 14.50 / 13.23 / 13.02 / 13.00 ms per step).
REDUCE_CTAS = 296                            # CTAs of a bucket's push / reduce kernels
TAIL_CTAS = 592                              # ... of the buckets that finish with the backward pass
UPDATE_CTAS = 592                            # CTAs of the AdamW + all-gather kernel
UPDATE_OVERLAP_CTAS = 592                    # ... also for the per-bucket updates under the forward pass


def shard_multiple(world: int) -> int:
    """The flat arena length is padded to a multiple of this (bucket ends stay 128-aligned)."""
    return 1024 * max(world, 1)


@dataclass(frozen=True)
class Bucket:
    lo: int       # first arena element
    hi: int       # one past the last
    shard: int    # elements of the bucket owned by each rank (multiple of 8); the last ranks' may be cut by hi
    off: int      # start of this bucket's shard in the rank-local shard arrays

    def owned(self, rank: int) -> Tuple[int, int]:
        """Arena range [a, b) of the bucket that ``rank`` owns (empty when a >= b)."""
        a = self.lo + rank * self.shard
        return a, max(a, min(a + self.shard, self.hi))


def plan_buckets(param_ranges: Sequence[Tuple[int, int]], numel: int, world: int,
                 target_elems: int = DEFAULT_BUCKET_ELEMS, max_buckets: int = DP_MAX_BUCKETS,
                 forced_cuts: Sequence[int] = ()) -> List[Bucket]:
    """Cut ``[0, numel)`` into buckets at parameter boundaries.

    ``param_ranges`` are the arena slots ``(start, end)`` in arena order (ends are 128-aligned, so
    every bucket boundary is).  Parameters are added to a bucket until it holds at least
    ``target_elems``; the last bucket takes the arena's tail padding.  ``forced_cuts`` are arena
    offsets where a boundary must fall (a model puts one behind the parameters whose gradients
    arrive last, e.g. the embeddings, so that they do not hold back a bucket of early finishers);
    a size cut that would fall less than half a target before a forced one is left to it.  The
    boundaries depend only on the arena layout, the world size and the target: every rank computes
    the same plan.
    """
    if numel % 8:
        raise ValueError("the arena length must be a multiple of 8")
    cuts, start, n_params = [], 0, len(param_ranges)
    forced = sorted(set(int(c) for c in forced_cuts if 0 < c < numel))
    for i, (a, b) in enumerate(param_ranges):
        if i + 1 == n_params:
            break
        if b in forced:
            cuts.append(b)
            start = b
        elif b - start >= target_elems and not any(b < c <= b + target_elems // 2 for c in forced):
            cuts.append(b)
            start = b
    edges = [0] + cuts + [numel]
    while len(edges) - 1 > max_buckets:             # merge the smallest neighbours until the table fits
        sizes = [edges[i + 2] - edges[i] for i in range(len(edges) - 2)]
        j = sizes.index(min(sizes))
        del edges[j + 1]
    out, off = [], 0
    for lo, hi in zip(edges[:-1], edges[1:]):
        if lo % 8 or hi % 8:
            raise ValueError("bucket boundaries must be multiples of 8 elements")
        shard = -(-(hi - lo) // world)
        shard = -(-shard // 8) * 8
        out.append(Bucket(lo, hi, shard, off))
        off += shard
    return out


def scatter_shards_to_arena(buckets: Sequence[Bucket], shards: Sequence[torch.Tensor], numel: int) -> torch.Tensor:
    """Rebuild a flat arena-ordered tensor from every rank's local shard array (``shards[r]``)."""
    full = torch.zeros(numel, dtype=shards[0].dtype, device=shards[0].device)
    for bk in buckets:
        for r, s in enumerate(shards):
            a, b = bk.owned(r)
            if b > a:
                full[a:b] = s[bk.off: bk.off + (b - a)]
    return full


def gather_arena_shard(buckets: Sequence[Bucket], full: torch.Tensor, rank: int, total: int) -> torch.Tensor:
    """The rank-local shard array (length ``total``) cut out of a flat arena-ordered tensor."""
    out = torch.zeros(total, dtype=full.dtype, device=full.device)
    for bk in buckets:
        a, b = bk.owned(rank)
        if b > a:
            out[bk.off: bk.off + (b - a)] = full[a:b]
    return out


class _Bucket(C.Structure):
    _fields_ = [("lo", C.c_longlong), ("hi", C.c_longlong), ("shard", C.c_longlong), ("off", C.c_longlong)]


class _Comm(C.Structure):
    _fields_ = [("inbox", C.POINTER(C.c_void_p)), ("params", C.POINTER(C.c_void_p)),
                ("flags", C.POINTER(C.c_void_p)), ("slots", C.POINTER(C.c_void_p)),
                ("buckets", C.c_void_p),
                ("rank", C.c_int), ("world", C.c_int), ("n_buckets", C.c_int), ("n_ctas", C.c_int),
                ("wire_fp32", C.c_int),
                ("gshard", C.c_void_p), ("partial", C.c_void_p), ("counters", C.c_void_p),
                ("seq", C.c_void_p), ("ok_word", C.c_void_p), ("pending", C.c_void_p),
                ("hyper_pending", C.c_void_p), ("params_mc", C.c_void_p)]


def _bind(lib):
    pc, vp, i, f = C.POINTER(_Comm), C.c_void_p, C.c_int, C.c_float
    lib.ftk_dp_begin_step.argtypes = [pc, vp]
    lib.ftk_dp_bucket_reduce.argtypes = [pc, i, vp, i, vp]
    lib.ftk_dp_norm.argtypes = [pc, f, vp, vp, vp, vp]
    lib.ftk_dp_update.argtypes = [pc, i, i, vp, vp, vp, f, f, f, f, i, vp]
    lib.ftk_dp_clear_pending.argtypes = [pc, vp]
    lib.ftk_dp_wait_params.argtypes = [pc, i, vp]
    for fn in (lib.ftk_dp_begin_step, lib.ftk_dp_bucket_reduce, lib.ftk_dp_norm, lib.ftk_dp_update,
               lib.ftk_dp_clear_pending, lib.ftk_dp_wait_params):
        fn.restype = C.c_int
    return lib


class FusedDataParallel:
    """Bucketed reduce-scatter + sharded AdamW + all-gather over peer memory.

    ``overlap=True`` launches each bucket's reduction on ``comm_stream`` as soon as its gradients are
    complete (needs :meth:`attach`); otherwise all buckets are launched after the backward pass.

    ``defer_update=True`` moves the AdamW update and the parameter all-gather of a step to the start
    of the next one, bucket by bucket in forward order on ``comm_stream``, so that they run under
    the forward pass: a step then consists of [update with the previous step's gradients | forward]
    -> backward | reductions -> norm exchange.  The arithmetic and its order are unchanged; the
    parameters in the arena lag the optimizer by one update until :meth:`flush` (called before
    state is read: checkpoints, evaluation, the end of training).  The forward pass must call
    :meth:`gate_param` before it reads a parameter (``models/gpt.py`` does); a model that does not
    gets all buckets waited for at the start of the step.

    ``wire`` is ``"bf16"`` (default) or ``"fp32"`` (twice the NVLink bytes, no rounding before the sum).
    """

    def __init__(self, arena, group: Optional[dist.ProcessGroup], device: torch.device, *,
                 bucket_elems: Optional[int] = None, wire: Optional[str] = None, overlap: bool = True,
                 defer_update: Optional[bool] = None):
        self.group, self.device = group, device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        if self.world > DP_MAX_RANKS:
            raise ValueError(f"at most {DP_MAX_RANKS} ranks per data-parallel group")
        if not getattr(arena, "symmetric", False):
            raise ValueError("FusedDataParallel needs an arena allocated in symmetric memory")
        self.arena = arena
        self.overlap = overlap and os.environ.get("FT_DP_OVERLAP", "1") != "0"
        if defer_update is None:
            defer_update = os.environ.get("FT_DP_DEFER", "1") != "0"
        self.defer_update = bool(defer_update)
        wire = wire or os.environ.get("FT_DP_WIRE", "bf16")
        if wire not in ("bf16", "fp32"):
            raise ValueError("wire must be 'bf16' or 'fp32'")
        self.wire = wire
        target = int(bucket_elems or float(os.environ.get("FT_DP_BUCKET_MB", "0")) * (1 << 19)
                     or DEFAULT_BUCKET_ELEMS)
        ranges = []
        for name, _ in arena.specs:
            off, shape = arena.offsets[name]
            n = 1
            for s in shape:
                n *= int(s)
            ranges.append((off, off + (n + arena.ALIGN - 1) // arena.ALIGN * arena.ALIGN))
        self.buckets = plan_buckets(ranges, arena.numel, self.world, target,
                                    forced_cuts=getattr(arena, "bucket_cuts", ()))
        self.total_shard = sum(b.shard for b in self.buckets)
        self.shard_len = self.total_shard
        # grids: narrow while the backward pass needs the SMs, wide for buckets that finish last
        self.ctas_overlap = int(os.environ.get("FT_DP_CTAS", REDUCE_CTAS))
        self.ctas_tail = max(self.ctas_overlap, int(os.environ.get("FT_DP_TAIL_CTAS", TAIL_CTAS)))
        self.ctas_update_overlap = int(os.environ.get("FT_DP_UPDATE_CTAS", UPDATE_OVERLAP_CTAS))
        nb = len(self.buckets)
        # peer-visible: inbox, flag block, sumsq slots
        wsize = 2 if wire == "bf16" else 4
        self.inbox = SymmetricBuffer(self.world * self.total_shard * wsize, group, device)
        flag_bytes = 3 * DP_MAX_BUCKETS * DP_MAX_RANKS * 8
        self.ctrl = SymmetricBuffer(flag_bytes + DP_MAX_RANKS * 4, group, device)
        # rank-local optimizer state for the owned shards only
        self.master = gather_arena_shard(self.buckets, arena.master, self.rank, self.total_shard)
        self.m = torch.zeros(self.total_shard, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.total_shard, dtype=torch.float32, device=device)
        arena.drop_full_optimizer_state()
        self.gshard = torch.zeros(self.total_shard, dtype=torch.float32, device=device)
        self.partial = torch.zeros(nb * self.ctas_tail, dtype=torch.float32, device=device)
        self.counters = torch.zeros(2 * DP_MAX_BUCKETS, dtype=torch.int32, device=device)
        # step sequence number: grows by one per step, never rewinds (the flags compare against it),
        # and lives on the device so a captured graph advances it on every replay
        self.seq_dev = torch.zeros((), dtype=torch.int64, device=device)
        self.ok_dev = torch.ones((), dtype=torch.int32, device=device)
        self.pending_dev = torch.zeros((), dtype=torch.int32, device=device)
        self.hyper_pending = torch.zeros(4, dtype=torch.float32, device=device)
        tbl = (_Bucket * nb)(*[_Bucket(b.lo, b.hi, b.shard, b.off) for b in self.buckets])
        self._bucket_host = torch.frombuffer(bytearray(bytes(tbl)), dtype=torch.int64).clone()
        self.bucket_dev = self._bucket_host.to(device)
        self._lib = _bind(_lib.load())
        self._tables = (self.inbox.peer_table(), arena.params_buf.peer_table(), self.ctrl.peer_table(),
                        self.ctrl.peer_table(flag_bytes))
        pv = C.POINTER(C.c_void_p)
        self._comm = _Comm(C.cast(self._tables[0], pv), C.cast(self._tables[1], pv), C.cast(self._tables[2], pv),
                           C.cast(self._tables[3], pv),
                           self.bucket_dev.data_ptr(), self.rank, self.world, nb, self.ctas_tail,
                           1 if wire == "fp32" else 0, self.gshard.data_ptr(), self.partial.data_ptr(),
                           self.counters.data_ptr(), self.seq_dev.data_ptr(), self.ok_dev.data_ptr(),
                           self.pending_dev.data_ptr(), self.hyper_pending.data_ptr(),
                           int(getattr(arena.params_buf, "mc_ptr", 0) or 0) or None)
        # True when the updated parameters are broadcast with multimem stores through NVSwitch
        self.nvls_params = bool(getattr(arena.params_buf, "mc_ptr", 0))
        self.comm_stream = torch.cuda.Stream(device=device)
        self._opt: Optional[Tuple[float, float, float, float]] = None   # (beta1, beta2, eps, weight_decay)
        # bucket completion tracking (host side, drives the launches while a step is recorded)
        self._leaf_bucket: Dict[int, int] = {}
        self._name_bucket: Dict[str, int] = {}
        self._writes_seen: Dict[int, int] = {}
        self._write_clock = 0
        self._last_write_at: Dict[int, int] = {}
        self._expected: Optional[List[int]] = None
        self._tail: List[bool] = [True] * nb        # buckets that finish with the backward pass
        self._remaining: List[int] = []
        self._launched: List[bool] = [False] * nb
        self._events: List[torch.cuda.Event] = []
        self._update_events: List[Optional[torch.cuda.Event]] = [None] * nb
        self._gated_upto = nb                        # buckets [0, _gated_upto) are safe to read this step
        self.uses_gates = False                      # set by the engine when the model calls gate_param
        self.launch_order: List[int] = []            # bucket order of the last recorded step
        # optional time marks on the main stream (GPU nanosecond timer): step start, first bucket of
        # parameters usable, backward pass issued, optimizer step joined; see exposed_ms()
        self.record_stamps = os.environ.get("FT_DP_STAMPS", "0") == "1"
        self.stamps = torch.zeros(4, dtype=torch.int64, device=device)
        self._stamped_first_gate = False
        if group is not None:
            dist.barrier(group=group)

    # ------------------------------------------------------------------ wiring to the tape
    def attach(self, tape, leaf_ids: Dict[str, int]) -> None:
        """Track in-place gradient writes of the arena's parameter leaves (``leaf_ids``: name -> tape id)."""
        for name, nid in leaf_ids.items():
            if name not in self.arena.offsets:
                continue
            off = self.arena.offsets[name][0]
            for bi, bk in enumerate(self.buckets):
                if bk.lo <= off < bk.hi:
                    self._leaf_bucket[int(nid)] = bi
                    self._name_bucket[name] = bi
                    break
        tape.leaf_grad_written_fn = self._leaf_written

    def _leaf_written(self, nid: int) -> None:
        b = self._leaf_bucket.get(int(nid))
        if b is None:
            return
        if self._expected is None:                  # first step: count the writes per bucket
            self._writes_seen[b] = self._writes_seen.get(b, 0) + 1
            self._write_clock += 1
            self._last_write_at[b] = self._write_clock
            return
        self._remaining[b] -= 1
        if self._remaining[b] == 0 and self.overlap and not self._launched[b]:
            self._launch_bucket(b)

    # ------------------------------------------------------------------ start of a step
    def begin_step(self) -> None:
        """First thing of a step, on the main stream: advance the sequence number, arm the ok word
        and, when the update is deferred, start the previous step's update on the communication stream."""
        main = torch.cuda.current_stream()
        if self.record_stamps:
            K.timestamp(self.stamps, 0)
        self._stamped_first_gate = False
        K._chk(self._lib.ftk_dp_begin_step(C.byref(self._comm), main.cuda_stream), "ftk_dp_begin_step")
        if self._expected is not None:
            self._remaining = list(self._expected)
        nb = len(self.buckets)
        self._launched = [False] * nb
        self._events = []
        self.launch_order = []
        self._gated_upto = nb
        if self.defer_update and self._opt is not None:
            self._launch_updates(per_bucket=True)
            self._gated_upto = 0
            if not self.uses_gates:
                self.gate_all()

    def _launch_updates(self, per_bucket: bool) -> None:
        """AdamW + all-gather of the pending gradients on the communication stream (after everything
        the main stream holds so far), one launch per bucket or one for all."""
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.comm_stream.wait_event(ev)
        self._events.append(ev)
        cs, c = self.comm_stream.cuda_stream, C.byref(self._comm)
        b1, b2, eps, wd = self._opt
        nb = len(self.buckets)
        spans = [(b, b + 1) for b in range(nb)] if per_bucket else [(0, nb)]
        for lo, hi in spans:
            # the first bucket gates the forward pass and gets the whole GPU; the others run under it
            ctas = UPDATE_CTAS if (lo == 0 or not per_bucket) else self.ctas_update_overlap
            K._chk(self._lib.ftk_dp_update(c, lo, hi, self.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                                           b1, b2, eps, wd, ctas, cs), "ftk_dp_update")
            if per_bucket:
                e = torch.cuda.Event()
                e.record(self.comm_stream)
                self._update_events[lo] = e
        K._chk(self._lib.ftk_dp_clear_pending(c, cs), "ftk_dp_clear_pending")

    def gate_param(self, name: str) -> None:
        """Called by the forward pass before it reads parameter ``name``: makes the main stream wait
        until the bucket holding it (and every earlier one) has this step's values from all ranks."""
        b = self._name_bucket.get(name)
        if b is not None:
            self._gate_upto(b + 1)

    def gate_all(self) -> None:
        self._gate_upto(len(self.buckets))

    def _gate_upto(self, n: int) -> None:
        main = torch.cuda.current_stream()
        c = C.byref(self._comm)
        while self._gated_upto < n:
            b = self._gated_upto
            ev = self._update_events[b]
            if ev is not None:
                main.wait_event(ev)                                        # this rank's shard of the bucket
            K._chk(self._lib.ftk_dp_wait_params(c, b, main.cuda_stream), "ftk_dp_wait_params")   # the peers' shards
            self._gated_upto += 1
        if self.record_stamps and not self._stamped_first_gate:
            K.timestamp(self.stamps, 1)
            self._stamped_first_gate = True

    # ------------------------------------------------------------------ during / after the backward pass
    def _launch_bucket(self, b: int) -> None:
        """Push + reduce of bucket ``b`` on the communication stream, after everything the main stream
        has been given so far (that includes the kernels that wrote the bucket's gradients)."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.comm_stream.wait_event(ev)
        self._events.append(ev)
        ctas = self.ctas_tail if (self._tail[b] or not self.overlap) else self.ctas_overlap
        K._chk(self._lib.ftk_dp_bucket_reduce(C.byref(self._comm), b, self.arena.grads.data_ptr(), ctas,
                                              self.comm_stream.cuda_stream), "ftk_dp_bucket_reduce")
        K._launches += 1            # two kernels behind one launcher call (the call itself counted one)
        self._launched[b] = True
        self.launch_order.append(b)

    def reduce_and_update(self, arena, hyper, opt, sumsq, grad_norm, step_dev, extra_sumsq=None) -> None:
        """``extra_sumsq``: device scalar with the squared norm of the gradients that only this rank
        holds (rank-local arenas); it enters the global norm that sets the clip factor."""
        nb = len(self.buckets)
        if self._expected is None and self._writes_seen:
            self._expected = [self._writes_seen.get(b, 0) for b in range(nb)]
            # buckets whose last gradient arrives with the last few writes of the backward pass have
            # nothing left to hide behind: they get the wide grid
            self._tail = [self._write_clock - self._last_write_at.get(b, self._write_clock) <= 2 for b in range(nb)]
        self._opt = (float(opt.beta1), float(opt.beta2), float(opt.eps), float(opt.weight_decay))
        if self._gated_upto < nb:
            self.gate_all()     # a forward pass that did not read every bucket still has to take them in
        # buckets whose gradients were not all written in place (or the first, counting step)
        for b in reversed(range(nb)):
            if not self._launched[b]:
                self._launch_bucket(b)
        cs, c = self.comm_stream.cuda_stream, C.byref(self._comm)
        if extra_sumsq is not None:                 # computed on the main stream just before this call
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(ev)
            self._events.append(ev)
        K._chk(self._lib.ftk_dp_norm(c, float(opt.grad_clip or 0.0), hyper.data_ptr(), grad_norm.data_ptr(),
                                     None if extra_sumsq is None else extra_sumsq.data_ptr(), cs), "ftk_dp_norm")
        main = torch.cuda.current_stream()
        if self.record_stamps:
            if not self._stamped_first_gate:
                K.timestamp(self.stamps, 1)
                self._stamped_first_gate = True
            K.timestamp(self.stamps, 2)
        main.wait_stream(self.comm_stream)
        if not self.defer_update:
            self._launch_updates(per_bucket=False)
            K._chk(self._lib.ftk_dp_wait_params(c, 0, cs), "ftk_dp_wait_params")
            main.wait_stream(self.comm_stream)
        if self.record_stamps:
            K.timestamp(self.stamps, 3)

    def exposed_ms(self) -> Optional[float]:
        """Time of the last step (ms) the main stream spent waiting for communication: from the start
        of the step until the first parameters could be read, plus from the end of the backward pass
        until the optimizer step was joined.  Needs ``record_stamps``; synchronises."""
        if not self.record_stamps:
            return None
        t = [int(x) for x in self.stamps.tolist()]
        self.exposed_parts_ms = ((t[1] - t[0]) / 1e6, (t[3] - t[2]) / 1e6)    # (start of step, end of step)
        return ((t[1] - t[0]) + (t[3] - t[2])) / 1e6

    def flush(self) -> None:
        """Apply a deferred update now (no-op when nothing is pending) and make every rank's
        parameters current.  Host-synchronising; not for the step path."""
        if self.defer_update and self._opt is not None:
            self._launch_updates(per_bucket=False)
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        torch.cuda.synchronize(self.device)
        if self.group is not None and self.world > 1:
            dist.barrier(group=self.group)         # every peer's stores into this arena are complete
            torch.cuda.synchronize(self.device)

    def discard_pending(self) -> None:
        """Forget reduced gradients that have not been applied (used when optimizer state is restored)."""
        torch.cuda.synchronize(self.device)
        self.pending_dev.zero_()

    # ------------------------------------------------------------------ state access
    def gather_master(self) -> torch.Tensor:
        """Full fp32 master weights in arena order on every rank (checkpointing; not on the step path)."""
        return self._gather(self.master)

    def _gather(self, local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            shards = [local]
        else:
            allv = torch.empty(self.world * self.total_shard, dtype=local.dtype, device=self.device)
            dist.all_gather_into_tensor(allv, local.contiguous(), group=self.group)
            shards = list(allv.view(self.world, self.total_shard))
        return scatter_shards_to_arena(self.buckets, shards, self.arena.numel)

    def gather_optimizer_state(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(master, m, v) in arena order on every rank: what a replicated optimizer would hold."""
        self.flush()
        return self._gather(self.master), self._gather(self.m), self._gather(self.v)

    def layout_tensor(self) -> torch.Tensor:
        """The bucket table ``[n_buckets, 4]`` = (lo, hi, shard, off) as float64 (checkpoint metadata)."""
        return self._bucket_host.view(-1, 4).to(torch.float64)

    def step_ok(self) -> bool:
        """Host read of the step's ok word (synchronises): False when a bounded wait ran out."""
        return bool(int(self.ok_dev.item()) == 1)


class NcclDataParallel:
    """Baseline / fallback: NCCL all-reduce of the flat fp32 gradient, then local fused AdamW."""

    eager_only = True   # the engine does not capture this path in a CUDA graph

    def __init__(self, arena, group: Optional[dist.ProcessGroup], device: torch.device):
        self.group, self.device = group, device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        self.arena = arena

    def reduce_and_update(self, arena, hyper, opt, sumsq, grad_norm, step_dev, extra_sumsq=None) -> None:
        if self.world > 1:
            dist.all_reduce(arena.grads, op=dist.ReduceOp.AVG, group=self.group)
        if opt.grad_clip is not None:
            K.sumsq(arena.grads, out=sumsq)
            if extra_sumsq is not None:            # rank-local gradients: summed over the ranks, then added
                ex = extra_sumsq.clone()
                if self.world > 1:
                    dist.all_reduce(ex, group=self.group)
                sumsq.add_(ex)
            K.clip_scale(sumsq, opt.grad_clip, hyper, grad_norm)
        K.adamw_dev(arena.master, arena.params, arena.grads, arena.m, arena.v, hyper,
                    beta1=opt.beta1, beta2=opt.beta2, eps=opt.eps, weight_decay=opt.weight_decay)
