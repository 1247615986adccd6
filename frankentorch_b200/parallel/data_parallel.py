"""Data parallelism (ZeRO-1 style) with the gradient reduce-scatter fused into the sharded
AdamW update and the parameter all-gather, all through in-kernel NVLink peer accesses.

``FusedDataParallel`` owns the peer-visible gradient / parameter arenas and the flag blocks;
``reduce_and_update`` launches the four kernels of ``csrc/dp_fused.cu`` on the current stream
(capturable in a CUDA graph: the step number lives in device memory).

``NcclDataParallel`` is the stock path - NCCL all-reduce of the flat gradient followed by the
single-GPU fused AdamW - kept as the baseline and as the hardened-mode fallback.

The reference has no distributed training at all (docs/planning/FEATURE_PARITY.md:176); the
single-process optimizer semantics that must be preserved are those of AdamW,
ft-optim/src/lib.rs:800-1085.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as K
from .symm import SymmetricBuffer

DP_MAX_RANKS = 16
REDUCE_CTAS = 296


def shard_multiple(world: int) -> int:
    """The flat arena length must be a multiple of this so shards are float4-aligned."""
    return 1024 * max(world, 1)


class FusedDataParallel:
    def __init__(self, arena, group: dist.ProcessGroup, device: torch.device):
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > DP_MAX_RANKS:
            raise ValueError(f"at most {DP_MAX_RANKS} ranks per data-parallel group")
        n = arena.numel
        if n % shard_multiple(self.world):
            raise ValueError("arena length must be padded to shard_multiple(world)")
        self.shard_len = n // self.world
        if not getattr(arena, "symmetric", False):
            raise ValueError("FusedDataParallel needs an arena allocated in symmetric memory")
        self.arena = arena
        # flags: [3 phases][DP_MAX_RANKS] u64, then sumsq slots [DP_MAX_RANKS] fp32
        self.ctrl = SymmetricBuffer(3 * DP_MAX_RANKS * 8 + DP_MAX_RANKS * 4, group, device)
        self.slots_off = 3 * DP_MAX_RANKS * 8
        lo, hi = self.rank * self.shard_len, (self.rank + 1) * self.shard_len
        # optimizer state is kept for the owned shard only
        self.master = arena.master[lo:hi].clone()
        self.m = torch.zeros(self.shard_len, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.shard_len, dtype=torch.float32, device=device)
        arena.drop_full_optimizer_state()
        self.gshard = torch.empty(self.shard_len, dtype=torch.float32, device=device)
        self.partial = torch.zeros(REDUCE_CTAS, dtype=torch.float32, device=device)
        self.gate = torch.zeros(1, dtype=torch.int64, device=device)
        # communication sequence number: grows by one per call, never rewinds (the flags compare
        # against it), and lives on the device so a captured graph advances it on every replay
        self.seq_dev = torch.zeros((), dtype=torch.int64, device=device)
        self._seq_scratch = torch.zeros(4, dtype=torch.float32, device=device)
        lib = _lib.load()
        self._fn = lib.ftk_dp_step
        vpp = C.POINTER(C.c_void_p)
        self._fn.argtypes = [vpp, vpp, vpp, vpp, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p,
                             C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_void_p]
        self._fn.restype = C.c_int
        self._grads_tbl = arena.grads_buf.peer_table()
        self._params_tbl = arena.params_buf.peer_table()
        self._flags_tbl = self.ctrl.peer_table()
        self._slots_tbl = self.ctrl.peer_table(self.slots_off)
        dist.barrier(group=group)

    def reduce_and_update(self, arena, hyper, opt, sumsq, grad_norm, step_dev) -> None:
        K.adamw_tick(self.seq_dev, self._seq_scratch, 0.5, 0.5)   # seq += 1 (reuses the counter kernel)
        rc = self._fn(self._grads_tbl, self._params_tbl, self._flags_tbl, self._slots_tbl, self.rank, self.world,
                      self.gshard.data_ptr(), self.partial.data_ptr(), REDUCE_CTAS, self.gate.data_ptr(),
                      self.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr(), self.shard_len,
                      self.seq_dev.data_ptr(), hyper.data_ptr(), grad_norm.data_ptr(),
                      float(opt.grad_clip or 0.0), float(opt.beta1), float(opt.beta2), float(opt.eps),
                      float(opt.weight_decay), torch.cuda.current_stream().cuda_stream)
        K._chk(rc, "ftk_dp_step")
        K._launches += 3   # four kernels in one launcher call

    def gather_master(self) -> torch.Tensor:
        """Full fp32 master weights on every rank (checkpointing; not on the step path)."""
        full = torch.empty(self.shard_len * self.world, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(full, self.master, group=self.group)
        return full


class NcclDataParallel:
    """Baseline / fallback: NCCL all-reduce of the flat fp32 gradient, then local fused AdamW."""

    eager_only = True   # the engine does not capture this path in a CUDA graph

    def __init__(self, arena, group: dist.ProcessGroup, device: torch.device):
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.arena = arena

    def reduce_and_update(self, arena, hyper, opt, sumsq, grad_norm, step_dev) -> None:
        dist.all_reduce(arena.grads, op=dist.ReduceOp.AVG, group=self.group)
        if opt.grad_clip is not None:
            K.sumsq(arena.grads, out=sumsq)
            K.clip_scale(sumsq, opt.grad_clip, hyper, grad_norm)
        K.adamw_dev(arena.master, arena.params, arena.grads, arena.m, arena.v, hyper,
                    beta1=opt.beta1, beta2=opt.beta2, eps=opt.eps, weight_decay=opt.weight_decay)
