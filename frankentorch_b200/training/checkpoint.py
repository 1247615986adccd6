"""Save / resume the full training state of a :class:`TrainEngine`, one FTSV file per rank.

What is stored (all fp32 / f64, in the reference's state-dict container, ft-serialize FTSV:
sorted keys, shape, dtype tag, raw little-endian data - no pickle):

* ``optim.master`` / ``optim.m`` / ``optim.v``: fp32 master weights and AdamW moments of the
  replicated arena - the whole arena on a single GPU, this rank's shard under
  ``FusedDataParallel`` (keys end in ``@shard{rank}`` so ``consolidate_shards`` can rebuild the
  unsharded tensors);
* ``local{i}.master`` / ``.m`` / ``.v``: rank-local arenas (tensor-parallel shards, ZeRO-3 weight
  shards, this rank's experts);
* ``step`` (AdamW step counter) and ``hyper`` (learning rate, bias corrections, clip factor).

Resuming restores those tensors, rebuilds the bf16 compute copies from the masters and leaves the
captured CUDA graph intact (the graph reads the same buffers), so ``k`` steps + save + load +
``n - k`` steps reproduces ``n`` uninterrupted steps bit for bit.  Scheduler / data-loader
positions are plain Python state of their own objects (``optim.schedulers``, ``data``) and are
saved by their ``state_dict`` methods, as in the reference (SchedulerState, ft-optim).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..serialize.state_dict import load_state_dict, save_sharded


def _rank_world(engine):
    dp = engine.dp
    if dp is not None and hasattr(dp, "rank"):
        return int(dp.rank), int(dp.world)
    return 0, 1


def training_state_dict(engine) -> Dict[str, torch.Tensor]:
    """Tensors that define the optimizer trajectory of ``engine`` on this rank (CPU copies)."""
    rank, world = _rank_world(engine)
    a = engine.model.arena
    sharded = engine.dp is not None and a.master is None
    own = engine.dp if sharded else a
    suffix = f"@shard{rank}" if sharded else ""
    sd = {
        "optim.master" + suffix: own.master, "optim.m" + suffix: own.m, "optim.v" + suffix: own.v,
        f"rank{rank}.step": engine.step_dev.reshape(1).to(torch.float64),
        f"rank{rank}.hyper": engine.hyper,
    }
    for i, la in enumerate(engine.local_arenas):
        sd[f"rank{rank}.local{i}.master"] = la.master
        sd[f"rank{rank}.local{i}.m"] = la.m
        sd[f"rank{rank}.local{i}.v"] = la.v
    return {k: v.detach().to("cpu").contiguous() for k, v in sd.items()}


def save_training_state(engine, stem: str) -> str:
    """Write ``<stem>.rank{r}.ftsv`` for this rank; returns the path."""
    torch.cuda.synchronize()
    rank, _ = _rank_world(engine)
    return save_sharded(training_state_dict(engine), stem, rank)


def load_training_state(engine, stem: str) -> None:
    """Restore what :func:`save_training_state` wrote for this rank (same model, same world size)."""
    rank, world = _rank_world(engine)
    sd = load_state_dict(f"{stem}.rank{rank}.ftsv")
    a = engine.model.arena
    sharded = engine.dp is not None and a.master is None
    own = engine.dp if sharded else a
    suffix = f"@shard{rank}" if sharded else ""
    dev = engine.step_dev.device

    def put(dst: torch.Tensor, key: str) -> None:
        src = sd[key]
        if src.numel() != dst.numel():
            raise ValueError(f"{key}: checkpoint has {src.numel()} elements, the engine expects {dst.numel()}")
        dst.copy_(src.to(dev).reshape(dst.shape))

    put(own.master, "optim.master" + suffix)
    put(own.m, "optim.m" + suffix)
    put(own.v, "optim.v" + suffix)
    engine.step_dev.copy_(sd[f"rank{rank}.step"].to(dev).to(torch.int64).reshape(()))
    put(engine.hyper, f"rank{rank}.hyper")
    for i, la in enumerate(engine.local_arenas):
        put(la.master, f"rank{rank}.local{i}.master")
        put(la.m, f"rank{rank}.local{i}.m")
        put(la.v, f"rank{rank}.local{i}.v")
        la.sync_shadow()
    # bf16 compute copy of the replicated arena
    if sharded:
        full = engine.dp.gather_master()
        a.params.copy_(full[: a.params.numel()])
    else:
        a.sync_shadow()
    torch.cuda.synchronize()
