"""Save / resume the full training state of a :class:`TrainEngine`, one FTSV file per rank.

What is stored (all fp32 / f64, in the reference's state-dict container, ft-serialize FTSV:
sorted keys, shape, dtype tag, raw little-endian data - no pickle):

* ``optim.master`` / ``optim.m`` / ``optim.v``: fp32 master weights and AdamW moments of the
  replicated arena - the whole arena on a single GPU, this rank's shard under
  ``FusedDataParallel`` (keys end in ``@bshard{rank}`` and come with the bucket table
  ``<key>@layout``, so ``consolidate_shards`` can rebuild the unsharded, arena-ordered tensors);
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
    if hasattr(engine, "sync_parameters"):
        engine.sync_parameters()          # a deferred optimizer update belongs to the state that is saved
    a = engine.model.arena
    sharded = engine.dp is not None and a.master is None
    own = engine.dp if sharded else a
    suffix = f"@bshard{rank}" if sharded else ""
    sd = {
        "optim.master" + suffix: own.master, "optim.m" + suffix: own.m, "optim.v" + suffix: own.v,
        f"rank{rank}.step": engine.step_dev.reshape(1).to(torch.float64),
        f"rank{rank}.hyper": engine.hyper,
    }
    if sharded:
        # the bucket table (lo, hi, shard, off per bucket) lets consolidate_shards put the pieces back
        for k in ("optim.master", "optim.m", "optim.v"):
            sd[k + "@layout"] = engine.dp.layout_tensor()
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
    suffix = f"@bshard{rank}" if sharded else ""
    dev = engine.step_dev.device

    def put(dst: torch.Tensor, key: str) -> None:
        src = sd[key]
        if src.numel() != dst.numel():
            raise ValueError(f"{key}: checkpoint has {src.numel()} elements, the engine expects {dst.numel()}")
        dst.copy_(src.to(dev).reshape(dst.shape))

    if sharded and hasattr(engine.dp, "discard_pending"):
        engine.dp.discard_pending()       # gradients reduced before the load belong to the old trajectory
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


# --------------------------------------------------------------------------- job state sidecar
def job_state(*, scheduler=None, session=None, loader=None, step: int = 0, extra: Dict = None) -> Dict:
    """Host-side state that, with the tensors above, makes a resumed job replay the original one:
    learning-rate scheduler (``SchedulerState``: last_epoch / last_lrs / extra, ft-optim
    ``:2301``), the session's xoshiro256++ stream (four 64-bit words), and the data loader's
    position (LCG state, cursor, current shuffled order).  Plain JSON-able values."""
    out: Dict = {"schema": "ft-job-state-v1", "step": int(step), "extra": dict(extra or {})}
    if scheduler is not None:
        st = scheduler.state()
        out["scheduler"] = {"last_epoch": int(st.last_epoch), "last_lrs": [float(x) for x in st.last_lrs],
                            "extra": {k: float(v) for k, v in st.extra.items()}}
    if session is not None:
        out["prng"] = [int(session.rng.state[i]) for i in range(4)]
    if loader is not None:
        out["loader"] = loader.state_dict()
    return out


def restore_job_state(state: Dict, *, scheduler=None, session=None, loader=None) -> int:
    """Inverse of :func:`job_state`; returns the saved step.  Unknown schemas are rejected."""
    if state.get("schema") != "ft-job-state-v1":
        raise ValueError(f"unknown job-state schema {state.get('schema')!r}")
    if scheduler is not None and "scheduler" in state:
        from ..optim.schedulers import SchedulerState
        s = state["scheduler"]
        scheduler.load_state(SchedulerState(int(s["last_epoch"]), list(s["last_lrs"]), dict(s["extra"])))
    if session is not None and "prng" in state:
        words = state["prng"]
        if len(words) != 4:
            raise ValueError("the PRNG state has four 64-bit words")
        for i, w in enumerate(words):
            session.rng.state[i] = int(w) & ((1 << 64) - 1)
    if loader is not None and "loader" in state:
        loader.load_state_dict(state["loader"])
    return int(state.get("step", 0))


def save_job_state(path: str, **kw) -> str:
    import json
    with open(path, "w") as f:
        json.dump(job_state(**kw), f, sort_keys=True, separators=(",", ":"))
    return path


def load_job_state(path: str, **kw) -> int:
    import json
    with open(path) as f:
        return restore_job_state(json.load(f), **kw)
