"""Failure detection for multi-rank jobs, kept on the host.

The reference is a single process; its failure model is fail-closed typed errors plus the
strict / hardened mode split (strict rejects, hardened performs a bounded, ledger-recorded
fallback: ft-dispatch/src/lib.rs:1369-1383, ft-autograd/src/lib.rs:11744-11757).  The multi-GPU
rebuild keeps that model:

* ``RankHealth``: every rank publishes a heartbeat (its step counter and a wall-clock stamp) in
  the job's key-value store before each step and reads its peers' entries; a peer that
  announced a failure, or whose heartbeat is older than ``timeout_s``, raises :class:`PeerFailure`
  *before* the next kernel that would wait for that peer is launched.  A rank that fails calls
  ``announce_failure`` from its exception handler (best effort) and leaves between steps.
* device-side waits on peer flags are bounded (see ``csrc``); when one runs out the kernel
  records a code in the status word, which :func:`device_status_error` turns into
  :class:`DeviceWaitTimeout`.
* ``HardenedTrainer`` wraps the training engine: between steps it reads the status word and lets
  the ranks agree on it; in strict mode a failure is raised on every rank, in hardened mode the
  engine is switched to the NCCL all-reduce path for the rest of the run and the event is
  recorded in the evidence ledger.

Nothing here faults, traps or hangs a GPU: failures are raised on the host, and tests inject them
on the host (a rank that raises, exits or stops publishing).
"""
from __future__ import annotations

import json
import time
from typing import Callable, Dict, List, Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out (status word non-zero)."""

    def __init__(self, code: int, cta: int, name: str):
        super().__init__(f"device wait timed out: {name} (code {code}, CTA {cta})")
        self.code, self.cta, self.name = code, cta, name


class RankHealth:
    """Heartbeats through a ``torch.distributed`` store (TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, world: int, *, timeout_s: float = 30.0, prefix: str = "ft/health",
                 clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix, self.clock = timeout_s, prefix, clock
        self.step = 0
        self.beat(0)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: Optional[int] = None) -> None:
        if step is not None:
            self.step = step
        self.store.set(self._key("hb", self.rank), json.dumps({"step": self.step, "t": self.clock()}))

    def announce_failure(self, reason: str) -> None:
        try:
            self.store.set(self._key("failed", self.rank), json.dumps({"reason": reason, "step": self.step}))
        except Exception:
            pass

    def peer_states(self) -> Dict[int, dict]:
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            st = {"failed": None, "hb": None}
            if self.store.check([self._key("failed", r)]):
                st["failed"] = json.loads(self.store.get(self._key("failed", r)))
            if self.store.check([self._key("hb", r)]):
                st["hb"] = json.loads(self.store.get(self._key("hb", r)))
            out[r] = st
        return out

    def check_peers(self) -> None:
        """Raise :class:`PeerFailure` if a peer announced a failure or stopped beating."""
        now = self.clock()
        for r, st in self.peer_states().items():
            if st["failed"] is not None:
                raise PeerFailure(r, f"announced failure at step {st['failed'].get('step')}: {st['failed'].get('reason')}")
            hb = st["hb"]
            if hb is None:
                raise PeerFailure(r, "never published a heartbeat")
            if now - float(hb["t"]) > self.timeout_s:
                raise PeerFailure(r, f"no heartbeat for {now - float(hb['t']):.1f}s (last step {hb['step']})")

    def before_step(self, step: int) -> None:
        """Publish this rank's heartbeat, then make sure every peer is alive."""
        self.beat(step)
        self.check_peers()


_STATUS_NAMES = {1: "TMA data never landed", 2: "pipeline stage never released", 3: "accumulator never completed",
                 4: "accumulator never drained", 5: "a flag owned by another rank never reached the expected value",
                 6: "probabilities never arrived", 7: "bad argument",
                 8: "a warp barrier was abandoned after an abort elsewhere in the CTA",
                 9: "an index read from a tensor (a token id) was out of range; the access was skipped"}


def device_status_error(status_word: int) -> Optional[DeviceWaitTimeout]:
    """Translate the kernels' status word (0 = healthy) into a typed error."""
    if status_word == 0:
        return None
    code, cta = status_word & 0xFF, status_word >> 8
    return DeviceWaitTimeout(code, cta, _STATUS_NAMES.get(code, "unknown"))


class HardenedTrainer:
    """Strict / hardened failure policy around a :class:`TrainEngine` whose optimizer step runs
    through the fused peer-memory data-parallel kernels.

    The engine's step is a replayed CUDA graph, so nothing inside it can change course; the policy
    therefore lives on the host, between steps:

    * every ``check_every`` steps the device status word is read (``read_status``; it
      synchronises) and the ranks agree on the outcome (``agree``: an integer MAX over a host-side
      group, e.g. ``gloo`` - every rank must take the same branch, a rank that switched to a library
      collective while its peers still spin on peer flags would only move the failure);
    * a fused step whose bounded waits ran out has updated nothing: the kernels poison the norm
      exchange so that every rank skips the AdamW update and the all-gather of that step
      (``csrc/dp_fused.cu``), and the master weights, moments and parameters are those of the
      last good step;
    * strict mode raises :class:`DeviceWaitTimeout` on every rank; hardened mode records the event
      (ledger kind ``durability``), rebuilds the full fp32 optimizer state from the shards, swaps
      the engine's data-parallel object for ``fallback_factory()`` (the NCCL all-reduce path, run
      eagerly), and re-runs the last step if it was one of the skipped ones.
    """

    def __init__(self, engine, fallback_factory: Callable[[], object], *, mode: str = "strict",
                 read_status: Optional[Callable[[], int]] = None, agree: Optional[Callable[[int], int]] = None,
                 check_every: int = 16, ledger=None):
        if mode not in ("strict", "hardened"):
            raise ValueError("mode must be 'strict' or 'hardened'")
        self.engine, self.fallback_factory, self.mode = engine, fallback_factory, mode
        self.read_status, self.agree = read_status, agree or (lambda v: v)
        self.check_every, self.ledger = max(1, check_every), ledger
        self.fell_back = False
        self.events: List[dict] = []
        self._n = 0

    def step(self, ids_host, targets_host, *, read_loss: bool = True):
        loss = self.engine.step(ids_host, targets_host, read_loss=read_loss)
        self._n += 1
        if not self.fell_back and self.read_status is not None and self._n % self.check_every == 0:
            redo = self.poll()
            if redo:
                loss = self.engine.step_device(read_loss=read_loss)
        return loss

    def poll(self) -> bool:
        """Read and agree on the status; returns True when the caller should re-run the last step."""
        local = int(self.read_status())
        agreed = int(self.agree(local))
        if agreed == 0:
            return False
        err = device_status_error(local if local else agreed)
        ev = {"event": "dp_device_wait_timeout", "code": err.code, "cta": err.cta, "mode": self.mode,
              "step": self._n, "local_status": local, "agreed_status": agreed}
        self.events.append(ev)
        if self.ledger is not None:
            self.ledger.record("durability", "fused data-parallel step failed: " + str(err), ev)
        if self.mode == "strict":
            raise err
        dp = self.engine.dp
        last_skipped = bool(hasattr(dp, "step_ok") and not dp.step_ok())
        self.engine.switch_data_parallel(self.fallback_factory)
        self.fell_back = True
        ev["last_step_rerun"] = last_skipped
        return last_skipped


def gloo_max_agreement(group) -> Callable[[int], int]:
    """``agree`` callable for :class:`HardenedTrainer`: integer MAX over a host-side process group."""
    import torch
    import torch.distributed as dist

    def agree(v: int) -> int:
        t = torch.tensor([int(v)], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return int(t.item())
    return agree
