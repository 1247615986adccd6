"""Evidence-ledger record of one GPU training step.

The CPU session writes a dispatch decision per operator call (ft-api/src/lib.rs `record_dispatch`, the
`EvidenceLedger` of ft-runtime/src/lib.rs:46-55).  The GPU training path replays a captured CUDA graph, so
there is nothing to record per step; instead :class:`StepLedger` observes the ONE eager step that precedes the
capture and writes, per distinct (phase, operator, output shape, kernels) combination, one interned entry

    op=<operator> phase=fwd|bwd|optimizer mode=strict backend=sm100 kernel=[<launcher calls, GEMMs with their tile>]
    out=[shape] dtype=<dtype> count=<how many nodes of the step it covers>

followed by one `Backward` entry with the scheduler telemetry of that step (nodes executed, queue pushes and
pops, a fingerprint of the execution order).  The kernel names are the launcher calls that were actually made
while the node's forward rule (or backward rule) ran, collected through ``ops.kernels.trace_*``: the ledger
names what was launched, not what a table says should have been.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch

from ..ops import kernels as K
from ..runtime.ledger import EvidenceKind, EvidenceLedger


class StepLedger:
    def __init__(self, tape, ledger: EvidenceLedger, mode: str = "strict"):
        self.tape, self.ledger, self.mode = tape, ledger, mode
        self._groups: "OrderedDict[tuple, int]" = OrderedDict()
        self._prev_hook = None
        self._prev_range = None
        self.entries_written = 0

    # ------------------------------------------------------------------ observers
    def _add(self, phase: str, op: str, value: Optional[torch.Tensor], kernels) -> None:
        shape = tuple(value.shape) if isinstance(value, torch.Tensor) else ()
        dtype = str(value.dtype).replace("torch.", "") if isinstance(value, torch.Tensor) else "-"
        key = (phase, op, shape, dtype, tuple(kernels))
        self._groups[key] = self._groups.get(key, 0) + 1

    def _on_record(self, nid: int, op: str, value: torch.Tensor) -> None:
        self._add("fwd", op, value, K.trace_take())
        if self._prev_hook is not None:
            self._prev_hook(nid, op, value)

    class _Rule:
        def __init__(self, outer: "StepLedger", name: str):
            self.outer, self.name, self.inner = outer, name, None

        def __enter__(self):
            K.trace_take()                                   # whatever ran between rules (gradient accumulation)
            if self.outer._prev_range is not None:
                self.inner = self.outer._prev_range(self.name)
                self.inner.__enter__()
            return self

        def __exit__(self, *exc):
            if self.inner is not None:
                self.inner.__exit__(*exc)
            rule = self.name.split(":", 1)[-1].rsplit("#", 1)[0]
            self.outer._add("bwd", rule, None, K.trace_take())
            return False

    # ------------------------------------------------------------------ context
    def __enter__(self) -> "StepLedger":
        self._prev_hook, self._prev_range = self.tape.record_hook, self.tape.range_fn
        self.tape.record_hook = self._on_record
        self.tape.range_fn = lambda name: StepLedger._Rule(self, name)
        K.trace_begin()
        return self

    def mark_optimizer(self) -> None:
        """Call after the backward pass and again after the optimizer: what was launched in between is the
        optimizer step (clip norm, AdamW, data-parallel reduction kernels)."""
        ks = K.trace_take()
        if ks:
            self._add("optimizer", "optimizer_step", None, ks)

    def __exit__(self, *exc) -> bool:
        self.mark_optimizer()
        K.trace_end()
        self.tape.record_hook, self.tape.range_fn = self._prev_hook, self._prev_range
        if exc and exc[0] is not None:
            return False
        for (phase, op, shape, dtype, kernels), count in self._groups.items():
            self.ledger.record(EvidenceKind.Dispatch,
                               "op=%s phase=%s mode=%s backend=sm100 kernel=[%s] out=%s dtype=%s count=%d" %
                               (op, phase, self.mode, ", ".join(kernels) or "-", list(shape), dtype, count))
            self.entries_written += 1
        return False

    def record_backward(self, report) -> None:
        """One ``Backward`` entry with the scheduler telemetry of the observed step."""
        order = [s.node for s in getattr(report, "steps", [])]
        h = 0xcbf29ce484222325
        for n in order:
            h = ((h ^ (n & 0xFFFFFFFFFFFFFFFF)) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
        tel = getattr(report, "telemetry", None)
        self.ledger.record(EvidenceKind.Backward,
                           "backward nodes=%d queue_pushes=%s queue_pops=%s order_fnv1a=%016x" %
                           (len(order), getattr(tel, "queue_pushes", "-"), getattr(tel, "queue_pops", "-"), h))
        self.entries_written += 1
