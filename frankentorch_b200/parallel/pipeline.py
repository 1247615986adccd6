"""Pipeline parallelism: GPipe and 1F1B schedules over point-to-point sends between consecutive stages.

The reference has no pipeline parallelism; this module only adds the scheduling and the
activation / gradient hand-off, every stage runs on the Deterministic Autograd Contract tape
like any other model code.  Transfers are ``torch.distributed`` point-to-point operations
(NCCL on GPUs, gloo on CPU) posted asynchronously: all receives of a phase are posted up front
and a send is only waited for when its buffer is needed again, so communication overlaps the
compute of the neighbouring micro-batches.

Schedule of one step with ``M`` micro-batches on stage ``r`` of ``W``:

  forward   m = 0..M-1 : recv activation (r > 0) -> stage_fn -> send activation (r < W-1)
                         / loss_fn on the last stage
  backward  m = M-1..0 : recv output gradient (r < W-1) -> tape.backward -> send input
                         gradient (r > 0)

Parameter gradients accumulate over the micro-batches in the tape's leaf accumulators in a fixed
order (micro-batch M-1 first), so a step is reproducible bit for bit.  The loss reported by the
last stage is the mean over micro-batches; every micro-batch's backward is seeded with ``1 / M``.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..autograd import functions_nn, functions_shape  # noqa: F401  (they register their operators)
from ..autograd.functions import OPS
from ..autograd.tape import BackwardOptions, TensorTape


def tape_op(tape: TensorTape, name: str, inputs: Sequence[int], **kw) -> int:
    """Record operator ``name`` of the VJP rule table on ``tape`` (what the session's
    ``tensor_<name>`` methods do, without ledger and autocast)."""
    op = OPS[name]
    vals = [tape.value(i) for i in inputs]
    out = op.fwd(*vals, **kw)
    rg = tape.grad_enabled and any(tape.nodes[i].requires_grad for i in inputs)
    vjp = None
    if rg and op.vjp is not None:
        gdt = tape.grad_dtype

        def vjp(g, targets, _op=op, _vals=vals, _out=out, _kw=kw):
            ins = [v.to(gdt) if (gdt is not None and v.is_floating_point()) else v for v in _vals]
            o = _out.to(gdt) if (gdt is not None and _out.is_floating_point()) else _out
            return list(_op.vjp(g, ins, o, _kw))
    return tape.record(name, list(inputs), out, vjp, op.rule)


class GPipeStage:
    """One stage of a GPipe pipeline.

    ``stage_fn(tape, x_id, m)`` maps the tape id of the stage input of micro-batch ``m`` to the
    id of the stage output.  On the last stage ``loss_fn(tape, y_id, target, m)`` returns the id
    of the scalar loss of that micro-batch.
    """

    def __init__(self, tape: TensorTape, stage_fn: Callable, *, rank: int, world: int,
                 group: Optional[dist.ProcessGroup] = None, loss_fn: Optional[Callable] = None):
        self.tape, self.stage_fn, self.loss_fn = tape, stage_fn, loss_fn
        self.rank, self.world, self.group = rank, world, group
        self.first, self.last = rank == 0, rank == world - 1
        if self.last and loss_fn is None:
            raise ValueError("the last stage needs a loss_fn")

    def _peer(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def step(self, *, n_micro: int, micro_inputs: Optional[List[torch.Tensor]] = None,
             targets: Optional[List[torch.Tensor]] = None, in_shape: Optional[Sequence[int]] = None,
             out_shape: Optional[Sequence[int]] = None, dtype: torch.dtype = torch.float64,
             device: str = "cpu", schedule: str = "gpipe") -> Optional[float]:
        """Run forward and backward of ``n_micro`` micro-batches; returns the mean loss on the
        last stage (None elsewhere).  Parameter gradients are left in the tape's accumulators.

        ``schedule``: ``"gpipe"`` runs every forward, then the backwards from the last micro-batch
        to the first; ``"1f1b"`` runs ``world - 1 - rank`` warm-up forwards, then alternates one
        forward with one backward (micro-batches in ascending order) and drains the remaining
        backwards, so at most ``world - rank`` micro-batches are live on a stage.  Both orders are
        fixed, hence replayable; they differ in the order parameter gradients are summed."""
        if schedule not in ("gpipe", "1f1b"):
            raise ValueError(f"unknown pipeline schedule {schedule!r}")
        tape, M = self.tape, n_micro
        prev, nxt = self._peer(self.rank - 1) if not self.first else None, \
            self._peer(self.rank + 1) if not self.last else None
        # every receive of the step is posted up front; tags separate micro-batches and directions
        recv_bufs, recv_req, grad_bufs, grad_req = [], [], [], []
        if not self.first:
            for m in range(M):
                buf = torch.empty(tuple(in_shape), dtype=dtype, device=device)
                recv_bufs.append(buf)
                recv_req.append(dist.irecv(buf, src=prev, group=self.group, tag=m))
        if not self.last:
            for m in range(M):
                buf = torch.empty(tuple(out_shape), dtype=dtype, device=device)
                grad_bufs.append(buf)
                grad_req.append(dist.irecv(buf, src=nxt, group=self.group, tag=1000 + m))
        x_ids, y_ids, loss_ids = [None] * M, [None] * M, [None] * M
        pending = []
        total = [0.0]
        self.max_live = live = 0

        def forward(m: int) -> None:
            if self.first:
                x = tape.leaf(micro_inputs[m], requires_grad=False)
            else:
                recv_req[m].wait()
                x = tape.leaf(recv_bufs[m], requires_grad=True)
            y = self.stage_fn(tape, x, m)
            x_ids[m], y_ids[m] = x, y
            if self.last:
                loss_ids[m] = self.loss_fn(tape, y, targets[m], m)
            else:
                pending.append(dist.isend(tape.value(y).detach().contiguous(), dst=nxt, group=self.group, tag=m))

        def backward(m: int) -> None:
            if self.last:
                root = loss_ids[m]
                total[0] += float(tape.value(root))
                seed = torch.full_like(tape.value(root), 1.0 / M, dtype=tape.grad_dtype or tape.value(root).dtype)
            else:
                grad_req[m].wait()
                root = y_ids[m]
                seed = grad_bufs[m].to(tape.grad_dtype) if tape.grad_dtype is not None else grad_bufs[m]
            # the micro-batch graphs share the parameter leaves: keep them until the caller
            # truncates the tape after the step
            report = tape.backward(root, BackwardOptions(retain_graph=True), seed=seed)
            if not self.first:
                gx = report.gradient(x_ids[m])
                pending.append(dist.isend(gx.to(dtype).contiguous(), dst=prev, group=self.group, tag=1000 + m))

        if schedule == "gpipe":
            order = [("f", m) for m in range(M)] + [("b", m) for m in reversed(range(M))]
        else:
            warm = min(self.world - 1 - self.rank, M)
            order = [("f", m) for m in range(warm)]
            for k in range(M - warm):
                order += [("f", warm + k), ("b", k)]
            order += [("b", m) for m in range(M - warm, M)]
        self.last_order = order
        for kind, m in order:
            if kind == "f":
                forward(m)
                live += 1
                self.max_live = max(self.max_live, live)
            else:
                backward(m)
                live -= 1
        for r in pending:
            r.wait()
        return total[0] / M if self.last else None
