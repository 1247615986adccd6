"""Pipeline parallelism: GPipe and 1F1B schedules over point-to-point sends between consecutive stages.

The reference has no pipeline parallelism; this module only adds the scheduling and the
activation / gradient hand-off, every stage runs on the Deterministic Autograd Contract tape
like any other model code.  Transfers are ``torch.distributed`` point-to-point operations
(NCCL on GPUs, gloo on CPU).  A library such as NCCL runs all transfers between one pair of
ranks on one stream in the order they were posted and ignores tags, so the order of posting is
the protocol: every transfer is posted when the schedule reaches it (a send right after the
compute that produced it, a receive right before the compute that needs it), and when a send is
directly followed by a receive from the same neighbour - the steady state of 1F1B, where two
stages would otherwise both be sending first - the two are posted as one group
(``batch_isend_irecv``).  EVERY transfer goes through ``batch_isend_irecv``, a lone one as a
group of one: ProcessGroupNCCL runs grouped point-to-point operations on the group-wide
communicator and ungrouped ones on a two-rank communicator of their own, and a send on one
communicator never meets a receive on the other (a step that mixed the two forms ended in the
process group's timeout).  On the group-wide communicator all of a rank's transfers, to either
neighbour, run on one stream in posting order; before anything is posted,
:func:`check_pair_orders` (each pair on its own) and :func:`check_fifo_orders` (one queue per
rank over all its neighbours) replay the posting orders on the host and refuse a schedule in
which ranks would wait for each other.  Sends are only waited for at the end of the step, so
they overlap the compute of the following micro-batches.

NCCL sets up the connection of a (peer, direction) pair the first time a group uses it, with a
HOST-side handshake that returns only when the peer's host sets up its end.  A schedule group
such as "send activation 3 + receive gradient 3" would then hold back the send until the peer
posts its first gradient send, which the peer reaches only after that very activation has
arrived: the step would end in the process group's timeout.  So before its first step every
stage exchanges one small tensor with each neighbour in both directions, all four transfers in
one group that every rank posts at the same point (:func:`connect_neighbours`); afterwards no
group waits for a connection.

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

from typing import Callable, List, Optional, Sequence, Tuple

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


def stage_order(rank: int, world: int, n_micro: int, schedule: str) -> List[Tuple[str, int]]:
    """The fixed sequence of ``("f", m)`` / ``("b", m)`` items stage ``rank`` runs in one step."""
    M = n_micro
    if schedule == "gpipe":
        return [("f", m) for m in range(M)] + [("b", m) for m in reversed(range(M))]
    if schedule == "1f1b":
        warm = min(world - 1 - rank, M)
        order = [("f", m) for m in range(warm)]
        for k in range(M - warm):
            order += [("f", warm + k), ("b", k)]
        return order + [("b", m) for m in range(M - warm, M)]
    raise ValueError(f"unknown pipeline schedule {schedule!r}")


def comm_groups(rank: int, world: int, n_micro: int, schedule: str) -> List[List[Tuple[str, int, str, int]]]:
    """Posting order of stage ``rank``: a list of groups of ``(kind, peer, what, m)`` with ``kind`` in
    ``{"send", "recv"}``, ``what`` in ``{"act", "grad"}``.  Transfers in one group are posted together;
    groups are posted in list order.  A send joins the following receive's group when both go to
    the same neighbour and nothing is computed in between."""
    first, last = rank == 0, rank == world - 1
    groups: List[List[Tuple[str, int, str, int]]] = []
    carry: Optional[Tuple[str, int, str, int]] = None      # a send waiting to see what comes next
    for kind, m in stage_order(rank, world, n_micro, schedule):
        recv = None
        if kind == "f" and not first:
            recv = ("recv", rank - 1, "act", m)
        if kind == "b" and not last:
            recv = ("recv", rank + 1, "grad", m)
        if carry is not None:
            if recv is not None and recv[1] == carry[1]:
                groups.append([carry, recv])
                recv = None
            else:
                groups.append([carry])
            carry = None
        if recv is not None:
            groups.append([recv])
        if kind == "f" and not last:
            carry = ("send", rank + 1, "act", m)
        if kind == "b" and not first:
            carry = ("send", rank - 1, "grad", m)
    if carry is not None:
        groups.append([carry])
    return groups


def check_pair_orders(rank: int, world: int, n_micro: int, schedule: str) -> None:
    """Replay, on the host, the transfers between stage ``rank`` and each neighbour the way an in-order
    point-to-point stream executes them: the head groups of the two sides run concurrently, a send
    completes with the matching receive, a group retires when all of its transfers have.  Raises
    ``RuntimeError`` if neither head can make progress (the ranks would wait for each other)."""
    for peer in (rank - 1, rank + 1):
        if peer < 0 or peer >= world:
            continue
        mine = [[t for t in g if t[1] == peer] for g in comm_groups(rank, world, n_micro, schedule)]
        theirs = [[t for t in g if t[1] == rank] for g in comm_groups(peer, world, n_micro, schedule)]
        a = [set((k, w, m) for k, _, w, m in g) for g in mine if g]
        b = [set((k, w, m) for k, _, w, m in g) for g in theirs if g]
        while a and b:
            matched = [(k, w, m) for (k, w, m) in a[0] if (("recv" if k == "send" else "send"), w, m) in b[0]]
            if not matched:
                raise RuntimeError(f"pipeline schedule '{schedule}' would deadlock between stages {rank} and {peer}: "
                                   f"{sorted(a[0])} faces {sorted(b[0])}")
            for k, w, m in matched:
                a[0].discard((k, w, m))
                b[0].discard((("recv" if k == "send" else "send"), w, m))
            if not a[0]:
                a.pop(0)
            if b and not b[0]:
                b.pop(0)
        if a or b:
            raise RuntimeError(f"pipeline schedule '{schedule}': unmatched transfers between stages {rank} and {peer}")


def check_fifo_orders(world: int, n_micro: int, schedule: str) -> None:
    """Replay the whole pipeline with ONE in-order queue of groups per rank (all neighbours together,
    the way grouped point-to-point operations run on a group-wide NCCL communicator): the head groups
    of all ranks are in flight, a transfer completes when the peer's head group holds its counterpart,
    a group retires when all of its transfers have.  Raises ``RuntimeError`` when no head can progress."""
    queues = [[set((k, p, w, m) for k, p, w, m in g) for g in comm_groups(r, world, n_micro, schedule)]
              for r in range(world)]
    while any(queues):
        progress = False
        for r in range(world):
            if not queues[r]:
                continue
            for k, p, w, m in sorted(queues[r][0]):
                other = ("recv" if k == "send" else "send", r, w, m)
                if queues[p] and other in queues[p][0]:
                    queues[r][0].discard((k, p, w, m))
                    queues[p][0].discard(other)
                    progress = True
        for r in range(world):
            while queues[r] and not queues[r][0]:
                queues[r].pop(0)
                progress = True
        if not progress:
            heads = {r: sorted(q[0]) for r, q in enumerate(queues) if q}
            raise RuntimeError(f"pipeline schedule '{schedule}' would deadlock on in-order queues: heads {heads}")


_CONNECTED = set()


def connect_neighbours(rank: int, world: int, group: Optional[dist.ProcessGroup], device) -> None:
    """Once per (group, device): a symmetric exchange of one element with the previous and the next stage,
    both directions in one group, so that every point-to-point connection the schedules use exists
    before a schedule group depends on it.  Collective over the stages (all call it at the same point)."""
    key = (id(group) if group is not None else 0, str(device))
    if key in _CONNECTED or world < 2 or dist.get_backend(group) == "gloo":
        return
    peer = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    keep, ops = [], []
    for nb in (rank + 1, rank - 1):
        if 0 <= nb < world:
            out, inp = torch.zeros(1, device=device), torch.empty(1, device=device)
            keep += [out, inp]
            ops += [dist.P2POp(dist.isend, out, peer(nb), group), dist.P2POp(dist.irecv, inp, peer(nb), group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    torch.cuda.synchronize(device)
    _CONNECTED.add(key)


class GPipeStage:
    """One stage of a pipeline (GPipe or 1F1B order).

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
        backwards, so at most ``world - rank`` micro-batches are live on a stage: the values and
        saved tensors of a micro-batch's nodes are dropped as soon as its backward has run
        (``max_live`` counts micro-batches whose activations are held).  Both orders are fixed, hence
        replayable; they differ in the order parameter gradients are summed."""
        tape, M = self.tape, n_micro
        check_pair_orders(self.rank, self.world, M, schedule)      # refuse an order that would hang, before posting
        check_fifo_orders(self.world, M, schedule)
        connect_neighbours(self.rank, self.world, self.group, device)
        groups = comm_groups(self.rank, self.world, M, schedule)
        order = stage_order(self.rank, self.world, M, schedule)
        self.last_order = order
        gi = [0]                                                    # next group to post
        bufs, works, posted, payloads, pending = {}, {}, set(), {}, []
        x_ids, y_ids, loss_ids = [None] * M, [None] * M, [None] * M
        node_span = [None] * M
        total = [0.0]
        self.max_live = live = 0

        def post_next() -> None:
            """Post the next group of the schedule: one transfer, or a send and a receive together."""
            g = groups[gi[0]]
            gi[0] += 1
            ops, keys = [], []
            for kind, peer, what, m in g:
                key = (kind, what, m)
                tag = m if what == "act" else 1000 + m            # honoured by gloo, ignored by NCCL
                if kind == "recv":
                    bufs[key] = torch.empty(tuple(in_shape if what == "act" else out_shape), dtype=dtype, device=device)
                    ops.append(dist.P2POp(dist.irecv, bufs[key], self._peer(peer), self.group, tag))
                else:
                    ops.append(dist.P2POp(dist.isend, payloads.pop(key), self._peer(peer), self.group, tag))
                keys.append(key)
            # always as a group, also a lone transfer: grouped and ungrouped NCCL point-to-point
            # operations use different communicators and never match each other
            ws = dist.batch_isend_irecv(ops)
            for n, key in enumerate(keys):
                works[key] = [ws[n]] if len(ws) == len(keys) else list(ws)   # a coalesced group has one handle
                posted.add(key)
                if key[0] == "send":
                    pending.extend(works[key])

        def wait_recv(key) -> torch.Tensor:
            while key not in posted:
                post_next()
            for w in works[key]:
                w.wait()
            return bufs.pop(key)

        def send(key, tensor: torch.Tensor) -> None:
            """Hand a payload to the schedule.  A send that stands alone in its group is posted at once;
            one grouped with the next receive from the same neighbour is posted when that receive is."""
            payloads[key] = tensor
            while gi[0] < len(groups) and all(k == "send" and (k, w, m) in payloads for k, _, w, m in groups[gi[0]]):
                post_next()

        def forward(m: int) -> None:
            lo = len(tape)
            if self.first:
                x = tape.leaf(micro_inputs[m], requires_grad=False)
            else:
                x = tape.leaf(wait_recv(("recv", "act", m)), requires_grad=True)
            y = self.stage_fn(tape, x, m)
            x_ids[m], y_ids[m] = x, y
            if self.last:
                loss_ids[m] = self.loss_fn(tape, y, targets[m], m)
            else:
                send(("send", "act", m), tape.value(y).detach().contiguous())
            node_span[m] = (lo, len(tape))

        def backward(m: int) -> None:
            if self.last:
                root = loss_ids[m]
                total[0] += float(tape.value(root))
                seed = torch.full_like(tape.value(root), 1.0 / M, dtype=tape.grad_dtype or tape.value(root).dtype)
            else:
                g = wait_recv(("recv", "grad", m))
                root = y_ids[m]
                seed = g.to(tape.grad_dtype) if tape.grad_dtype is not None else g
            # the micro-batch graphs share the parameter leaves: the graph stays on the tape until the
            # caller truncates it after the step, but this micro-batch's activations are released below
            report = tape.backward(root, BackwardOptions(retain_graph=True), seed=seed)
            if not self.first:
                gx = report.gradient(x_ids[m])
                send(("send", "grad", m), gx.to(dtype).contiguous())
            tape.release_values(*node_span[m])

        for kind, m in order:
            if kind == "f":
                forward(m)
                live += 1
                self.max_live = max(self.max_live, live)
            else:
                backward(m)
                live -= 1
        if gi[0] != len(groups) or payloads:
            raise RuntimeError("pipeline step ended with transfers of the schedule not posted")
        for r in pending:
            r.wait()
        return total[0] / M if self.last else None
