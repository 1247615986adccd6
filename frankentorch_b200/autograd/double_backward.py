"""Graph-building backward (``create_graph=True``): gradients as tape nodes, so that a second
backward can differentiate through the first.

Reference behaviour: ``backward_create_graph`` and its ``cg_*`` helpers (ft-autograd/src/lib.rs
:15755-19498) append, for every rule applied during the backward pass, nodes that compute that
rule's contributions; custom functions need a tape-building backward for this
(``apply_function_with_create_graph``, :8951, :1520-1533).

Here every contribution is one node produced by :func:`torch_fn_node`: its value is the rule's own
formula ``vjp(g, inputs, out)[k]`` (so a first-order gradient has the same bits with or without
``create_graph``), and its derivative - needed only when a later backward reaches it - is taken by
differentiating that formula locally with ``torch.autograd`` inside the node.  The construction is
recursive (the derivative of a contribution node is again such a node), which gives derivatives of
any order while the tape keeps deciding what runs and in which order.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch


def _as_leaf(t: torch.Tensor) -> torch.Tensor:
    """``t`` itself when it already takes part in a local differentiation, else a fresh differentiable copy."""
    if not isinstance(t, torch.Tensor) or not (t.is_floating_point() or t.is_complex()):
        return t
    return t if t.requires_grad else t.detach().requires_grad_(True)


def torch_fn_node(tape, f: Callable[..., torch.Tensor], in_ids: Sequence[int], name: str, rule: str) -> int:
    """Record ``f(*values(in_ids))`` as one tape node.  ``f`` must be written in differentiable torch
    operations of its tensor arguments.  Backward of the node = local differentiation of ``f``;
    graph-building backward = further nodes of the same kind."""
    in_ids = list(in_ids)
    vals = [tape.value(i) for i in in_ids]
    with torch.no_grad():
        out = f(*vals)
    out = out.detach()
    diff = [k for k, v in enumerate(vals) if isinstance(v, torch.Tensor) and (v.is_floating_point() or v.is_complex())]

    def partial(k: int) -> Callable[..., torch.Tensor]:
        """``(gg, *ins) -> d<gg, f(ins)>/d ins[k]``, itself differentiable in all of its arguments."""
        def fk(gg, *ins):
            with torch.enable_grad():
                xs = [_as_leaf(t) for t in ins]
                y = f(*xs)
                if not y.requires_grad:                      # f does not depend on its differentiable arguments
                    return torch.zeros_like(ins[k])
                (g,) = torch.autograd.grad(y, [xs[k]], gg.to(y.dtype), allow_unused=True, create_graph=True)
            return g if g is not None else torch.zeros_like(ins[k])
        return fk

    def vjp(gg, targets):
        res: List[Optional[torch.Tensor]] = [None] * len(in_ids)
        need = [k for k in diff if tape.nodes[in_ids[k]].requires_grad]
        if not need:
            return res
        with torch.enable_grad():
            xs = [_as_leaf(v) if k in need else v for k, v in enumerate(vals)]
            y = f(*xs)
            if not y.requires_grad:
                return res
            gs = torch.autograd.grad(y, [xs[k] for k in need], gg.to(y.dtype), allow_unused=True)
        for k, g in zip(need, gs):
            res[k] = g
        return res

    def cg(g_id: int) -> List[Optional[int]]:
        res: List[Optional[int]] = [None] * len(in_ids)
        for k in diff:
            if tape.nodes[in_ids[k]].requires_grad:
                res[k] = torch_fn_node(tape, partial(k), [g_id] + in_ids, f"grad[{name}]#{k}", f"d({rule})")
        return res

    return tape.record(name, in_ids, out, vjp, rule, cg=cg)


def op_cg(tape, op, kw: dict, in_ids: Sequence[int]) -> Callable[[int], List[Optional[int]]]:
    """Graph-building backward of a rule-table operator: contribution ``k`` is the node
    ``vjp(g, inputs, fwd(inputs))[k]`` with inputs ``[g, *inputs]``."""
    in_ids = list(in_ids)

    def contribution(k: int) -> Callable[..., torch.Tensor]:
        def fk(g, *ins):
            ins = list(ins)
            out = op.fwd(*ins, **kw)
            c = op.vjp(g, ins, out, kw)[k]
            return c if c is not None else torch.zeros_like(ins[k])
        return fk

    def cg(g_id: int) -> List[Optional[int]]:
        res: List[Optional[int]] = [None] * len(in_ids)
        for k, i in enumerate(in_ids):
            v = tape.value(i)
            if not tape.nodes[i].requires_grad or not (v.is_floating_point() or v.is_complex()):
                continue
            res[k] = torch_fn_node(tape, contribution(k), [g_id] + in_ids, f"grad[{op.name}]#{k}", op.rule)
        return res
    return cg
