"""Scalar tape of the Deterministic Autograd Contract.

Reference: ft-autograd/src/lib.rs - ``Tape`` :1562, ``leaf`` :1600, ``binary`` :3185,
``backward_with_options`` :3256-4079 (same scheduler as the tensor tape: max-heap on node id,
dependency counters, telemetry), ``BackwardReport`` (:1068).  Every forward op resolves a
dispatch decision (kernel string ``autograd_cpu::add_scalar`` etc.) that the session records
in the evidence ledger.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

from ..dispatch.keys import DispatchDecision, DispatchKeySet, dispatch_scalar_binary
from ..runtime import native
from ..runtime.ledger import ExecutionMode
from .tape import (BackwardOptions, ReentrantDepthExceeded, ReentrantPolicy, TensorSchedulerTelemetry, AutogradError)


class UnknownNode(AutogradError):
    pass


class RootDoesNotRequireGrad(AutogradError):
    pass


class GraphConsumed(AutogradError):
    pass


@dataclass
class BackwardStep:
    node: int
    incoming_grad: float
    rule: str


@dataclass
class BackwardReport:
    gradients: List[Optional[float]]
    steps: List[BackwardStep]
    telemetry: TensorSchedulerTelemetry

    def gradient(self, node: int) -> Optional[float]:
        return self.gradients[node] if 0 <= node < len(self.gradients) else None


_BINARY_RULES: Dict[str, Tuple[str, Callable[[float, float, float], Tuple[float, float]]]] = {
    "add": ("d(a+b)/da=1; d(a+b)/db=1", lambda g, a, b: (g, g)),
    "sub": ("d(a-b)/da=1; d(a-b)/db=-1", lambda g, a, b: (g, -g)),
    "mul": ("d(a*b)/da=b; d(a*b)/db=a", lambda g, a, b: (g * b, g * a)),
    "div": ("d(a/b)/da=1/b; d(a/b)/db=-(a/b^2)", lambda g, a, b: (g / b, -g * a / (b * b))),
    "min": ("d(min(a,b))/da=1(a<b) or 0.5(a=b); db=1(b<a) or 0.5(a=b)",
            lambda g, a, b: (g * (1.0 if a < b else 0.5 if a == b else 0.0), g * (1.0 if b < a else 0.5 if a == b else 0.0))),
    "max": ("d(max(a,b))/da=1(a>b) or 0.5(a=b); db=1(b>a) or 0.5(a=b)",
            lambda g, a, b: (g * (1.0 if a > b else 0.5 if a == b else 0.0), g * (1.0 if b > a else 0.5 if a == b else 0.0))),
}
_UNARY_RULES: Dict[str, Tuple[str, Callable[[float], float], Callable[[float, float, float], float]]] = {
    "neg": ("d(-x)/dx=-1", lambda x: -x, lambda g, x, y: -g),
    "abs": ("d|x|/dx=sign(x)", abs, lambda g, x, y: g * (1.0 if x > 0 else -1.0 if x < 0 else 0.0)),
    "exp": ("d(exp(x))/dx=exp(x)", math.exp, lambda g, x, y: g * y),
    "log": ("d(ln(x))/dx=1/x", math.log, lambda g, x, y: g / x),
    "relu": ("d(relu(x))/dx=1 if x>0 else 0", lambda x: x if x > 0 else 0.0, lambda g, x, y: g if x > 0 else 0.0),
    "sigmoid": ("d(sigmoid(x))/dx=sigmoid(x)*(1-sigmoid(x))", lambda x: 1 / (1 + math.exp(-x)), lambda g, x, y: g * y * (1 - y)),
    "tanh": ("d(tanh(x))/dx=1-tanh(x)^2", math.tanh, lambda g, x, y: g * (1 - y * y)),
    "sqrt": ("d(sqrt(x))/dx=0.5/sqrt(x)", math.sqrt, lambda g, x, y: g * 0.5 / y),
    "sin": ("d(sin(x))/dx=cos(x)", math.sin, lambda g, x, y: g * math.cos(x)),
    "cos": ("d(cos(x))/dx=-sin(x)", math.cos, lambda g, x, y: -g * math.sin(x)),
    "square": ("d(x^2)/dx=2x", lambda x: x * x, lambda g, x, y: g * 2 * x),
    "reciprocal": ("d(1/x)/dx=-1/x^2", lambda x: 1.0 / x, lambda g, x, y: -g * y * y),
}


@dataclass
class _Node:
    value: float
    requires_grad: bool
    op: str
    inputs: Tuple[int, ...]
    rule: str


class Tape:
    def __init__(self, mode: ExecutionMode = ExecutionMode.Strict):
        self.mode = mode
        self._lib = native.load()
        self._h = self._lib.ftc_tape_new()
        self.nodes: List[_Node] = []

    def __del__(self):
        try:
            if self._h:
                self._lib.ftc_tape_free(self._h)
                self._h = None
        except Exception:
            pass

    def _append(self, node: _Node) -> int:
        arr = (C.c_int64 * max(1, len(node.inputs)))(*node.inputs)
        nid = self._lib.ftc_tape_add_node(self._h, arr, len(node.inputs), int(node.requires_grad), int(node.op == "leaf"))
        self.nodes.append(node)
        return int(nid)

    def leaf(self, value: float, requires_grad: bool) -> int:
        return self._append(_Node(float(value), bool(requires_grad), "leaf", (), "leaf"))

    def value(self, nid: int) -> float:
        if nid < 0 or nid >= len(self.nodes):
            raise UnknownNode(f"node {nid}")
        return self.nodes[nid].value

    def binary(self, op: str, lhs: int, rhs: int, keyset: Optional[DispatchKeySet] = None) -> Tuple[int, DispatchDecision]:
        a, b = self.value(lhs), self.value(rhs)
        rg = self.nodes[lhs].requires_grad or self.nodes[rhs].requires_grad
        out, decision = dispatch_scalar_binary(op, self.mode, a, b, rg, keyset)
        nid = self._append(_Node(out, rg, op, (lhs, rhs), _BINARY_RULES[op][0]))
        return nid, decision

    def unary(self, op: str, x: int) -> int:
        rule, f, _ = _UNARY_RULES[op]
        v = self.value(x)
        return self._append(_Node(f(v), self.nodes[x].requires_grad, op, (x,), rule))

    def backward(self, root: int, options: Optional[BackwardOptions] = None) -> BackwardReport:
        opts = options or BackwardOptions.for_mode(self.mode)
        guard = fallback = False
        if opts.current_reentrant_depth > opts.max_reentrant_depth:
            if opts.policy == ReentrantPolicy.StrictFail:
                raise ReentrantDepthExceeded(opts.current_reentrant_depth, opts.max_reentrant_depth)
            guard = fallback = True
        n = len(self.nodes)
        order = (C.c_int64 * max(1, n))()
        deps = (C.c_int64 * max(1, n))()
        stats = (C.c_int64 * 3)()
        cnt = self._lib.ftc_tape_schedule(self._h, root, 1, order, deps, stats)
        if cnt == -1:
            raise UnknownNode(f"node {root}")
        if cnt == -2:
            raise RootDoesNotRequireGrad(f"node {root} does not require grad")
        if cnt == -3:
            raise GraphConsumed("graph already consumed; pass retain_graph")
        if cnt < 0:
            raise AutogradError(f"scheduler error {cnt}")
        grads: List[Optional[float]] = [None] * n
        grads[root] = 1.0
        steps: List[BackwardStep] = []
        for k in range(cnt):
            nid = int(order[k])
            node = self.nodes[nid]
            g = grads[nid] if grads[nid] is not None else 0.0
            if node.op == "leaf":
                if node.requires_grad:
                    steps.append(BackwardStep(nid, g, "leaf"))
                continue
            if not node.requires_grad:
                continue
            steps.append(BackwardStep(nid, g, node.rule))
            if len(node.inputs) == 2:
                a, b = self.nodes[node.inputs[0]].value, self.nodes[node.inputs[1]].value
                contrib = _BINARY_RULES[node.op][1](g, a, b)
            else:
                x = self.nodes[node.inputs[0]].value
                contrib = (_UNARY_RULES[node.op][2](g, x, node.value),)
            for inp, c in zip(node.inputs, contrib):
                grads[inp] = c if grads[inp] is None else grads[inp] + c
        out = [grads[i] if self.nodes[i].requires_grad else None for i in range(n)]
        if not opts.retain_graph:
            self._lib.ftc_tape_mark_consumed(self._h)
        tel = TensorSchedulerTelemetry([int(order[k]) for k in range(cnt)], int(stats[0]), int(stats[1]), int(stats[2]),
                                       [int(deps[i]) for i in range(n)],
                                       min(opts.current_reentrant_depth, opts.max_reentrant_depth), guard, fallback)
        return BackwardReport(out, steps, tel)
