"""Operation events: the typed record that every tape-recording operator returns next to its node id
(ft-autograd/src/lib.rs:876-1060: ``OperationEvent``, ``UnaryOperationEvent``, ``TensorOperationEvent``,
``TensorUnaryOperationEvent``, ``TensorReductionOperationEvent`` ... ``TensorTopKOperationEvent``).

An event names the operator (as the family's enum member), the input node(s), the output node, the
family's parameters and the dispatch decision that chose the kernel.  ``record_tensor_op`` runs one
operator of a session and returns ``(node id, event)``; the typed wrappers below it are the tape-level
entry points of the reference (``TensorTape::unary / binary / reduction / ...``).  The session keeps the
last event in ``last_operation_event`` and, while ``operation_events`` is a list, appends to it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from ..core.dtype import DType
from ..dispatch import families as F
from ..dispatch.keys import DispatchDecision

NodeId = int          # index of a node of the scalar tape
TensorNodeId = int    # index of a node of the tensor tape


@dataclass(frozen=True)
class OperationEvent:
    op: F.BinaryOp
    lhs: NodeId
    rhs: NodeId
    out: NodeId
    decision: object


@dataclass(frozen=True)
class UnaryOperationEvent:
    op: F.UnaryOp
    input: NodeId
    out: NodeId
    decision: object


@dataclass(frozen=True)
class PowOperationEvent:
    input: NodeId
    out: NodeId
    exponent: float
    decision: object


@dataclass(frozen=True)
class ClampOperationEvent:
    input: NodeId
    out: NodeId
    min_val: float
    max_val: float
    decision: object


@dataclass(frozen=True)
class TensorOperationEvent:
    op: F.BinaryOp
    lhs: TensorNodeId
    rhs: TensorNodeId
    out: TensorNodeId
    decision: object


@dataclass(frozen=True)
class TensorScalarOperationEvent:
    op: F.BinaryOp
    input: TensorNodeId
    scalar: float
    out: TensorNodeId
    output_dtype: DType


@dataclass(frozen=True)
class TensorUnaryOperationEvent:
    op: F.UnaryOp
    input: TensorNodeId
    out: TensorNodeId
    decision: object


@dataclass(frozen=True)
class TensorReductionOperationEvent:
    op: F.ReductionOp
    input: TensorNodeId
    out: TensorNodeId
    decision: object


@dataclass(frozen=True)
class TensorReductionDimOperationEvent:
    op: F.ReductionOp
    input: TensorNodeId
    out: TensorNodeId
    dim: int
    decision: object


@dataclass(frozen=True)
class TensorScanDimOperationEvent:
    op: F.ScanOp
    input: TensorNodeId
    out: TensorNodeId
    dim: int
    decision: object


@dataclass(frozen=True)
class TensorNormalizeDimOperationEvent:
    op: F.NormalizeOp
    input: TensorNodeId
    out: TensorNodeId
    dim: int
    decision: object


@dataclass(frozen=True)
class TensorJoinOperationEvent:
    op: F.JoinOp
    inputs: Tuple[TensorNodeId, ...]
    out: TensorNodeId
    dim: int
    decision: object


@dataclass(frozen=True)
class TensorPowOperationEvent:
    input: TensorNodeId
    out: TensorNodeId
    exponent: float
    decision: object


@dataclass(frozen=True)
class TensorClampOperationEvent:
    input: TensorNodeId
    out: TensorNodeId
    min_val: float
    max_val: float
    decision: object


@dataclass(frozen=True)
class TensorNormOperationEvent:
    input: TensorNodeId
    out: TensorNodeId
    p: float
    decision: object


@dataclass(frozen=True)
class TensorNormDimOperationEvent:
    input: TensorNodeId
    out: TensorNodeId
    p: float
    dim: int
    decision: object


@dataclass(frozen=True)
class TensorLerpOperationEvent:
    start: TensorNodeId
    end: TensorNodeId
    out: TensorNodeId
    weight: float
    decision: object


@dataclass(frozen=True)
class TensorAddmmOperationEvent:
    input: TensorNodeId
    mat1: TensorNodeId
    mat2: TensorNodeId
    out: TensorNodeId
    beta: float
    alpha: float
    decision: object


@dataclass(frozen=True)
class TensorAddmvOperationEvent:
    input: TensorNodeId
    mat: TensorNodeId
    vec: TensorNodeId
    out: TensorNodeId
    beta: float
    alpha: float
    decision: object


@dataclass(frozen=True)
class TensorSortOperationEvent:
    input: TensorNodeId
    out: TensorNodeId
    dim: int
    descending: bool
    decision: object


@dataclass(frozen=True)
class TensorTopKOperationEvent:
    input: TensorNodeId
    out: TensorNodeId
    k: int
    dim: int
    largest: bool
    sorted: bool
    decision: object


@dataclass(frozen=True)
class TensorGenericOperationEvent:
    """An operator outside the typed families (the long tail of the rule table): name, inputs, parameters."""
    op: str
    inputs: Tuple[TensorNodeId, ...]
    out: TensorNodeId
    params: Tuple[Tuple[str, object], ...]
    decision: object


def _family_decision(cls, op, d: DispatchDecision, **extra):
    return cls(op, d.mode, d.kernel, d.selected_key, d.backend_key, d.keyset_bits, d.fallback_used, **extra)


def event_for(name: str, inputs: Sequence[int], out: int, kw: dict, d: DispatchDecision):
    """The typed event of operator ``name`` (family chosen by the schema base name)."""
    i = tuple(inputs)
    if len(i) == 2 and F.BinaryOp.from_schema_base(name):
        op = F.BinaryOp(name)
        return TensorOperationEvent(op, i[0], i[1], out, _family_decision(F.BinaryDispatchDecision, op, d))
    if len(i) == 1 and F.UnaryOp.from_schema_base(name):
        op = F.UnaryOp(name)
        return TensorUnaryOperationEvent(op, i[0], out, _family_decision(F.UnaryDispatchDecision, op, d))
    if len(i) == 1 and F.ReductionOp.from_schema_base(name):
        op = F.ReductionOp(name)
        return TensorReductionOperationEvent(op, i[0], out, _family_decision(F.ReductionDispatchDecision, op, d))
    if len(i) == 1 and name.endswith("_dim") and F.ReductionOp.from_schema_base(name[:-4]):
        op, dim = F.ReductionOp(name[:-4]), int(kw.get("dim", 0))
        return TensorReductionDimOperationEvent(op, i[0], out, dim, _family_decision(F.ReductionDimDispatchDecision, op, d, dim=dim))
    if F.ScanOp.from_schema_base(name):
        op, dim = F.ScanOp(name), int(kw.get("dim", 0))
        return TensorScanDimOperationEvent(op, i[0], out, dim, _family_decision(F.ScanDimDispatchDecision, op, d, dim=dim))
    if F.NormalizeOp.from_schema_base(name):
        op, dim = F.NormalizeOp(name), int(kw.get("dim", -1))
        return TensorNormalizeDimOperationEvent(op, i[0], out, dim, _family_decision(F.NormalizeDimDispatchDecision, op, d, dim=dim))
    if F.JoinOp.from_schema_base(name):
        op, dim = F.JoinOp(name), int(kw.get("dim", 0))
        return TensorJoinOperationEvent(op, i, out, dim, _family_decision(F.JoinDispatchDecision, op, d, dim=dim, num_inputs=len(i)))
    if name == "pow":
        e = float(kw.get("n", 2.0))
        return TensorPowOperationEvent(i[0], out, e, _family_decision(F.PowDispatchDecision, name, d, exponent=e))
    if name == "clamp":
        lo = float("-inf") if kw.get("min") is None else float(kw["min"])
        hi = float("inf") if kw.get("max") is None else float(kw["max"])
        return TensorClampOperationEvent(i[0], out, lo, hi, _family_decision(F.ClampDispatchDecision, name, d, min_val=lo, max_val=hi))
    if name == "norm":
        p = float(kw.get("p", 2.0))
        return TensorNormOperationEvent(i[0], out, p, _family_decision(F.NormDispatchDecision, name, d, p=p))
    if name == "norm_dim":
        p, dim = float(kw.get("p", 2.0)), int(kw.get("dim", 0))
        return TensorNormDimOperationEvent(i[0], out, p, dim, _family_decision(F.NormDimDispatchDecision, name, d, p=p, dim=dim))
    if name == "lerp":
        w = float(kw.get("w", 0.5))
        return TensorLerpOperationEvent(i[0], i[1], out, w, _family_decision(F.LerpDispatchDecision, name, d, weight=w))
    if name in ("addmm", "addmv"):
        b, a = float(kw.get("beta", 1.0)), float(kw.get("alpha", 1.0))
        cls = TensorAddmmOperationEvent if name == "addmm" else TensorAddmvOperationEvent
        return cls(i[0], i[1], i[2], out, b, a, _family_decision(F.AddmmDispatchDecision, name, d, beta=b, alpha=a))
    if name == "sort":
        dim, desc = int(kw.get("dim", -1)), bool(kw.get("descending", False))
        return TensorSortOperationEvent(i[0], out, dim, desc, _family_decision(F.SortDispatchDecision, name, d, dim=dim, descending=desc))
    if name == "topk":
        k, dim, lg = int(kw.get("k", 1)), int(kw.get("dim", -1)), bool(kw.get("largest", True))
        return TensorTopKOperationEvent(i[0], out, k, dim, lg, True,
                                        _family_decision(F.TopKDispatchDecision, name, d, k=k, dim=dim, largest=lg, sorted=True))
    return TensorGenericOperationEvent(name, i, out, tuple(sorted((k, v if isinstance(v, (int, float, str, bool, type(None))) else repr(v))
                                                                   for k, v in kw.items())), d)


def record_tensor_op(session, name: str, inputs: Sequence[int], **kw):
    """Run operator ``name`` of ``session`` on tape nodes ``inputs``; returns ``(node id, event)``."""
    out = session._apply(name, list(inputs), **kw)
    ev = event_for(name, inputs, out, kw, session.last_decision)
    session.last_operation_event = ev
    if isinstance(getattr(session, "operation_events", None), list):
        session.operation_events.append(ev)
    return out, ev


# ------------------------------------------------------------------------------------ typed tape entry points
def tensor_binary(session, op, lhs: int, rhs: int):
    return record_tensor_op(session, F._enum(F.BinaryOp, op).value, [lhs, rhs])


def tensor_unary(session, op, x: int, **params):
    return record_tensor_op(session, F._enum(F.UnaryOp, op).value, [x], **params)


def tensor_reduction(session, op, x: int):
    op = F._enum(F.ReductionOp, op)
    if op.value in ("prod", "var", "std"):      # built from the dim forms over the flattened tensor
        flat = session.tensor_reshape(x, shape=(-1,))
        out, ev = record_tensor_op(session, op.value + "_dim", [flat], dim=0)
        d = ev.decision
        ev = TensorReductionOperationEvent(op, x, out, F.ReductionDispatchDecision(op, d.mode, d.kernel, d.selected_key, d.backend_key,
                                                                                   d.keyset_bits, d.fallback_used))
        session.last_operation_event = ev
        if isinstance(session.operation_events, list):
            session.operation_events[-1] = ev
        return out, ev
    return record_tensor_op(session, op.value, [x])


def tensor_reduction_dim(session, op, x: int, dim: int):
    return record_tensor_op(session, F._enum(F.ReductionOp, op).value + "_dim", [x], dim=dim)


def tensor_scan_dim(session, op, x: int, dim: int):
    return record_tensor_op(session, F._enum(F.ScanOp, op).value, [x], dim=dim)


def tensor_normalize_dim(session, op, x: int, dim: int):
    return record_tensor_op(session, F._enum(F.NormalizeOp, op).value, [x], dim=dim)


def tensor_join(session, op, xs: Sequence[int], dim: int):
    return record_tensor_op(session, F._enum(F.JoinOp, op).value, list(xs), dim=dim)


def tensor_pow(session, x: int, exponent: float):
    return record_tensor_op(session, "pow", [x], n=float(exponent))


def tensor_clamp(session, x: int, min_val: float, max_val: float):
    return record_tensor_op(session, "clamp", [x], min=min_val, max=max_val)


def tensor_norm(session, x: int, p: float = 2.0):
    return record_tensor_op(session, "norm", [x], p=float(p))


def tensor_norm_dim(session, x: int, p: float, dim: int):
    return record_tensor_op(session, "norm_dim", [x], p=float(p), dim=dim)


def tensor_lerp(session, start: int, end: int, weight: float):
    return record_tensor_op(session, "lerp", [start, end], w=float(weight))


def tensor_addmm(session, x: int, m1: int, m2: int, beta: float = 1.0, alpha: float = 1.0):
    return record_tensor_op(session, "addmm", [x, m1, m2], beta=beta, alpha=alpha)


def tensor_addmv(session, x: int, m: int, v: int, beta: float = 1.0, alpha: float = 1.0):
    return record_tensor_op(session, "addmv", [x, m, v], beta=beta, alpha=alpha)


def tensor_sort(session, x: int, dim: int, descending: bool = False):
    return record_tensor_op(session, "sort", [x], dim=dim, descending=descending)


def tensor_topk(session, x: int, k: int, dim: int, largest: bool = True):
    return record_tensor_op(session, "topk", [x], k=k, dim=dim, largest=largest)


def tensor_scalar(session, op, x: int, scalar: float):
    """Tensor (op) Python scalar: no second node is created; the event carries the scalar and the output dtype."""
    op = F._enum(F.BinaryOp, op)
    name = {"add": "add_scalar", "mul": "mul_scalar"}.get(op.value)
    if name is not None and hasattr(session, "tensor_" + name):
        out = getattr(session, "tensor_" + name)(x, scalar)
    else:
        c = session.full(session.tensor_shape(x), float(scalar), dtype=session.tensor_dtype(x))
        out = session._apply(op.value, [x, c])
    ev = TensorScalarOperationEvent(op, x, float(scalar), out, session.tensor_dtype(out))
    session.last_operation_event = ev
    if isinstance(getattr(session, "operation_events", None), list):
        session.operation_events.append(ev)
    return out, ev


# ------------------------------------------------------------------------------------ scalar tape
def scalar_binary(session, op, lhs: int, rhs: int):
    """Scalar-tape binary operator; returns ``(node id, OperationEvent)``."""
    op = F._enum(F.BinaryOp, op)
    out, d = session.tape.binary(op.value, lhs, rhs)
    ev = OperationEvent(op, lhs, rhs, out, _family_decision(F.BinaryDispatchDecision, op, d))
    session.last_operation_event = ev
    return out, ev
