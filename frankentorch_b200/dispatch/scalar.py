"""Scalar-tensor dispatch entry points: unary, comparison, pow, clamp, binary with an explicit or a
registered key set, and the key-set helpers they share.

Reference: ft-dispatch/src/lib.rs - ``highest_priority_type_id`` :607 and
``highest_priority_backend_type_id`` :618 (the strict-mode selectors), ``schema_dispatch_key_from_tag``
:1257, ``schema_dispatch_keyset_from_tags`` :1270, ``dispatch_keyset_for_tensors`` :1324 (and the
``_tensor_meta`` / ``_single_tensor`` / ``_single_tensor_meta`` forms :1333 / :1804 / :1812),
``dispatch_scalar_binary_with_keyset`` :1395, ``dispatch_scalar_binary_registered`` :1496,
``dispatch_scalar_unary`` :1819, ``dispatch_scalar_comparison`` :3154, ``dispatch_scalar_pow`` :3403,
``dispatch_scalar_clamp`` :3811.

Scalar tensors live on the host (a 0-d f64 value with metadata), so the arithmetic here is plain
``math``; what the functions add is the key resolution, the kernel name of the decision and the
versioned result tensor.  Device tensors go through ``families.py``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, Union

from ..core.meta import Device, TensorMeta
from ..core.storage import ScalarTensor
from ..runtime.ledger import ExecutionMode
from .families import BinaryOp, ComparisonOp, UnaryOp
from .keys import (DispatchDecision, DispatchError, DispatchKey, DispatchKeyError, DispatchKeySet, decide,
                   ensure_meta_compatible, keyset_for)
from .schema import OpSchemaError, SchemaRegistry

# Strict-mode selectors walk these lists front to back.
TYPE_PRIORITY = (DispatchKey.AutogradSM100, DispatchKey.AutogradCPU, DispatchKey.CompositeExplicitAutograd,
                 DispatchKey.CompositeImplicitAutograd, DispatchKey.SM100, DispatchKey.CPU,
                 DispatchKey.BackendSelect)
BACKEND_PRIORITY = (DispatchKey.SM100, DispatchKey.CPU)


def highest_priority_type_id(keyset: DispatchKeySet) -> DispatchKey:
    """The type key a strict resolution selects: the first member of ``TYPE_PRIORITY`` in the set."""
    if keyset.is_empty():
        raise DispatchKeyError("EmptySet", "dispatch keyset is empty")
    for key in TYPE_PRIORITY:
        if keyset.has(key):
            return key
    raise DispatchKeyError("NoTypeKey", "dispatch keyset has no resolvable type key")


def highest_priority_backend_type_id(keyset: DispatchKeySet) -> DispatchKey:
    """The backend key under the selected type key: the first member of ``BACKEND_PRIORITY``."""
    if keyset.is_empty():
        raise DispatchKeyError("EmptySet", "dispatch keyset is empty")
    for key in BACKEND_PRIORITY:
        if keyset.has(key):
            return key
    raise DispatchKeyError("NoBackendKey", "dispatch keyset has no backend key")


DispatchKeySet.highest_priority_type_id = highest_priority_type_id
DispatchKeySet.highest_priority_backend_type_id = highest_priority_backend_type_id

_SCHEMA_TAGS = ("BackendSelect", "CompositeImplicitAutograd", "CompositeExplicitAutograd", "CPU", "AutogradCPU",
                "SM100", "AutogradSM100")


def schema_dispatch_key_from_tag(tag: str) -> DispatchKey:
    """A schema file's dispatch tag as a key; unknown tags are a schema error, not a key error."""
    if tag not in _SCHEMA_TAGS:
        raise OpSchemaError(f"unknown dispatch key {tag!r}")
    return DispatchKey[tag]


def schema_dispatch_keyset_from_tags(tags: Iterable[str]) -> DispatchKeySet:
    """The key set of a schema entry; it must be resolvable for a scalar binary op (a backend key present,
    an autograd key only with its backend)."""
    keyset = DispatchKeySet.empty()
    for tag in tags:
        keyset.add(schema_dispatch_key_from_tag(tag))
    try:
        keyset.validate_for_scalar_binary()
    except DispatchKeyError as e:
        raise OpSchemaError(f"incompatible dispatch keyset: {e}") from e
    return keyset


def _device_of(x: Union[ScalarTensor, TensorMeta]) -> Device:
    meta = x.meta if isinstance(x, ScalarTensor) else x
    return meta.device


def dispatch_keyset_for_tensors(lhs: ScalarTensor, rhs: ScalarTensor, requires_grad: bool) -> DispatchKeySet:
    """The key set of a binary op: the left operand's device decides (operand compatibility is checked
    separately, so both sit on one device by the time a kernel runs)."""
    return keyset_for(_device_of(lhs), requires_grad)


def dispatch_keyset_for_tensor_meta(lhs: TensorMeta, rhs: TensorMeta, requires_grad: bool) -> DispatchKeySet:
    return keyset_for(_device_of(lhs), requires_grad)


def dispatch_keyset_for_single_tensor(input: ScalarTensor, requires_grad: bool) -> DispatchKeySet:
    return keyset_for(_device_of(input), requires_grad)


def dispatch_keyset_for_single_tensor_meta(meta: TensorMeta, requires_grad: bool) -> DispatchKeySet:
    return keyset_for(_device_of(meta), requires_grad)


@dataclass
class ScalarDispatchOutcome:
    """Result tensor (new id, version + 1, the input's metadata) and the decision that produced it."""
    tensor: ScalarTensor
    decision: DispatchDecision


DispatchOutcome = UnaryDispatchOutcome = ComparisonDispatchOutcome = ScalarDispatchOutcome
PowDispatchOutcome = ClampDispatchOutcome = ScalarDispatchOutcome


def _sigmoid(x: float) -> float:
    if x >= 0:
        return 1.0 / (1.0 + math.exp(-x))
    e = math.exp(x)
    return e / (1.0 + e)


def _softplus(x: float) -> float:
    return x if x > 20.0 else math.log1p(math.exp(x))


def _safe(f: Callable[[float], float], domain_nan: bool = True) -> Callable[[float], float]:
    """IEEE behaviour where ``math`` raises: a domain error gives NaN, an overflow gives +inf."""
    def g(x: float) -> float:
        try:
            return f(x)
        except ValueError:
            return math.nan
        except OverflowError:
            return math.inf
        except ZeroDivisionError:
            return math.copysign(math.inf, x) if x == 0 else math.nan
    return g


def _log(x: float) -> float:
    if x == 0.0:
        return -math.inf
    return math.log(x)


def _round_half_even(x: float) -> float:
    return x if not math.isfinite(x) else float(round(x))


_UNARY: Dict[UnaryOp, Callable[[float], float]] = {
    UnaryOp.Neg: lambda x: -x,
    UnaryOp.Abs: abs,
    UnaryOp.Exp: _safe(math.exp),
    UnaryOp.Log: _safe(_log),
    UnaryOp.Relu: lambda x: x if (x > 0.0 or x != x) else 0.0,
    UnaryOp.Sigmoid: _safe(_sigmoid),
    UnaryOp.Tanh: math.tanh,
    UnaryOp.Sqrt: _safe(math.sqrt),
    UnaryOp.Reciprocal: _safe(lambda x: 1.0 / x),
    UnaryOp.Sin: _safe(math.sin),
    UnaryOp.Cos: _safe(math.cos),
    UnaryOp.Tan: _safe(math.tan),
    UnaryOp.Floor: lambda x: float(math.floor(x)) if math.isfinite(x) else x,
    UnaryOp.Ceil: lambda x: float(math.ceil(x)) if math.isfinite(x) else x,
    UnaryOp.Round: _round_half_even,
    UnaryOp.Log2: _safe(lambda x: -math.inf if x == 0.0 else math.log2(x)),
    UnaryOp.Log10: _safe(lambda x: -math.inf if x == 0.0 else math.log10(x)),
    UnaryOp.Log1p: _safe(lambda x: -math.inf if x == -1.0 else math.log1p(x)),
    UnaryOp.Expm1: _safe(math.expm1),
    UnaryOp.Sign: lambda x: x if x != x else float((x > 0) - (x < 0)),
    UnaryOp.Trunc: lambda x: float(math.trunc(x)) if math.isfinite(x) else x,
    UnaryOp.Frac: lambda x: x - math.trunc(x) if math.isfinite(x) else math.nan,
    UnaryOp.Asin: _safe(math.asin),
    UnaryOp.Acos: _safe(math.acos),
    UnaryOp.Atan: math.atan,
    UnaryOp.Sinh: _safe(lambda x: math.sinh(x)),
    UnaryOp.Cosh: _safe(math.cosh),
    UnaryOp.Gelu: lambda x: 0.5 * x * (1.0 + math.erf(x / math.sqrt(2.0))),
    UnaryOp.Silu: _safe(lambda x: x * _sigmoid(x)),
    UnaryOp.LeakyRelu: lambda x: x if x >= 0.0 or x != x else 0.01 * x,
    UnaryOp.Elu: _safe(lambda x: x if x > 0.0 or x != x else math.expm1(x)),
    UnaryOp.Rsqrt: _safe(lambda x: math.inf if x == 0.0 else 1.0 / math.sqrt(x)),
    UnaryOp.Erf: math.erf,
    UnaryOp.Erfc: math.erfc,
    UnaryOp.Hardswish: lambda x: x * min(max(x + 3.0, 0.0), 6.0) / 6.0,
    UnaryOp.Hardsigmoid: lambda x: x if x != x else min(max(x + 3.0, 0.0), 6.0) / 6.0,
    UnaryOp.Hardtanh: lambda x: x if x != x else min(max(x, -1.0), 1.0),
    UnaryOp.Softplus: _safe(_softplus),
    UnaryOp.Mish: _safe(lambda x: x * math.tanh(_softplus(x))),
    UnaryOp.Square: _safe(lambda x: x * x),
    UnaryOp.IsNan: lambda x: float(x != x),
    UnaryOp.IsInf: lambda x: float(math.isinf(x)),
    UnaryOp.IsFinite: lambda x: float(math.isfinite(x)),
}

_COMPARE: Dict[ComparisonOp, Callable[[float, float], bool]] = {
    ComparisonOp.Eq: lambda a, b: a == b, ComparisonOp.Ne: lambda a, b: a != b,
    ComparisonOp.Lt: lambda a, b: a < b, ComparisonOp.Gt: lambda a, b: a > b,
    ComparisonOp.Le: lambda a, b: a <= b, ComparisonOp.Ge: lambda a, b: a >= b,
}


def _div(a: float, b: float) -> float:
    if b == 0.0:
        if a == 0.0 or a != a:
            return math.nan
        return math.copysign(math.inf, a) * math.copysign(1.0, b)
    return a / b


def _nan_min(a: float, b: float) -> float:
    return math.nan if (a != a or b != b) else min(a, b)


def _nan_max(a: float, b: float) -> float:
    return math.nan if (a != a or b != b) else max(a, b)


def _pow(x: float, e: float) -> float:
    try:
        return math.pow(x, e)
    except ValueError:
        return math.nan                      # negative base, fractional exponent
    except OverflowError:
        return -math.inf if (x < 0 and float(e).is_integer() and int(e) % 2 == 1) else math.inf
    except ZeroDivisionError:
        return math.inf


_BINARY: Dict[BinaryOp, Callable[[float, float], float]] = {}
for _name, _fn in (("Add", lambda a, b: a + b), ("Sub", lambda a, b: a - b), ("Mul", lambda a, b: a * b),
                   ("Div", _div), ("Min", _nan_min), ("Max", _nan_max), ("Pow", _pow),
                   ("Atan2", math.atan2), ("Fmod", lambda a, b: math.fmod(a, b) if b != 0.0 else math.nan),
                   ("Remainder", lambda a, b: a - b * math.floor(a / b) if b != 0.0 else math.nan)):
    if hasattr(BinaryOp, _name):
        _BINARY[getattr(BinaryOp, _name)] = _fn
_TENSOR_ONLY = tuple(getattr(BinaryOp, n) for n in ("MatMul", "Dot", "Outer", "Bmm") if hasattr(BinaryOp, n))


def _coerce(enum_cls, op):
    return op if isinstance(op, enum_cls) else enum_cls(op)


def _decide_host(op_name: str, mode: ExecutionMode, keyset: DispatchKeySet) -> DispatchDecision:
    """Resolve the set; a scalar tensor lives on the host, so the backend must be the CPU one."""
    decision = decide(op_name, mode, keyset, f"{op_name}_scalar")
    if decision.backend_key is not DispatchKey.CPU:
        raise DispatchKeyError("IncompatibleSet", "resolved dispatch keys are incompatible with scalar ops")
    return decision


def dispatch_scalar_unary(op: Union[UnaryOp, str], mode: ExecutionMode, input: ScalarTensor,
                          requires_grad: bool = False) -> ScalarDispatchOutcome:
    op = _coerce(UnaryOp, op)
    decision = _decide_host(op.value, mode, dispatch_keyset_for_single_tensor(input, requires_grad))
    return ScalarDispatchOutcome(input.with_value(_UNARY[op](input.value)), decision)


def dispatch_scalar_comparison(op: Union[ComparisonOp, str], mode: ExecutionMode, lhs: ScalarTensor,
                               rhs: ScalarTensor, requires_grad: bool = False) -> ScalarDispatchOutcome:
    """Comparison of two scalar tensors; the result holds 1.0 or 0.0 (any comparison with NaN is false,
    ``ne`` true)."""
    op = _coerce(ComparisonOp, op)
    ensure_meta_compatible(lhs.meta.dtype, rhs.meta.dtype, lhs.meta.device, rhs.meta.device)
    decision = _decide_host(op.value, mode, dispatch_keyset_for_tensors(lhs, rhs, requires_grad))
    return ScalarDispatchOutcome(lhs.with_value(float(_COMPARE[op](lhs.value, rhs.value))), decision)


def dispatch_scalar_pow(mode: ExecutionMode, input: ScalarTensor, exponent: float,
                        requires_grad: bool = False) -> ScalarDispatchOutcome:
    decision = _decide_host("pow", mode, dispatch_keyset_for_single_tensor(input, requires_grad))
    return ScalarDispatchOutcome(input.with_value(_pow(input.value, float(exponent))), decision)


def dispatch_scalar_clamp(mode: ExecutionMode, input: ScalarTensor, min_val: float, max_val: float,
                          requires_grad: bool = False) -> ScalarDispatchOutcome:
    """``min(max(x, lo), hi)``; NaN input stays NaN, and ``lo > hi`` gives ``hi`` as in torch."""
    decision = _decide_host("clamp", mode, dispatch_keyset_for_single_tensor(input, requires_grad))
    x = input.value
    y = x if x != x else min(max(x, float(min_val)), float(max_val))
    return ScalarDispatchOutcome(input.with_value(y), decision)


def dispatch_scalar_binary_with_keyset(op: Union[BinaryOp, str], mode: ExecutionMode, lhs: ScalarTensor,
                                       rhs: ScalarTensor, keyset: DispatchKeySet) -> ScalarDispatchOutcome:
    """Binary op on two scalar tensors under an explicit key set (a schema entry's, or a test's)."""
    op = _coerce(BinaryOp, op)
    ensure_meta_compatible(lhs.meta.dtype, rhs.meta.dtype, lhs.meta.device, rhs.meta.device)
    if op in _TENSOR_ONLY:
        raise DispatchKeyError("IncompatibleSet", f"{op.value} is unsupported for scalar tensors")
    if op not in _BINARY:
        raise DispatchError(f"no scalar kernel for binary op {op.value!r}")
    decision = _decide_host(op.value, mode, keyset)
    return ScalarDispatchOutcome(lhs.with_value(_BINARY[op](lhs.value, rhs.value)), decision)


def dispatch_scalar_binary_tensors(op: Union[BinaryOp, str], mode: ExecutionMode, lhs: ScalarTensor,
                                   rhs: ScalarTensor, requires_grad: bool = False) -> ScalarDispatchOutcome:
    """The same with the key set derived from the operands."""
    return dispatch_scalar_binary_with_keyset(op, mode, lhs, rhs,
                                              dispatch_keyset_for_tensors(lhs, rhs, requires_grad))


def dispatch_scalar_binary_registered(registry: SchemaRegistry, normalized_name: str, mode: ExecutionMode,
                                      lhs: ScalarTensor, rhs: ScalarTensor) -> ScalarDispatchOutcome:
    """Look the op and its key set up in a schema registry, then dispatch.  A missing entry raises the
    registry's error, a bad key set the dispatcher's."""
    entry = registry.lookup(normalized_name)
    return dispatch_scalar_binary_with_keyset(entry.op, mode, lhs, rhs, entry.keyset)
