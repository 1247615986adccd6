"""Typed dispatch entry points per operator family (ft-dispatch/src/lib.rs:253-490 for the operator
enums, :680-800 and :2830-3990 for the decision / outcome records, :1507-6776 for the
``dispatch_tensor_<family>_contiguous_*`` functions).

An entry point takes the operator as an enum member, the execution mode, the operand values (a
``torch.Tensor`` on either device, or a flat list with a :class:`TensorMeta`) and ``requires_grad``; it
resolves the dispatch key set of the operand's device, runs the kernel and returns an *outcome*: the
result plus a *decision* record that names the kernel, the selected and backend keys, the key-set bits
and whether a fallback path ran, extended with the family's parameters (``dim``, ``exponent``,
``p``, ``k`` ...).

Execution goes through the same operator entry point as ``FrankenTorchSession`` (one cached session per
mode and device, its graph truncated after every call), so the CPU path is the f64 / f32 reference
arithmetic and the CUDA path is the sm_100a route table with its strict / hardened rules: a strict-mode
call without a kernel raises, a hardened-mode call records ``fallback_path=true``.  On the CPU the kernel
string follows the reference's naming, ``<namespace>::<op>_tensor_contiguous_<dtype>``; on the GPU it is the
name of the kernel that was launched.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..core.dtype import DType
from ..core.meta import Device, TensorMeta
from ..runtime.ledger import ExecutionMode
from .keys import DispatchDecision, DispatchError, DispatchKey, DispatchKeyError, DispatchKeySet, ensure_meta_compatible


class _SchemaEnum(enum.Enum):
    """Operator enum whose values are the schema base names (``aten::<base>``)."""

    @classmethod
    def from_schema_base(cls, base: str):
        try:
            return cls(base)
        except ValueError:
            return None

    @property
    def schema_base(self) -> str:
        return self.value


class BinaryOp(_SchemaEnum):
    Add = "add"; Sub = "sub"; Div = "div"; Mul = "mul"; MatMul = "matmul"; Min = "min"; Max = "max"      # noqa: E702
    Dot = "dot"; Outer = "outer"; Bmm = "bmm"; Atan2 = "atan2"; Fmod = "fmod"; Remainder = "remainder"   # noqa: E702


class UnaryOp(_SchemaEnum):
    Neg = "neg"; Abs = "abs"; Exp = "exp"; Log = "log"; Relu = "relu"; Sigmoid = "sigmoid"; Tanh = "tanh"   # noqa: E702
    Sqrt = "sqrt"; Reciprocal = "reciprocal"; Sin = "sin"; Cos = "cos"; Tan = "tan"; Floor = "floor"         # noqa: E702
    Ceil = "ceil"; Round = "round"; Log2 = "log2"; Log10 = "log10"; Log1p = "log1p"; Expm1 = "expm1"         # noqa: E702
    Sign = "sign"; Trunc = "trunc"; Frac = "frac"; Asin = "asin"; Acos = "acos"; Atan = "atan"               # noqa: E702
    Sinh = "sinh"; Cosh = "cosh"; Gelu = "gelu"; Silu = "silu"; LeakyRelu = "leaky_relu"; Elu = "elu"        # noqa: E702
    Rsqrt = "rsqrt"; Erf = "erf"; Erfc = "erfc"; Hardswish = "hardswish"; Hardsigmoid = "hardsigmoid"        # noqa: E702
    Hardtanh = "hardtanh"; Softplus = "softplus"; Mish = "mish"; Square = "square"                           # noqa: E702
    IsNan = "isnan"; IsInf = "isinf"; IsFinite = "isfinite"                                                  # noqa: E702


class ReductionOp(_SchemaEnum):
    Sum = "sum"; Mean = "mean"; Prod = "prod"; Var = "var"; Std = "std"; Trace = "trace"   # noqa: E702


class ScanOp(_SchemaEnum):
    CumSum = "cumsum"; CumProd = "cumprod"   # noqa: E702


class NormalizeOp(_SchemaEnum):
    Softmax = "softmax"; LogSoftmax = "log_softmax"   # noqa: E702


class JoinOp(_SchemaEnum):
    Cat = "cat"; Stack = "stack"   # noqa: E702


class ComparisonOp(_SchemaEnum):
    Eq = "eq"; Ne = "ne"; Lt = "lt"; Gt = "gt"; Le = "le"; Ge = "ge"   # noqa: E702


# ------------------------------------------------------------------------------------ decisions
@dataclass(frozen=True)
class FamilyDecision:
    """Fields every family's decision record shares (``op`` is the family's enum member, or the
    operator name for the single-operator families)."""
    op: object
    mode: ExecutionMode
    kernel: str
    selected_key: DispatchKey
    backend_key: DispatchKey
    keyset_bits: int
    fallback_used: bool

    def summary(self) -> str:
        name = self.op.schema_base if isinstance(self.op, _SchemaEnum) else str(self.op)
        extra = "".join(f" {k}={getattr(self, k)}" for k in self.__dataclass_fields__
                        if k not in FamilyDecision.__dataclass_fields__)
        return (f"op={name} mode={self.mode.value} kernel={self.kernel} dispatch_key={self.selected_key.name} "
                f"backend_key={self.backend_key.name} keyset_bits=0x{self.keyset_bits:x} "
                f"fallback_path={str(self.fallback_used).lower()}{extra}")


@dataclass(frozen=True)
class BinaryDispatchDecision(FamilyDecision):
    pass


@dataclass(frozen=True)
class UnaryDispatchDecision(FamilyDecision):
    pass


@dataclass(frozen=True)
class ReductionDispatchDecision(FamilyDecision):
    pass


@dataclass(frozen=True)
class ComparisonDispatchDecision(FamilyDecision):
    pass


@dataclass(frozen=True)
class ReductionDimDispatchDecision(FamilyDecision):
    dim: int = 0


@dataclass(frozen=True)
class ScanDimDispatchDecision(FamilyDecision):
    dim: int = 0


@dataclass(frozen=True)
class NormalizeDimDispatchDecision(FamilyDecision):
    dim: int = 0


@dataclass(frozen=True)
class JoinDispatchDecision(FamilyDecision):
    dim: int = 0
    num_inputs: int = 0


@dataclass(frozen=True)
class PowDispatchDecision(FamilyDecision):
    exponent: float = 1.0


@dataclass(frozen=True)
class NormDispatchDecision(FamilyDecision):
    p: float = 2.0


@dataclass(frozen=True)
class NormDimDispatchDecision(FamilyDecision):
    p: float = 2.0
    dim: int = 0


@dataclass(frozen=True)
class LerpDispatchDecision(FamilyDecision):
    weight: float = 0.5


@dataclass(frozen=True)
class AddmmDispatchDecision(FamilyDecision):
    beta: float = 1.0
    alpha: float = 1.0


@dataclass(frozen=True)
class ClampDispatchDecision(FamilyDecision):
    min_val: float = float("-inf")
    max_val: float = float("inf")


@dataclass(frozen=True)
class SortDispatchDecision(FamilyDecision):
    dim: int = 0
    descending: bool = False


@dataclass(frozen=True)
class TopKDispatchDecision(FamilyDecision):
    k: int = 1
    dim: int = 0
    largest: bool = True
    sorted: bool = True


# ------------------------------------------------------------------------------------ outcomes
@dataclass
class TensorOutcome:
    """Result values (a tensor of the operand dtype on the operand's device) plus the decision.
    ``storage`` is the typed-storage view of the same result (``TypedUnaryOutcome`` ... of the reference)."""
    values: torch.Tensor
    decision: FamilyDecision

    @property
    def storage(self):
        from ..core.storage import TensorStorage
        return TensorStorage.from_tensor(self.values)

    def tolist(self) -> List[float]:
        return self.values.detach().reshape(-1).to("cpu", torch.float64).tolist()


@dataclass
class ScalarOutcome:
    """A full reduction: one value plus the decision."""
    value: float
    decision: FamilyDecision


@dataclass
class IndexedOutcome(TensorOutcome):
    """Sort / top-k: values and the positions they came from."""
    indices: torch.Tensor = field(default_factory=lambda: torch.empty(0, dtype=torch.long))


# reference names of the outcome records, by family
TensorDispatchOutcome = TensorUnaryDispatchOutcome = TensorComparisonDispatchOutcome = TensorOutcome
TensorReductionDimDispatchOutcome = TensorScanDimDispatchOutcome = TensorNormalizeDimDispatchOutcome = TensorOutcome
TensorJoinDispatchOutcome = TensorPowDispatchOutcome = TensorNormDimDispatchOutcome = TensorLerpDispatchOutcome = TensorOutcome
TensorAddmmDispatchOutcome = TensorAddmvDispatchOutcome = TensorClampDispatchOutcome = TensorOutcome
TensorReductionDispatchOutcome = TensorNormDispatchOutcome = ScalarOutcome
TensorSortDispatchOutcome = TensorTopKDispatchOutcome = IndexedOutcome
TypedUnaryOutcome = TypedBinaryOutcome = TypedReductionDimOutcome = TypedPowOutcome = TypedClampOutcome = TensorOutcome
TypedNormDimOutcome = TypedScanDimOutcome = TypedNormalizeDimOutcome = TypedJoinOutcome = TypedLerpOutcome = TensorOutcome
TypedAddmmOutcome = TypedAddmvOutcome = TensorOutcome
TypedReductionOutcome = TypedNormOutcome = ScalarOutcome
TypedSortOutcome = TypedTopKOutcome = IndexedOutcome

Operand = Union[torch.Tensor, Tuple[Sequence[float], TensorMeta]]


# ------------------------------------------------------------------------------------ execution
_SESSIONS: Dict[Tuple[str, str], object] = {}
_TORCH_DT = {DType.F64: torch.float64, DType.F32: torch.float32, DType.F16: torch.float16, DType.BF16: torch.bfloat16}
_DT_TAG = {torch.float64: "f64", torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}


def _session(mode: ExecutionMode, device: torch.device):
    from ..session import FrankenTorchSession
    key = (ExecutionMode.parse(mode).value, str(device))
    s = _SESSIONS.get(key)
    if s is None:
        s = _SESSIONS[key] = FrankenTorchSession(mode=mode, device=str(device), ledger_dispatch=False)
    return s


def _as_tensor(x: Operand) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x
    values, meta = x
    dev = "cuda" if meta.device == Device.Cuda else "cpu"
    t = torch.as_tensor(list(values), dtype=_TORCH_DT[meta.dtype], device=dev)
    if t.numel() != meta.numel:
        raise DispatchError(f"{t.numel()} values for a tensor of shape {list(meta.shape)}")
    return t.reshape(tuple(meta.shape))


def _check_compatible(ts: Sequence[torch.Tensor]) -> None:
    first = ts[0]
    for t in ts[1:]:
        ensure_meta_compatible(DType.from_torch(first.dtype), DType.from_torch(t.dtype),
                               Device.Cuda if first.is_cuda else Device.Cpu, Device.Cuda if t.is_cuda else Device.Cpu)


def _run(name: str, mode: ExecutionMode, operands: Sequence[Operand], requires_grad: bool, **kw):
    """Run session operator ``name`` on fresh leaves; returns ``(result tensor, session decision, dtype tag)``."""
    ts = [_as_tensor(o) for o in operands]
    if not ts:
        raise DispatchKeyError("IncompatibleSet", f"{name} needs at least one input")
    _check_compatible(ts)
    s = _session(mode, ts[0].device)
    tape = s.tensor_tape
    mark = len(tape)
    try:
        ids = [tape.leaf(t, requires_grad) for t in ts]
        if name in _SESSION_FORMS:
            out = _SESSION_FORMS[name](s, ids, kw)
            # these session methods are built from other rules or run outside the rule table: the decision is theirs
            rg = requires_grad and name in ("prod", "var", "std")
            decision = s._record_dispatch(name, rg, launched=f"torch::{name}" if s.is_cuda and not rg else None)
        else:
            out = s._apply(name, ids, **kw)
            decision = s.last_decision
        val = tape.value(out).detach()
    finally:
        tape.truncate_graph_to(mark)
    return val, decision, _DT_TAG.get(ts[0].dtype, str(ts[0].dtype).replace("torch.", ""))


# operators that the session builds from other rules (their decision is that of the last rule they ran)
_SESSION_FORMS = {
    "eq": lambda s, i, kw: s.tensor_eq(*i), "ne": lambda s, i, kw: s.tensor_ne(*i), "lt": lambda s, i, kw: s.tensor_lt(*i),
    "gt": lambda s, i, kw: s.tensor_gt(*i), "le": lambda s, i, kw: s.tensor_le(*i), "ge": lambda s, i, kw: s.tensor_ge(*i),
    "isnan": lambda s, i, kw: s.tensor_isnan(*i), "isfinite": lambda s, i, kw: s.tensor_isfinite(*i),
    "prod": lambda s, i, kw: s.tensor_prod(*i), "var": lambda s, i, kw: s.tensor_var(*i), "std": lambda s, i, kw: s.tensor_std(*i),
}


def _kernel(decision: DispatchDecision, suffix: str, tag: str) -> str:
    if decision.backend_key is DispatchKey.CPU:
        ns = decision.kernel.split("::", 1)[0]
        return f"{ns}::{suffix}_{tag}"
    return decision.kernel


def _decide(cls, op, d: DispatchDecision, suffix: str, tag: str, **extra):
    return cls(op, d.mode, _kernel(d, suffix, tag), d.selected_key, d.backend_key, d.keyset_bits, d.fallback_used, **extra)


def _dim(t: torch.Tensor, dim: int) -> int:
    if not -t.dim() <= dim < max(t.dim(), 1):
        raise DispatchError(f"dim {dim} out of range for a tensor of rank {t.dim()}")
    return dim % max(t.dim(), 1)


def _enum(cls, op):
    if isinstance(op, cls):
        return op
    member = cls.from_schema_base(str(op))
    if member is None:
        raise DispatchError(f"unknown {cls.__name__} {op!r}")
    return member


# ------------------------------------------------------------------------------------ entry points
def dispatch_tensor_binary(op, mode: ExecutionMode, lhs: Operand, rhs: Operand, requires_grad: bool = False) -> TensorOutcome:
    op = _enum(BinaryOp, op)
    val, d, tag = _run(op.value, mode, [lhs, rhs], requires_grad)
    return TensorOutcome(val, _decide(BinaryDispatchDecision, op, d, f"{op.value}_tensor_contiguous", tag))


_UNARY_PARAMS = {UnaryOp.LeakyRelu: {"negative_slope": 0.01}, UnaryOp.Elu: {"alpha": 1.0}}


def dispatch_tensor_unary(op, mode: ExecutionMode, input: Operand, requires_grad: bool = False, **params) -> TensorOutcome:
    op = _enum(UnaryOp, op)
    val, d, tag = _run(op.value, mode, [input], requires_grad, **params)
    if op in (UnaryOp.IsNan, UnaryOp.IsInf, UnaryOp.IsFinite):
        val = val.to(_as_tensor(input).dtype)       # predicates answer 0.0 / 1.0 in the operand dtype
    return TensorOutcome(val, _decide(UnaryDispatchDecision, op, d, f"{op.value}_tensor_contiguous", tag))


def dispatch_tensor_comparison(op, mode: ExecutionMode, lhs: Operand, rhs: Operand, requires_grad: bool = False) -> TensorOutcome:
    op = _enum(ComparisonOp, op)
    val, d, tag = _run(op.value, mode, [lhs, rhs], False)
    val = val.to(_as_tensor(lhs).dtype)
    return TensorOutcome(val, _decide(ComparisonDispatchDecision, op, d, f"{op.value}_tensor_contiguous", tag))


def dispatch_tensor_reduction(op, mode: ExecutionMode, input: Operand, requires_grad: bool = False) -> ScalarOutcome:
    op = _enum(ReductionOp, op)
    val, d, tag = _run(op.value, mode, [input], requires_grad)
    return ScalarOutcome(float(val), _decide(ReductionDispatchDecision, op, d, f"{op.value}_tensor_contiguous", tag))


def dispatch_tensor_reduction_dim(op, mode: ExecutionMode, input: Operand, dim: int, requires_grad: bool = False) -> TensorOutcome:
    op = _enum(ReductionOp, op)
    if op is ReductionOp.Trace:
        raise DispatchError("trace has no dim form")
    dim = _dim(_as_tensor(input), dim)
    val, d, tag = _run(op.value + "_dim", mode, [input], requires_grad, dim=dim)
    return TensorOutcome(val, _decide(ReductionDimDispatchDecision, op, d, f"{op.value}_dim_tensor_contiguous", tag, dim=dim))


def dispatch_tensor_scan_dim(op, mode: ExecutionMode, input: Operand, dim: int, requires_grad: bool = False) -> TensorOutcome:
    op = _enum(ScanOp, op)
    dim = _dim(_as_tensor(input), dim)
    val, d, tag = _run(op.value, mode, [input], requires_grad, dim=dim)
    return TensorOutcome(val, _decide(ScanDimDispatchDecision, op, d, f"{op.value}_tensor_contiguous", tag, dim=dim))


def dispatch_tensor_normalize_dim(op, mode: ExecutionMode, input: Operand, dim: int, requires_grad: bool = False) -> TensorOutcome:
    op = _enum(NormalizeOp, op)
    dim = _dim(_as_tensor(input), dim)
    val, d, tag = _run(op.value, mode, [input], requires_grad, dim=dim)
    return TensorOutcome(val, _decide(NormalizeDimDispatchDecision, op, d, f"{op.value}_dim_tensor_contiguous", tag, dim=dim))


def dispatch_tensor_join(op, mode: ExecutionMode, inputs: Sequence[Operand], dim: int, requires_grad: bool = False) -> TensorOutcome:
    op = _enum(JoinOp, op)
    if not inputs:
        raise DispatchKeyError("IncompatibleSet", "join op requires at least one input")
    val, d, tag = _run(op.value, mode, list(inputs), requires_grad, dim=dim)
    return TensorOutcome(val, _decide(JoinDispatchDecision, op, d, f"{op.value}_tensor_contiguous", tag, dim=dim, num_inputs=len(inputs)))


def dispatch_tensor_pow(mode: ExecutionMode, input: Operand, exponent: float, requires_grad: bool = False) -> TensorOutcome:
    val, d, tag = _run("pow", mode, [input], requires_grad, n=float(exponent))
    return TensorOutcome(val, _decide(PowDispatchDecision, "pow", d, "pow_tensor_contiguous", tag, exponent=float(exponent)))


def dispatch_tensor_clamp(mode: ExecutionMode, input: Operand, min_val: float, max_val: float, requires_grad: bool = False) -> TensorOutcome:
    val, d, tag = _run("clamp", mode, [input], requires_grad, min=min_val, max=max_val)
    return TensorOutcome(val, _decide(ClampDispatchDecision, "clamp", d, "clamp_tensor_contiguous", tag, min_val=float(min_val), max_val=float(max_val)))


def dispatch_tensor_norm(mode: ExecutionMode, input: Operand, p: float, requires_grad: bool = False) -> ScalarOutcome:
    val, d, tag = _run("norm", mode, [input], requires_grad, p=float(p))
    return ScalarOutcome(float(val), _decide(NormDispatchDecision, "norm", d, "norm_tensor_contiguous", tag, p=float(p)))


def dispatch_tensor_norm_dim(mode: ExecutionMode, input: Operand, p: float, dim: int, requires_grad: bool = False) -> TensorOutcome:
    dim = _dim(_as_tensor(input), dim)
    val, d, tag = _run("norm_dim", mode, [input], requires_grad, p=float(p), dim=dim)
    return TensorOutcome(val, _decide(NormDimDispatchDecision, "norm_dim", d, "norm_dim_tensor_contiguous", tag, p=float(p), dim=dim))


def dispatch_tensor_lerp(mode: ExecutionMode, start: Operand, end: Operand, weight: float, requires_grad: bool = False) -> TensorOutcome:
    val, d, tag = _run("lerp", mode, [start, end], requires_grad, w=float(weight))
    return TensorOutcome(val, _decide(LerpDispatchDecision, "lerp", d, "lerp_tensor_contiguous", tag, weight=float(weight)))


def dispatch_tensor_addmm(mode: ExecutionMode, input: Operand, mat1: Operand, mat2: Operand, beta: float = 1.0,
                          alpha: float = 1.0, requires_grad: bool = False) -> TensorOutcome:
    val, d, tag = _run("addmm", mode, [input, mat1, mat2], requires_grad, beta=float(beta), alpha=float(alpha))
    return TensorOutcome(val, _decide(AddmmDispatchDecision, "addmm", d, "addmm_tensor_contiguous", tag, beta=float(beta), alpha=float(alpha)))


def dispatch_tensor_addmv(mode: ExecutionMode, input: Operand, mat: Operand, vec: Operand, beta: float = 1.0,
                          alpha: float = 1.0, requires_grad: bool = False) -> TensorOutcome:
    val, d, tag = _run("addmv", mode, [input, mat, vec], requires_grad, beta=float(beta), alpha=float(alpha))
    return TensorOutcome(val, _decide(AddmmDispatchDecision, "addmv", d, "addmv_tensor_contiguous", tag, beta=float(beta), alpha=float(alpha)))


def dispatch_tensor_sort(mode: ExecutionMode, input: Operand, dim: int, descending: bool = False, requires_grad: bool = False) -> IndexedOutcome:
    t = _as_tensor(input)
    dim = _dim(t, dim)
    val, d, tag = _run("sort", mode, [input], requires_grad, dim=dim, descending=bool(descending))
    idx = torch.argsort(t, dim=dim, descending=bool(descending), stable=True)
    return IndexedOutcome(val, _decide(SortDispatchDecision, "sort", d, "sort_tensor_contiguous", tag, dim=dim, descending=bool(descending)), idx)


def dispatch_tensor_topk(mode: ExecutionMode, input: Operand, k: int, dim: int, largest: bool = True, sorted: bool = True,
                         requires_grad: bool = False) -> IndexedOutcome:
    t = _as_tensor(input)
    dim = _dim(t, dim)
    if not 0 <= k <= t.shape[dim]:
        raise DispatchError(f"k={k} out of range for extent {t.shape[dim]}")
    val, d, tag = _run("topk", mode, [input], requires_grad, k=int(k), dim=dim, largest=bool(largest))
    idx = torch.topk(t, int(k), dim=dim, largest=bool(largest), sorted=True).indices
    return IndexedOutcome(val, _decide(TopKDispatchDecision, "topk", d, "topk_tensor_contiguous", tag, k=int(k), dim=dim,
                                       largest=bool(largest), sorted=bool(sorted)), idx)


# the reference's per-dtype spellings of the same entry points
for _fam in ("binary", "unary", "comparison", "reduction", "reduction_dim", "scan_dim", "normalize_dim", "join", "pow", "clamp",
             "norm", "norm_dim", "lerp", "addmm", "addmv", "sort", "topk"):
    for _suffix in ("f64", "f32", "typed"):
        globals()[f"dispatch_tensor_{_fam}_contiguous_{_suffix}"] = globals()[f"dispatch_tensor_{_fam}"]


def dispatch_tensor_binary_contiguous_f64_with_keyset(op, mode: ExecutionMode, lhs: Operand, rhs: Operand,
                                                      keyset: DispatchKeySet) -> TensorOutcome:
    """Binary family under an explicit key set (ft-dispatch/src/lib.rs:1523): the set is resolved first, so an
    empty set, a set without a backend key or, in strict mode, a composite-only set is refused with the typed
    key error before any kernel runs.  The decision carries the resolution of the given set; whether the result
    is recorded for autograd follows from the effective key."""
    from dataclasses import replace
    from .keys import resolve
    selected, backend, effective, fallback = resolve(mode, keyset)
    autograd = effective in (DispatchKey.AutogradCPU, DispatchKey.AutogradSM100)
    t = _as_tensor(lhs)
    on_device = backend is DispatchKey.SM100
    if on_device != t.is_cuda:
        raise DispatchKeyError("IncompatibleSet", f"backend key {backend.name} does not match operands on {t.device.type}")
    out = dispatch_tensor_binary(op, mode, lhs, rhs, autograd)
    d = out.decision
    ns = {DispatchKey.AutogradCPU: "autograd_cpu", DispatchKey.CPU: "cpu", DispatchKey.AutogradSM100: "autograd_sm100",
          DispatchKey.SM100: "sm100"}[effective]
    kernel = d.kernel if "::" not in d.kernel or d.kernel.startswith(("ftk::", "torch::")) else ns + "::" + d.kernel.split("::", 1)[1]
    return TensorOutcome(out.values, replace(d, kernel=kernel, selected_key=selected, backend_key=backend,
                                             keyset_bits=keyset.bits, fallback_used=fallback or d.fallback_used))


def _f32_only(fn, name):
    def native(mode: ExecutionMode, input: Operand, *args, **kw):
        if _as_tensor(input).dtype != torch.float32:
            raise DispatchError(f"{name}: the native f32 entry point takes float32 operands, got {_as_tensor(input).dtype}")
        return fn(mode, input, *args, **kw)
    native.__name__ = name
    native.__doc__ = (f"``{fn.__name__}`` for float32 operands only: no widening to f64 and back on the way "
                      "(ft-dispatch's ``*_contiguous_f32_native`` forms).")
    return native


dispatch_tensor_pow_contiguous_f32_native = _f32_only(dispatch_tensor_pow, "dispatch_tensor_pow_contiguous_f32_native")
dispatch_tensor_clamp_contiguous_f32_native = _f32_only(dispatch_tensor_clamp, "dispatch_tensor_clamp_contiguous_f32_native")
