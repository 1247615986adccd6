"""Typed dispatch families, operation events, scalar tensors and typed storage
(ft-dispatch/src/lib.rs:253-490, :680-800, :2830-3990; ft-autograd/src/lib.rs:876-1060; ft-core/src/lib.rs:827, :915)."""
import math

import pytest
import torch

from frankentorch_b200.autograd import events as E
from frankentorch_b200.core.dtype import DType
from frankentorch_b200.core.meta import Device, TensorMeta
from frankentorch_b200.core.storage import ScalarTensor, TensorStorage
from frankentorch_b200.dispatch import families as F
from frankentorch_b200.dispatch.keys import DispatchError, DispatchKey, DispatchKeyError
from frankentorch_b200.core.meta import TensorCompatError
from frankentorch_b200.runtime.ledger import ExecutionMode as M
from frankentorch_b200.session import FrankenTorchSession

X = torch.tensor([[0.5, -1.0, 2.0], [3.0, 0.25, -0.75]], dtype=torch.float64)


def test_operator_enums_round_trip_their_schema_base_names():
    for cls, n in ((F.BinaryOp, 13), (F.UnaryOp, 43), (F.ReductionOp, 6), (F.ScanOp, 2), (F.NormalizeOp, 2), (F.JoinOp, 2),
                   (F.ComparisonOp, 6)):
        assert len(cls) == n
        for m in cls:
            assert cls.from_schema_base(m.schema_base) is m
        assert cls.from_schema_base("no_such_op") is None
    assert F.UnaryOp.from_schema_base("leaky_relu") is F.UnaryOp.LeakyRelu and F.BinaryOp.from_schema_base("matmul") is F.BinaryOp.MatMul


@pytest.mark.parametrize("op", list(F.UnaryOp), ids=lambda o: o.value)
def test_every_unary_member_dispatches_and_matches_pytorch(op):
    x = X.abs() + 0.1 if op in (F.UnaryOp.Log, F.UnaryOp.Sqrt, F.UnaryOp.Rsqrt, F.UnaryOp.Log2, F.UnaryOp.Log10) else X / 4
    out = F.dispatch_tensor_unary(op, M.Strict, x, requires_grad=True)
    ref = {"gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, "leaky_relu": torch.nn.functional.leaky_relu,
           "elu": torch.nn.functional.elu, "hardswish": torch.nn.functional.hardswish, "hardsigmoid": torch.nn.functional.hardsigmoid,
           "hardtanh": torch.nn.functional.hardtanh, "softplus": torch.nn.functional.softplus, "mish": torch.nn.functional.mish,
           "relu": torch.relu}.get(op.value) or getattr(torch, op.value)
    want = ref(x)
    assert torch.allclose(out.values, want.to(x.dtype), atol=1e-12)
    d = out.decision
    predicate = op in (F.UnaryOp.IsNan, F.UnaryOp.IsFinite)     # answered outside the rule table: no autograd key
    ns = "cpu" if predicate else "autograd_cpu"
    assert isinstance(d, F.UnaryDispatchDecision) and d.op is op and d.kernel == f"{ns}::{op.value}_tensor_contiguous_f64"
    assert d.selected_key is (DispatchKey.CPU if predicate else DispatchKey.AutogradCPU) and d.backend_key is DispatchKey.CPU
    assert not d.fallback_used


def test_binary_comparison_and_the_keyset_without_autograd():
    out = F.dispatch_tensor_binary(F.BinaryOp.Atan2, M.Hardened, X, X.flip(0))
    assert torch.allclose(out.values, torch.atan2(X, X.flip(0)))
    assert out.decision.kernel == "cpu::atan2_tensor_contiguous_f64" and out.decision.selected_key is DispatchKey.CPU
    assert out.decision.mode is M.Hardened
    mm = F.dispatch_tensor_binary("matmul", M.Strict, X, X.t().contiguous(), True)
    assert torch.allclose(mm.values, X @ X.t())
    for op in F.ComparisonOp:
        c = F.dispatch_tensor_comparison(op, M.Strict, X, X.flip(1))
        assert c.values.dtype == X.dtype and torch.equal(c.values.bool(), getattr(torch, op.value)(X, X.flip(1)))
        assert isinstance(c.decision, F.ComparisonDispatchDecision) and c.decision.kernel.endswith(f"::{op.value}_tensor_contiguous_f64")
    f32 = F.dispatch_tensor_binary("add", M.Strict, X.float(), X.float())
    assert f32.values.dtype == torch.float32 and f32.decision.kernel.endswith("add_tensor_contiguous_f32")
    with pytest.raises(TensorCompatError):
        F.dispatch_tensor_binary("add", M.Strict, X, X.float())
    with pytest.raises(DispatchError):
        F.dispatch_tensor_binary("nope", M.Strict, X, X)


def test_values_with_meta_operands_and_typed_storage_of_the_result():
    meta = TensorMeta.from_shape([2, 2], DType.F32, Device.Cpu)
    out = F.dispatch_tensor_unary_contiguous_f32(F.UnaryOp.Neg, M.Strict, ([1.0, -2.0, 3.0, 4.0], meta))
    assert out.tolist() == [-1.0, 2.0, -3.0, -4.0] and tuple(out.values.shape) == (2, 2)
    st = out.storage
    assert st.dtype is DType.F32 and len(st) == 4 and st.as_f64() is None and st.as_f32() is not None
    assert st.to_f64_vec() == [-1.0, 2.0, -3.0, -4.0]
    with pytest.raises(DispatchError):
        F.dispatch_tensor_unary(F.UnaryOp.Neg, M.Strict, ([1.0, 2.0], meta))


def test_reductions_scans_normalisations_joins():
    for op, ref in ((F.ReductionOp.Sum, X.sum()), (F.ReductionOp.Mean, X.mean()), (F.ReductionOp.Prod, X.prod()),
                    (F.ReductionOp.Var, X.var()), (F.ReductionOp.Std, X.std())):
        r = F.dispatch_tensor_reduction(op, M.Strict, X, True)
        assert math.isclose(r.value, ref.item(), rel_tol=1e-12) and r.decision.op is op
    sq = X[:, :2].contiguous()
    assert math.isclose(F.dispatch_tensor_reduction("trace", M.Strict, sq).value, sq.trace().item())
    rd = F.dispatch_tensor_reduction_dim(F.ReductionOp.Var, M.Strict, X, -1)
    assert torch.allclose(rd.values, X.var(1)) and rd.decision.dim == 1 and rd.decision.kernel == "cpu::var_dim_tensor_contiguous_f64"
    with pytest.raises(DispatchError):
        F.dispatch_tensor_reduction_dim("trace", M.Strict, X, 0)
    with pytest.raises(DispatchError):
        F.dispatch_tensor_reduction_dim("sum", M.Strict, X, 2)
    sc = F.dispatch_tensor_scan_dim(F.ScanOp.CumProd, M.Strict, X, 1)
    assert torch.allclose(sc.values, X.cumprod(1)) and isinstance(sc.decision, F.ScanDimDispatchDecision)
    nm = F.dispatch_tensor_normalize_dim(F.NormalizeOp.LogSoftmax, M.Strict, X, 1)
    assert torch.allclose(nm.values, torch.log_softmax(X, 1)) and nm.decision.dim == 1
    j = F.dispatch_tensor_join(F.JoinOp.Stack, M.Strict, [X, X, X], 0)
    assert tuple(j.values.shape) == (3, 2, 3) and j.decision.num_inputs == 3 and j.decision.dim == 0
    with pytest.raises(DispatchKeyError):
        F.dispatch_tensor_join("cat", M.Strict, [], 0)


def test_single_operator_families_carry_their_parameters():
    p = F.dispatch_tensor_pow(M.Strict, X.abs(), 2.5)
    assert torch.allclose(p.values, X.abs() ** 2.5) and p.decision.exponent == 2.5 and p.decision.op == "pow"
    c = F.dispatch_tensor_clamp(M.Strict, X, -0.5, 1.0)
    assert torch.equal(c.values, X.clamp(-0.5, 1.0)) and (c.decision.min_val, c.decision.max_val) == (-0.5, 1.0)
    n = F.dispatch_tensor_norm(M.Strict, X, 3.0)
    assert math.isclose(n.value, torch.linalg.vector_norm(X, 3.0).item(), rel_tol=1e-12) and n.decision.p == 3.0
    nd = F.dispatch_tensor_norm_dim(M.Strict, X, 2.0, 0)
    assert torch.allclose(nd.values, torch.linalg.vector_norm(X, 2.0, dim=0)) and nd.decision.dim == 0
    lp = F.dispatch_tensor_lerp(M.Strict, X, X.flip(0), 0.3)
    assert torch.allclose(lp.values, torch.lerp(X, X.flip(0), 0.3)) and lp.decision.weight == 0.3
    a = F.dispatch_tensor_addmm(M.Strict, torch.ones(2, 2, dtype=torch.float64), X, X.t().contiguous(), 0.5, 2.0)
    assert torch.allclose(a.values, 0.5 + 2.0 * X @ X.t()) and (a.decision.beta, a.decision.alpha) == (0.5, 2.0)
    v = F.dispatch_tensor_addmv(M.Strict, torch.ones(2, dtype=torch.float64), X, X[0].contiguous(), 1.0, 1.0)
    assert torch.allclose(v.values, 1 + X @ X[0])
    s = F.dispatch_tensor_sort(M.Strict, X, 1, True)
    ref = torch.sort(X, 1, descending=True)
    assert torch.equal(s.values, ref.values) and torch.equal(s.indices, ref.indices) and s.decision.descending
    t = F.dispatch_tensor_topk(M.Strict, X, 2, 1, largest=False)
    ref = torch.topk(X, 2, 1, largest=False)
    assert torch.equal(t.values, ref.values) and torch.equal(t.indices, ref.indices) and (t.decision.k, t.decision.largest) == (2, False)
    with pytest.raises(DispatchError):
        F.dispatch_tensor_topk(M.Strict, X, 4, 1)
    assert "exponent=2.5" in p.decision.summary() and "op=pow" in p.decision.summary()


def test_dispatch_calls_leave_no_nodes_behind():
    F.dispatch_tensor_unary("exp", M.Strict, X)
    s = F._session(M.Strict, X.device)
    n = s.autograd_graph_len()
    for _ in range(5):
        F.dispatch_tensor_binary("mul", M.Strict, X, X, True)
    assert s.autograd_graph_len() == n


def test_operation_events_name_nodes_parameters_and_decisions():
    s = FrankenTorchSession(ledger_dispatch=False)
    s.operation_events = []
    x = s.tensor_variable(X.reshape(-1).tolist(), [2, 3], True)
    y, ev = E.tensor_unary(s, F.UnaryOp.Tanh, x)
    assert isinstance(ev, E.TensorUnaryOperationEvent) and (ev.op, ev.input, ev.out) == (F.UnaryOp.Tanh, x, y)
    assert ev.decision.selected_key is DispatchKey.AutogradCPU and s.last_operation_event is ev
    z, ev = E.tensor_binary(s, "mul", y, x)
    assert isinstance(ev, E.TensorOperationEvent) and (ev.lhs, ev.rhs, ev.out) == (y, x, z)
    r, ev = E.tensor_reduction_dim(s, "sum", z, 1)
    assert isinstance(ev, E.TensorReductionDimOperationEvent) and ev.dim == 1 and ev.decision.dim == 1
    c, ev = E.tensor_scan_dim(s, "cumsum", z, 0)
    assert isinstance(ev, E.TensorScanDimOperationEvent)
    n, ev = E.tensor_normalize_dim(s, "softmax", z, 1)
    assert isinstance(ev, E.TensorNormalizeDimOperationEvent)
    j, ev = E.tensor_join(s, "cat", [z, n], 1)
    assert isinstance(ev, E.TensorJoinOperationEvent) and ev.inputs == (z, n) and ev.decision.num_inputs == 2
    p, ev = E.tensor_pow(s, j, 2.0)
    assert isinstance(ev, E.TensorPowOperationEvent) and ev.exponent == 2.0
    cl, ev = E.tensor_clamp(s, p, 0.1, 5.0)
    assert isinstance(ev, E.TensorClampOperationEvent) and (ev.min_val, ev.max_val) == (0.1, 5.0)
    nm, ev = E.tensor_norm(s, cl, 2.0)
    assert isinstance(ev, E.TensorNormOperationEvent) and ev.p == 2.0
    total, ev = E.tensor_reduction(s, "prod", r)
    assert isinstance(ev, E.TensorReductionOperationEvent) and ev.op is F.ReductionOp.Prod and ev.input == r
    sc, ev = E.tensor_scalar(s, "mul", nm, 0.5)
    assert isinstance(ev, E.TensorScalarOperationEvent) and ev.scalar == 0.5 and ev.output_dtype is DType.F64
    srt, ev = E.tensor_sort(s, x, 1, True)
    assert isinstance(ev, E.TensorSortOperationEvent) and ev.descending
    tk, ev = E.tensor_topk(s, x, 2, 1)
    assert isinstance(ev, E.TensorTopKOperationEvent) and ev.k == 2 and ev.sorted
    lp, ev = E.tensor_lerp(s, x, y, 0.25)
    assert isinstance(ev, E.TensorLerpOperationEvent) and ev.weight == 0.25
    g, ev = E.record_tensor_op(s, "logcumsumexp", [x], dim=1)
    assert isinstance(ev, E.TensorGenericOperationEvent) and ev.op == "logcumsumexp" and ev.params == (("dim", 1),)
    assert len(s.operation_events) == 15 and isinstance(s.operation_events[9], E.TensorReductionOperationEvent)
    # the nodes are ordinary tape nodes: the gradient flows through all of them
    loss = s.tensor_add(s.tensor_sum(sc), s.tensor_sum(lp))
    rep = s.tensor_backward(loss)
    assert rep.gradient(x) is not None and torch.isfinite(rep.gradient(x)).all()
    a, b = s.variable(2.0, True), s.variable(3.0)
    out, ev = E.scalar_binary(s, F.BinaryOp.Mul, a, b)
    assert isinstance(ev, E.OperationEvent) and s.value(out) == 6.0 and ev.decision.kernel == "autograd_cpu::mul_scalar"


def test_scalar_tensor_identity_versions_views_and_fingerprint():
    t = ScalarTensor(1.5, DType.F64, Device.Cpu)
    u = t.with_value(2.5)
    assert u.id != t.id and u.storage_id != t.storage_id and u.version == t.version + 1 and u.value == 2.5 and u.meta == t.meta
    v = t.alias_view(3)
    assert v.storage_id == t.storage_id and v.id != t.id and v.meta.storage_offset == 3 and v.version == t.version
    f0 = t.evidence_fingerprint64()
    t.set_in_place(-1.0)
    assert t.version == 1 and t.value == -1.0 and t.evidence_fingerprint64() != f0
    assert t.meta.shape == () and t.meta.dtype is DType.F64
    with pytest.raises(Exception):
        t.alias_view(-1)


def test_tensor_storage_variants_and_accessors():
    for dt, data in ((DType.F64, [1.0, 2.0]), (DType.F32, [1.0, 2.0]), (DType.F16, [1.0, 2.0]), (DType.BF16, [1.0, 2.0]),
                     (DType.QInt8, [-3, 4]), (DType.QUInt8, [3, 200])):
        st = TensorStorage.from_values(data, dt)
        assert st.dtype is dt and len(st) == 2 and not st.is_empty()
        hit = [n for n in ("f64", "f32", "f16", "bf16", "qint8", "quint8", "complex64", "complex128") if getattr(st, "as_" + n)() is not None]
        assert hit == [dt.value.lower()]
        assert st.to_f64_vec() == [float(v) for v in data] and st.to_f32_vec() == [float(v) for v in data]
    z = TensorStorage.from_tensor(torch.tensor([1 + 2j, 3 - 1j], dtype=torch.complex64))
    assert z.dtype is DType.Complex64 and z.to_f64_vec() == [1.0, 3.0] and z.as_complex64() is not None
    assert TensorStorage.from_values([], DType.F64).is_empty()
    assert TensorStorage.from_values([1.0], DType.F64) == TensorStorage.from_values([1.0], DType.F64)
    assert TensorStorage.from_values([1.0], DType.F64) != TensorStorage.from_values([1.0], DType.F32)
    with pytest.raises(ValueError):
        TensorStorage(DType.I64, torch.zeros(2, dtype=torch.int64))
    with pytest.raises(ValueError):
        TensorStorage(DType.F32, torch.zeros(2, dtype=torch.float64))


# ----------------------------------------------------------------------------- scalar entry points
def test_scalar_dispatch_entry_points_resolve_keys_and_version_the_result():
    import math
    from frankentorch_b200.core.storage import ScalarTensor
    from frankentorch_b200.dispatch import scalar as S
    from frankentorch_b200.dispatch.keys import DispatchKey, DispatchKeyError, DispatchKeySet
    from frankentorch_b200.dispatch.schema import OpSchemaError, SchemaRegistry, SchemaRegistryError, parse_schema_or_name
    from frankentorch_b200.runtime.ledger import ExecutionMode

    x, y = ScalarTensor(-2.5), ScalarTensor(4.0)
    out = S.dispatch_scalar_unary(F.UnaryOp.Abs, ExecutionMode.Strict, x, requires_grad=True)
    assert out.tensor.value == 2.5 and out.tensor.version == x.version + 1 and out.tensor.id != x.id
    assert out.decision.kernel == "autograd_cpu::abs_scalar" and out.decision.selected_key is DispatchKey.AutogradCPU
    assert S.dispatch_scalar_unary("sqrt", ExecutionMode.Strict, x).tensor.value != S.dispatch_scalar_unary("sqrt", ExecutionMode.Strict, x).tensor.value   # NaN
    assert S.dispatch_scalar_unary("log", ExecutionMode.Strict, ScalarTensor(0.0)).tensor.value == -math.inf
    assert S.dispatch_scalar_unary("exp", ExecutionMode.Strict, ScalarTensor(1e4)).tensor.value == math.inf
    # every unary member has a scalar kernel that agrees with torch in f64
    for op in F.UnaryOp:
        for v in (-1.7, 0.3, 2.2):
            got = S.dispatch_scalar_unary(op, ExecutionMode.Strict, ScalarTensor(v)).tensor.value
            fn = {"isnan": torch.isnan, "isinf": torch.isinf, "isfinite": torch.isfinite}.get(op.value) or getattr(torch, op.value, None) \
                or getattr(torch.nn.functional, op.value)
            want = float(fn(torch.tensor(v, dtype=torch.float64)))
            assert (got != got and want != want) or abs(got - want) <= 1e-12 * max(1.0, abs(want)), (op, v, got, want)

    cmp = S.dispatch_scalar_comparison(F.ComparisonOp.Lt, ExecutionMode.Strict, x, y)
    assert cmp.tensor.value == 1.0 and cmp.decision.kernel == "cpu::lt_scalar"
    nan = ScalarTensor(math.nan)
    assert S.dispatch_scalar_comparison("eq", ExecutionMode.Strict, nan, nan).tensor.value == 0.0
    assert S.dispatch_scalar_comparison("ne", ExecutionMode.Strict, nan, nan).tensor.value == 1.0

    assert S.dispatch_scalar_pow(ExecutionMode.Strict, y, 0.5).tensor.value == 2.0
    assert math.isnan(S.dispatch_scalar_pow(ExecutionMode.Strict, x, 0.5).tensor.value)
    assert S.dispatch_scalar_clamp(ExecutionMode.Strict, x, -1.0, 1.0).tensor.value == -1.0
    assert math.isnan(S.dispatch_scalar_clamp(ExecutionMode.Strict, nan, -1.0, 1.0).tensor.value)

    ks = S.dispatch_keyset_for_tensors(x, y, True)
    assert ks == S.dispatch_keyset_for_tensor_meta(x.meta, y.meta, True) and ks.has(DispatchKey.AutogradCPU)
    assert S.dispatch_keyset_for_single_tensor(x, False) == S.dispatch_keyset_for_single_tensor_meta(x.meta, False)
    assert ks.highest_priority_type_id() is DispatchKey.AutogradCPU
    assert ks.highest_priority_backend_type_id() is DispatchKey.CPU
    with pytest.raises(DispatchKeyError):
        S.highest_priority_type_id(DispatchKeySet.empty())
    with pytest.raises(DispatchKeyError):
        S.highest_priority_backend_type_id(DispatchKeySet.from_keys([DispatchKey.BackendSelect]))

    b = S.dispatch_scalar_binary_with_keyset(F.BinaryOp.Div, ExecutionMode.Strict, y, ScalarTensor(0.0), ks)
    assert b.tensor.value == math.inf and b.decision.kernel == "autograd_cpu::div_scalar"
    with pytest.raises(DispatchKeyError):
        S.dispatch_scalar_binary_with_keyset(F.BinaryOp.MatMul, ExecutionMode.Strict, x, y, ks)
    with pytest.raises(DispatchKeyError):      # composite-only set: strict refuses, hardened falls back
        S.dispatch_scalar_binary_with_keyset("add", ExecutionMode.Strict, x, y,
                                             DispatchKeySet.from_keys([DispatchKey.CompositeExplicitAutograd, DispatchKey.CPU]))
    h = S.dispatch_scalar_binary_with_keyset("add", ExecutionMode.Hardened, x, y,
                                             DispatchKeySet.from_keys([DispatchKey.CompositeExplicitAutograd, DispatchKey.CPU]))
    assert h.tensor.value == 1.5 and h.decision.fallback_used
    assert S.dispatch_scalar_binary_tensors("max", ExecutionMode.Strict, x, y).tensor.value == 4.0

    assert S.schema_dispatch_key_from_tag("AutogradCPU") is DispatchKey.AutogradCPU
    with pytest.raises(OpSchemaError):
        S.schema_dispatch_key_from_tag("XLA")
    with pytest.raises(OpSchemaError):
        S.schema_dispatch_keyset_from_tags(["AutogradCPU"])          # autograd without its backend
    reg = SchemaRegistry()
    name = reg.register(parse_schema_or_name("aten::mul.Tensor"), S.schema_dispatch_keyset_from_tags(["CPU", "AutogradCPU"]))
    r = S.dispatch_scalar_binary_registered(reg, name, ExecutionMode.Strict, x, y)
    assert r.tensor.value == -10.0 and r.decision.op == "mul"
    with pytest.raises(SchemaRegistryError):
        S.dispatch_scalar_binary_registered(reg, "aten::nope", ExecutionMode.Strict, x, y)


def test_binary_with_explicit_keyset_and_native_f32_entry_points():
    from frankentorch_b200.dispatch.keys import DispatchKey, DispatchKeyError, DispatchKeySet
    from frankentorch_b200.runtime.ledger import ExecutionMode
    a = torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64)
    b = torch.tensor([4.0, 5.0, 6.0], dtype=torch.float64)
    ks = DispatchKeySet.from_keys([DispatchKey.BackendSelect, DispatchKey.CPU, DispatchKey.AutogradCPU])
    out = F.dispatch_tensor_binary_contiguous_f64_with_keyset(F.BinaryOp.Mul, ExecutionMode.Strict, a, b, ks)
    assert out.values.tolist() == [4.0, 10.0, 18.0]
    assert out.decision.selected_key is DispatchKey.AutogradCPU and out.decision.keyset_bits == ks.bits
    assert out.decision.kernel.startswith("autograd_cpu::mul_tensor_contiguous")
    plain = DispatchKeySet.from_keys([DispatchKey.CPU])
    d = F.dispatch_tensor_binary_contiguous_f64_with_keyset("add", ExecutionMode.Strict, a, b, plain).decision
    assert d.selected_key is DispatchKey.CPU and d.kernel.startswith("cpu::add_tensor_contiguous") and not d.fallback_used
    comp = DispatchKeySet.from_keys([DispatchKey.CompositeExplicitAutograd, DispatchKey.CPU])
    with pytest.raises(DispatchKeyError):
        F.dispatch_tensor_binary_contiguous_f64_with_keyset("add", ExecutionMode.Strict, a, b, comp)
    h = F.dispatch_tensor_binary_contiguous_f64_with_keyset("add", ExecutionMode.Hardened, a, b, comp)
    assert h.decision.fallback_used and h.values.tolist() == [5.0, 7.0, 9.0]
    with pytest.raises(DispatchKeyError):
        F.dispatch_tensor_binary_contiguous_f64_with_keyset("add", ExecutionMode.Strict, a, b, DispatchKeySet.empty())
    with pytest.raises(DispatchKeyError):       # a device key set over host operands
        F.dispatch_tensor_binary_contiguous_f64_with_keyset("add", ExecutionMode.Strict, a, b,
                                                            DispatchKeySet.from_keys([DispatchKey.SM100]))
    x = torch.tensor([-2.0, 0.5, 3.0])
    assert F.dispatch_tensor_pow_contiguous_f32_native(ExecutionMode.Strict, x, 2.0).values.tolist() == [4.0, 0.25, 9.0]
    assert F.dispatch_tensor_clamp_contiguous_f32_native(ExecutionMode.Strict, x, -1.0, 1.0).values.tolist() == [-1.0, 0.5, 1.0]
    with pytest.raises(F.DispatchError):
        F.dispatch_tensor_pow_contiguous_f32_native(ExecutionMode.Strict, a, 2.0)
