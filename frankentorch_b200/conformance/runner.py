"""Golden-vector conformance runner (mirror of ft-conformance's ``run_*_conformance``).

The suite file ``golden_suite.json`` consolidates the reference's fixture families
(ft-conformance/fixtures/*.json: expected outputs / gradients with tolerances, adversarial
strict-vs-hardened dispatch cases, module-state cases ...).  Every family runs in BOTH
execution modes; each case yields a ``CaseResult`` and a structured log line of schema
``ft-conformance-log-v1`` (artifacts/phase2c/TEST_LOG_CONTRACT_V1.md; emitter
ft-conformance/src/logging.rs:13-84).
"""
from __future__ import annotations

import json
import math
import os
import platform
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..core.dtype import DType
from ..core.meta import Device, TensorMeta, TensorMetaError, ensure_compatible
from ..dispatch.keys import (DispatchKey, DispatchKeyError, DispatchKeySet, dispatch_scalar_binary)
from ..dispatch.schema import OpSchemaError, ParsedOpSchema, SchemaRegistry, SchemaRegistryError, parse_schema_or_name
from ..runtime.ledger import ExecutionMode
from ..runtime.native import fnv1a64
from ..session import FrankenTorchSession

SUITE_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_suite.json")
LOG_SCHEMA = "ft-conformance-log-v1"


@dataclass
class CaseResult:
    family: str
    name: str
    mode: str
    passed: bool
    detail: str = ""
    reason_code: str = "ok"


@dataclass
class FamilyReport:
    family: str
    mode: str
    cases_total: int = 0
    cases_passed: int = 0
    results: List[CaseResult] = field(default_factory=list)

    def ok(self) -> bool:
        return self.cases_total == self.cases_passed


def load_suite(path: str = SUITE_PATH) -> Dict[str, List[dict]]:
    with open(path) as f:
        return json.load(f)["families"]


def env_fingerprint() -> str:
    blob = f"{platform.system()}|{platform.machine()}|py{platform.python_version()}|torch{torch.__version__}"
    return f"det64:{fnv1a64(blob.encode()):016x}"


def structured_log(result: CaseResult, seed: int = 42, packet: str = "FT-P2C-005", suite: str = "golden") -> dict:
    """One JSONL record with the 13 required fields of the log contract."""
    return {
        "schema_version": LOG_SCHEMA, "ts_unix_ms": int(time.time() * 1000), "suite_id": suite,
        "scenario_id": f"{result.family}/{result.mode}:{result.name}", "fixture_id": f"{result.family}.json",
        "packet_id": packet, "mode": result.mode, "seed": seed, "env_fingerprint": env_fingerprint(),
        "artifact_refs": ["frankentorch_b200/conformance/golden_suite.json"],
        "replay_command": f"python -m frankentorch_b200.conformance.run_e2e_matrix --mode {result.mode} --family {result.family}",
        "outcome": "pass" if result.passed else "fail", "reason_code": result.reason_code,
        "detail": result.detail[:400],
    }


def canonicalize(name: str) -> str:
    """Scenario-id form of a case name: lower case, runs of other characters become one underscore."""
    out, prev = [], False
    for ch in name.lower():
        if ch.isalnum():
            out.append(ch)
            prev = False
        elif not prev:
            out.append("_")
            prev = True
    return "".join(out).strip("_")


def deterministic_seed(parts: Sequence[str]) -> int:
    """Seed of a scenario: FNV-1a 64 over its identifying strings, so a replay draws the same numbers."""
    return fnv1a64("\x1f".join(parts).encode())


@dataclass
class StructuredCaseLog:
    """One record of the structured conformance log, built from the identifiers of a case
    (ft-conformance/src/logging.rs:30 ``StructuredCaseLog::new``, :79 ``with_extra_fields``).  The scenario id
    is ``suite/mode:case``, the seed is derived from the identifiers, and family-specific values ride in
    ``extra_fields``, which flatten into the JSON record beside the fixed fields without replacing one."""
    suite_id: str
    fixture_id: str
    packet_id: str
    case_name: str
    mode: str
    artifact_refs: List[str]
    replay_command: str
    outcome: str
    reason_code: str
    extra_fields: Dict[str, object] = field(default_factory=dict)
    ts_unix_ms: int = field(default_factory=lambda: int(time.time() * 1000))

    def __post_init__(self):
        self.mode = getattr(self.mode, "value", self.mode)
        if self.mode not in ("strict", "hardened"):
            raise ValueError(f"mode must be strict or hardened, got {self.mode!r}")
        self.scenario_id = f"{self.suite_id}/{self.mode}:{canonicalize(self.case_name)}"
        self.seed = deterministic_seed([self.suite_id, self.fixture_id, self.packet_id, self.scenario_id, self.mode])

    def with_extra_fields(self, extra_fields: Dict[str, object]) -> "StructuredCaseLog":
        self.extra_fields = dict(sorted(extra_fields.items()))
        return self

    def to_record(self) -> dict:
        rec = {
            "schema_version": LOG_SCHEMA, "ts_unix_ms": self.ts_unix_ms, "suite_id": self.suite_id,
            "scenario_id": self.scenario_id, "fixture_id": self.fixture_id, "packet_id": self.packet_id,
            "mode": self.mode, "seed": self.seed, "env_fingerprint": env_fingerprint(),
            "artifact_refs": list(self.artifact_refs), "replay_command": self.replay_command,
            "outcome": self.outcome, "reason_code": self.reason_code,
        }
        for k, v in self.extra_fields.items():
            rec.setdefault(k, v)
        return rec

    def to_json_line(self) -> str:
        return json.dumps(self.to_record(), sort_keys=True)


def _close(got: Sequence[float], want: Sequence[float], tol: float) -> Optional[str]:
    if len(got) != len(want):
        return f"length {len(got)} != {len(want)}"
    for i, (g, w) in enumerate(zip(got, want)):
        if isinstance(w, str):
            w = float(w)
        if math.isnan(w) and math.isnan(g):
            continue
        if not (abs(g - w) <= tol * max(1.0, abs(w))):
            return f"index {i}: got {g!r}, want {w!r}"
    return None


def _sess(mode) -> FrankenTorchSession:
    return FrankenTorchSession(mode)


def _check(res: List[Optional[str]]) -> Optional[str]:
    for r in res:
        if r:
            return r
    return None


# --------------------------------------------------------------------------------------- families
def _scalar_autograd(c, mode):
    s = _sess(mode)
    a, b = s.variable(c["lhs"], True), s.variable(c["rhs"], True)
    o = getattr(s, c["op"])(a, b)
    rep = s.backward(o)
    tol = c.get("tolerance", 1e-12)
    return _check([_close([s.value(o)], [c["expected_output"]], tol),
                   _close([rep.gradient(a)], [c["expected_lhs_grad"]], tol),
                   _close([rep.gradient(b)], [c["expected_rhs_grad"]], tol)])


def _autograd_scheduler(c, mode):
    s = _sess(mode)
    x, y = s.variable(c["x"], True), s.variable(c["y"], True)
    out = s.mul(s.add(x, y), x)          # (x + y) * x
    rep = s.backward(out)
    tol = c.get("tolerance", 1e-12)
    if rep.telemetry.execution_order != c["expected_execution_order"]:
        return f"execution order {rep.telemetry.execution_order} != {c['expected_execution_order']}"
    return _check([_close([rep.gradient(x)], [c["expected_x_grad"]], tol), _close([rep.gradient(y)], [c["expected_y_grad"]], tol)])


def _dispatch_key(c, mode):
    exp = c["strict" if mode == ExecutionMode.Strict else "hardened"]
    try:
        ks = None
        if "keyset" in c:
            ks = DispatchKeySet.from_keys([DispatchKey.parse(k) for k in c["keyset"]])
        elif "keyset_bits" in c:
            ks = DispatchKeySet.from_bits_checked(int(c["keyset_bits"]))
        val, dec = dispatch_scalar_binary(
            c["op"], mode, c["lhs"], c["rhs"], c.get("requires_grad", False), ks,
            DType.parse(c.get("lhs_dtype", "F64")), DType.parse(c.get("rhs_dtype", "F64")),
            c.get("lhs_device", "Cpu"), c.get("rhs_device", "Cpu"))
    except Exception as e:   # every failure must be a typed, fail-closed error
        if exp.get("expect_error"):
            sub = exp.get("expect_error_contains") or exp.get("expected_error_contains")
            return None
        return f"unexpected error {type(e).__name__}: {e}"
    if exp.get("expect_error"):
        return "expected an error, dispatch succeeded"
    errs = [_close([val], [exp["expected_output"]], c.get("tolerance", 1e-12))]
    if dec.selected_key.name != exp["expected_selected_key"]:
        errs.append(f"selected key {dec.selected_key.name} != {exp['expected_selected_key']}")
    if dec.backend_key.name != exp["expected_backend_key"]:
        errs.append(f"backend key {dec.backend_key.name} != {exp['expected_backend_key']}")
    if dec.kernel != exp["expected_kernel"]:
        errs.append(f"kernel {dec.kernel} != {exp['expected_kernel']}")
    if dec.fallback_used != exp["expected_fallback"]:
        errs.append(f"fallback {dec.fallback_used} != {exp['expected_fallback']}")
    return _check(errs)


def _op_schema(c, mode):
    try:
        parsed = parse_schema_or_name(c["schema_input"])
    except OpSchemaError as e:
        return None if not c.get("expect_parse_ok", True) else f"parse failed: {e}"
    if not c.get("expect_parse_ok", True):
        return "expected a parse failure"
    if c.get("expect_schema_variant") and not isinstance(parsed, ParsedOpSchema):
        return "expected a full schema"
    if "expect_out_variant" in c and isinstance(parsed, ParsedOpSchema) and parsed.is_out_variant != c["expect_out_variant"]:
        return f"out variant {parsed.is_out_variant} != {c['expect_out_variant']}"
    if c.get("expect_name_normalization") and "name_input" in c:
        n1 = (parsed.op if isinstance(parsed, ParsedOpSchema) else parsed).unambiguous_name()
        n2 = parse_schema_or_name(c["name_input"]).unambiguous_name()
        if n1 != n2:
            return f"normalized names differ: {n1} vs {n2}"
    if "expect_dispatch_ok" in c:
        reg = SchemaRegistry()
        try:
            ks = DispatchKeySet.from_keys([DispatchKey.parse(k) for k in c.get("dispatch_tags", [])])
            name = reg.register(parsed, ks)
            entry = reg.lookup(name)
            _, dec = dispatch_scalar_binary(entry.op, mode, 1.0, 2.0, True, entry.keyset)
            ok = True
            if c.get("expected_kernel") and dec.kernel != c["expected_kernel"]:
                return f"kernel {dec.kernel} != {c['expected_kernel']}"
        except (SchemaRegistryError, DispatchKeyError):
            ok = False
        if ok != c["expect_dispatch_ok"]:
            return f"dispatch ok={ok}, expected {c['expect_dispatch_ok']}"
    return None


def _tensor_meta(c, mode):
    try:
        strides = c.get("strides")
        if strides is None:
            m = TensorMeta.from_shape(c["shape"]).with_storage_offset(c.get("storage_offset", 0))
        else:
            m = TensorMeta.from_shape_and_strides(c["shape"], strides, c.get("storage_offset", 0))
        lin = m.storage_index_for(c["index"])
    except TensorMetaError as e:
        return None if not c["expect_valid"] else f"unexpected meta error: {e}"
    if not c["expect_valid"]:
        return "expected invalid metadata"
    errs = []
    if lin != c["expected_linear_index"]:
        errs.append(f"linear index {lin} != {c['expected_linear_index']}")
    if m.numel != c["expected_numel"]:
        errs.append(f"numel {m.numel} != {c['expected_numel']}")
    if m.is_contiguous() != c["expected_contiguous"]:
        errs.append(f"contiguous {m.is_contiguous()} != {c['expected_contiguous']}")
    if "expect_compat_error" in c:
        a = TensorMeta.from_shape(c["shape"], DType.parse(c["lhs_dtype"]), Device.parse(c["lhs_device"]))
        b = TensorMeta.from_shape(c["shape"], DType.parse(c["rhs_dtype"]), Device.parse(c["rhs_device"]))
        try:
            ensure_compatible(a, b)
            failed, msg = False, ""
        except ValueError as e:
            failed, msg = True, str(e)
        if failed != c["expect_compat_error"]:
            errs.append(f"compat error {failed} != {c['expect_compat_error']}")
        elif failed and c.get("expected_compat_error_contains", "") not in msg:
            errs.append(f"compat message {msg!r} lacks {c['expected_compat_error_contains']!r}")
    return _check(errs)


def _tensor_unary(c, mode):
    s = _sess(mode)
    x = s.tensor_variable(c["input"], c["shape"], True)
    kw = {}
    if c["op"] == "leaky_relu":
        kw["slope"] = c.get("negative_slope", 0.01)
    y = getattr(s, "tensor_" + c["op"])(x, **kw)
    tol = c.get("tolerance", 1e-12)
    errs = [_close(s.tensor_values(y), c["expected_output"], tol)]
    if "expected_grad" in c:
        rep = s.tensor_backward(s.tensor_sum(y))
        errs.append(_close(s.tensor_gradient(rep, x), c["expected_grad"], tol))
    return _check(errs)


def _tensor_binary(c, mode):
    s = _sess(mode)
    op = c["op"]
    ls, rs = c.get("lhs_shape", c.get("shape")), c.get("rhs_shape", c.get("shape"))
    a, b = s.tensor_variable(c["lhs"], ls, True), s.tensor_variable(c["rhs"], rs, True)
    y = getattr(s, "tensor_" + op)(a, b)
    tol = c.get("tolerance", 1e-12)
    errs = [_close(s.tensor_values(y), c["expected_output"], tol)]
    if "expected_lhs_grad" in c:
        root = y if s.tensor_numel(y) == 1 and not s.tensor_shape(y) else s.tensor_sum(y)
        rep = s.tensor_backward(root)
        errs += [_close(s.tensor_gradient(rep, a), c["expected_lhs_grad"], tol),
                 _close(s.tensor_gradient(rep, b), c["expected_rhs_grad"], tol)]
    return _check(errs)


def _reduce_like(c, mode):
    s = _sess(mode)
    x = s.tensor_variable(c["input"], c["shape"], True)
    op, kw = c["op"], {}
    if "dim" in c and op not in ("sum", "mean", "trace"):
        kw["dim"] = c["dim"]
    if op == "norm":
        kw = {"p": c.get("p", 2.0)}
    y = getattr(s, "tensor_" + op)(x, **kw)
    tol = c.get("tolerance", 1e-12)
    errs = [_close(s.tensor_values(y), c["expected_output"], tol)]
    if "expected_grad" in c:
        rep = s.tensor_backward(y if s.tensor_numel(y) == 1 and not s.tensor_shape(y) else s.tensor_sum(y))
        errs.append(_close(s.tensor_gradient(rep, x), c["expected_grad"], tol))
    return _check(errs)


def _tensor_join(c, mode):
    s = _sess(mode)
    ids = [s.tensor_variable(v, sh, True) for v, sh in zip(c["inputs"], c["input_shapes"])]
    y = getattr(s, "tensor_" + c["op"])(ids, dim=c["dim"])
    errs = [_close(s.tensor_values(y), c["expected_output"], 1e-12)]
    if s.tensor_shape(y) != c["expected_shape"]:
        errs.append(f"shape {s.tensor_shape(y)} != {c['expected_shape']}")
    if "expected_grads" in c:
        rep = s.tensor_backward(s.tensor_sum(y))
        for i, g in zip(ids, c["expected_grads"]):
            errs.append(_close(s.tensor_gradient(rep, i), g, 1e-12))
    return _check(errs)


def _tensor_shape(c, mode):
    s = _sess(mode)
    x = s.tensor_variable(c["input"], c["input_shape"], False)
    p, op = c.get("params", {}), c["op"]
    if op == "reshape":
        y = s.tensor_reshape(x, shape=tuple(p["new_shape"]))
    elif op == "squeeze":
        y = s.tensor_squeeze(x, dim=p.get("dim"))
    elif op == "unsqueeze":
        y = s.tensor_unsqueeze(x, dim=p["dim"])
    elif op == "transpose":
        y = s.tensor_transpose(x, dim0=p["dim0"], dim1=p["dim1"])
    elif op == "permute":
        y = s.tensor_permute(x, dims=tuple(p["dims"]))
    elif op == "flatten":
        y = s.tensor_flatten(x, start=p.get("start_dim", 0), end=p.get("end_dim", -1))
    elif op == "narrow":
        y = s.tensor_narrow(x, dim=p["dim"], start=p["start"], length=p["length"])
    else:
        return f"unknown shape op {op}"
    errs = [_close(s.tensor_values(y), c["expected_output"], 1e-12)]
    if s.tensor_shape(y) != c["expected_shape"]:
        errs.append(f"shape {s.tensor_shape(y)} != {c['expected_shape']}")
    return _check(errs)


def _tensor_indexing(c, mode):
    s = _sess(mode)
    op = c["op"]
    if op == "where":
        y = s.tensor_where(s.tensor_variable(c["condition"], c["condition_shape"]), s.tensor_variable(c["x"], c["x_shape"]),
                           s.tensor_variable(c["y"], c["y_shape"]))
    else:
        x = s.tensor_variable(c["input"], c["input_shape"])
        if op == "masked_fill":
            y = s.tensor_masked_fill(x, s.tensor_variable(c["mask"], c["mask_shape"]), value=c["value"])
        else:
            idx = s.tensor_variable(c["index"], c["index_shape"])
            if op in ("scatter", "scatter_add"):
                y = getattr(s, "tensor_" + op)(x, idx, s.tensor_variable(c["src"], c["src_shape"]), dim=c["dim"])
            else:
                y = getattr(s, "tensor_" + op)(x, idx, dim=c["dim"])
    errs = [_close(s.tensor_values(y), c["expected_output"], 1e-12)]
    if s.tensor_shape(y) != c["expected_shape"]:
        errs.append(f"shape {s.tensor_shape(y)} != {c['expected_shape']}")
    return _check(errs)
