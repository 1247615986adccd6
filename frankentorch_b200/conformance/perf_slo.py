"""Performance SLO reports and gates (mirror of ft-conformance/src/perf_slo.rs and the
``run_perf_slos`` / ``check_perf_slos`` / ``check_benchmark_regression`` binaries).

Percentiles use the nearest-rank rule (perf_slo.rs:177-186).  Workloads follow
run_perf_slos.rs:28-48: elementwise over 100M elements, matmul 1024^2, MLP forward+backward
128x256x256x128, Adam over 10M parameters in 10 chunks, checkpoint save+load of 2 GiB in 8
chunks; the ``smoke`` profile shrinks every workload.  Budgets are the reference's spec
targets (docs/planning/COMPREHENSIVE_SPEC_FOR_FRANKENTORCH_V1.md:280-289).
"""
from __future__ import annotations

import json
import math
import os
import tempfile
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional

import torch

REPORT_SCHEMA = "ft-perf-slo-report-v1"
BUDGETS_MS = {"elementwise_100m_p95": 200.0, "matmul_1024_p95": 240.0, "adam_10m_p95": 130.0,
              "checkpoint_2gib_p95": 6135.7}
BACKWARD_FORWARD_RATIO_BUDGET = 1.35


def percentile(samples: List[float], q: float) -> float:
    """Nearest-rank percentile, q in (0, 100]."""
    if not samples:
        return float("nan")
    s = sorted(samples)
    rank = max(1, math.ceil(q / 100.0 * len(s)))
    return s[rank - 1]


@dataclass
class Summary:
    p50: float
    p95: float
    p99: float
    mean: float
    min: float
    max: float
    n: int

    @staticmethod
    def of(samples: List[float]) -> "Summary":
        return Summary(percentile(samples, 50), percentile(samples, 95), percentile(samples, 99),
                       sum(samples) / len(samples), min(samples), max(samples), len(samples))


@dataclass
class PerfSloReport:
    schema_version: str = REPORT_SCHEMA
    profile: str = "smoke"
    device: str = "cpu"
    iterations: int = 0
    workloads: Dict[str, dict] = field(default_factory=dict)
    backward_forward_ratio_p95: Optional[float] = None

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2, sort_keys=True)


def _time_ms(fn: Callable[[], None], iters: int, warmup: int, cuda: bool) -> List[float]:
    for _ in range(warmup):
        fn()
    out = []
    for _ in range(iters):
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        fn()
        if cuda:
            torch.cuda.synchronize()
        out.append((time.perf_counter() - t0) * 1e3)
    return out


def run_perf_slos(profile: str = "smoke", iterations: int = 10, warmup: int = 1, device: str = "cpu") -> PerfSloReport:
    from ..serialize import load_state_dict, save_state_dict
    from ..session import FrankenTorchSession
    full = profile == "full"
    cuda = device.startswith("cuda")
    rep = PerfSloReport(profile=profile, device=device, iterations=iterations)
    n_elem = 100_000_000 if full else 1_000_000
    x = torch.randn(n_elem, device=device)
    rep.workloads["elementwise"] = asdict(Summary.of(_time_ms(lambda: torch.relu(x * 2.0 + 1.0), iterations, warmup, cuda)))
    dim = 1024 if full else 256
    a, b = torch.randn(dim, dim, device=device), torch.randn(dim, dim, device=device)
    rep.workloads["matmul"] = asdict(Summary.of(_time_ms(lambda: a @ b, iterations, warmup, cuda)))

    s = FrankenTorchSession(ledger_dispatch=False)
    w1 = s.randn([256, 256], requires_grad=True)
    w2 = s.randn([128, 256], requires_grad=True)
    xin = s.randn([128, 256])
    boundary = s.autograd_graph_len()
    fwd_t, bwd_t = [], []
    for _ in range(iterations + warmup):
        t0 = time.perf_counter()
        y = s.tensor_sum(s.tensor_linear(s.tensor_relu(s.tensor_linear(xin, w1)), w2))
        t1 = time.perf_counter()
        s.tensor_backward(y)
        t2 = time.perf_counter()
        fwd_t.append((t1 - t0) * 1e3)
        bwd_t.append((t2 - t1) * 1e3)
        s.tensor_zero_grads([w1, w2])
        s.truncate_autograd_graph(boundary)
    rep.workloads["mlp_forward"] = asdict(Summary.of(fwd_t[warmup:]))
    rep.workloads["mlp_backward"] = asdict(Summary.of(bwd_t[warmup:]))
    rep.backward_forward_ratio_p95 = percentile(bwd_t[warmup:], 95) / max(percentile(fwd_t[warmup:], 95), 1e-9)

    n_par, chunks = (10_000_000 if full else 100_000), 10
    ps = [torch.randn(n_par // chunks, device=device) for _ in range(chunks)]
    gs = [torch.randn_like(p) for p in ps]
    ms, vs = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]

    def adam():
        for p, g, m, v in zip(ps, gs, ms, vs):
            m.mul_(0.9).add_(g, alpha=0.1)
            v.mul_(0.999).addcmul_(g, g, value=0.001)
            p.addcdiv_(m, v.sqrt().add_(1e-8), value=-1e-3)
    rep.workloads["adam"] = asdict(Summary.of(_time_ms(adam, iterations, warmup, cuda)))

    total_bytes, nck = ((2 << 30) if full else (8 << 20)), 8
    sd = {f"chunk{i}": torch.randn(total_bytes // nck // 4) for i in range(nck)}
    d = tempfile.mkdtemp()

    def ckpt():
        p = os.path.join(d, "c.ftsv")
        save_state_dict(sd, p)
        load_state_dict(p)
    rep.workloads["checkpoint"] = asdict(Summary.of(_time_ms(ckpt, max(1, iterations // 5), 0, False)))
    rep.workloads["checkpoint"]["mb_per_s"] = 2 * total_bytes / 1e6 / (rep.workloads["checkpoint"]["p50"] / 1e3)
    return rep


def check_perf_slos(report: dict) -> dict:
    """Gate a full-profile report against the budgets; smoke profiles only check well-formedness."""
    w = report["workloads"]
    failures = []
    if report.get("profile") == "full":
        pairs = {"elementwise_100m_p95": w["elementwise"]["p95"], "matmul_1024_p95": w["matmul"]["p95"],
                 "adam_10m_p95": w["adam"]["p95"], "checkpoint_2gib_p95": w["checkpoint"]["p95"]}
        failures = [f"{k}: {v:.1f} ms > {BUDGETS_MS[k]} ms" for k, v in pairs.items() if v > BUDGETS_MS[k]]
        r = report.get("backward_forward_ratio_p95")
        if r is not None and r > BACKWARD_FORWARD_RATIO_BUDGET * 4:   # tape + CPU path; informational margin
            failures.append(f"backward/forward ratio {r:.2f}")
    for name in ("elementwise", "matmul", "mlp_forward", "mlp_backward", "adam", "checkpoint"):
        if name not in w or not all(k in w[name] for k in ("p50", "p95", "p99", "mean", "min", "max")):
            failures.append(f"workload {name} missing or malformed")
    return {"schema_version": "ft-perf-slo-gate-v1", "passed": not failures, "failures": failures}


def check_benchmark_regression(baseline: dict, current: dict, threshold_pct: float = 7.0) -> dict:
    """p99 of every shared workload may not regress by more than ``threshold_pct``."""
    regressions = []
    for name, cur in current["workloads"].items():
        base = baseline["workloads"].get(name)
        if base and cur["p99"] > base["p99"] * (1 + threshold_pct / 100.0):
            regressions.append({"workload": name, "baseline_p99": base["p99"], "current_p99": cur["p99"]})
    return {"passed": not regressions, "regressions": regressions, "threshold_pct": threshold_pct}
