"""Library entry points of the conformance harness (ft-conformance/src/lib.rs:38 ``HarnessConfig``, :580
``HarnessReport`` / ``BenchReport``, :1627 ``E2EForensicsSummary``, :1685 ``run_smoke``, :1777-2680 the
``run_<family>_conformance`` functions, :2682 ``emit_e2e_forensics_matrix``, :4834 the micro-benchmarks).

The CLI (``conformance/cli.py``) and the gates drive the same runners; these functions are the form a test or
another program calls: a config names the fixture suite and the allow-list, every family has its own
``run_<family>_conformance(config, mode) -> (HarnessReport, case reports)``, and the forensics matrix writes one
structured JSONL record per case and mode, optionally restricted to the families of one packet.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..runtime.ledger import ExecutionMode
from .runner import SUITE_PATH, CaseResult, load_suite, structured_log
from .runner_more import FAMILIES, run_family

_HERE = os.path.dirname(os.path.abspath(__file__))

# packet -> fixture families (FT-P2C-005, the kernel packet, owns every family no other packet names)
PACKET_FAMILIES: Dict[str, List[str]] = {
    "FT-P2C-001": ["tensor_meta"], "FT-P2C-002": ["dispatch_key"], "FT-P2C-003": ["op_schema"],
    "FT-P2C-004": ["autograd_scheduler", "scalar_autograd"], "FT-P2C-006": ["serialization"],
    "FT-P2C-007": ["dispatch_key"], "FT-P2C-008": ["nn_state"], "FT-P2C-009": ["optimizer"],
}
PACKET_FAMILIES["FT-P2C-005"] = sorted(f for f in FAMILIES if not any(f in v for v in PACKET_FAMILIES.values()))


def packet_of(family: str) -> str:
    for p, fams in PACKET_FAMILIES.items():
        if family in fams and p != "FT-P2C-007":
            return p
    return "FT-P2C-005"


def mode_label(mode) -> str:
    return ExecutionMode.parse(mode).value


def now_unix_ms() -> int:
    return int(time.time() * 1000)


@dataclass
class HarnessConfig:
    """Where the harness finds its inputs.  ``oracle_root`` is a checkout of the legacy oracle (PyTorch sources)
    if one is present; this build uses the installed ``torch`` as the live oracle instead."""
    oracle_root: str
    fixture_root: str
    allowlist_path: str
    strict_mode: bool = True
    legacy_oracle_python: Optional[str] = None

    @staticmethod
    def default_paths() -> "HarnessConfig":
        return HarnessConfig(oracle_root=os.path.join(_HERE, "legacy_oracle"), fixture_root=_HERE,
                             allowlist_path=os.path.join(_HERE, "HARDENED_DEVIATION_ALLOWLIST_V1.json"))

    @property
    def suite_path(self) -> str:
        return os.path.join(self.fixture_root, os.path.basename(SUITE_PATH))

    def suite(self) -> Dict[str, List[dict]]:
        return load_suite(self.suite_path)


@dataclass(frozen=True)
class HarnessReport:
    suite: str
    oracle_present: bool
    fixture_count: int
    strict_mode: bool
    cases_total: int
    cases_passed: int

    def ok(self) -> bool:
        return self.cases_total == self.cases_passed


@dataclass(frozen=True)
class BenchReport:
    iterations: int
    p50_ns: int
    p95_ns: int
    p99_ns: int
    mean_ns: int

    @staticmethod
    def from_samples(samples_ns: Sequence[int]) -> "BenchReport":
        """Nearest-rank percentiles of the sorted samples."""
        xs = sorted(int(s) for s in samples_ns)
        if not xs:
            return BenchReport(0, 0, 0, 0, 0)

        def pct(p):
            return xs[min(len(xs) - 1, max(0, -(-p * len(xs) // 100) - 1))]
        return BenchReport(len(xs), pct(50), pct(95), pct(99), sum(xs) // len(xs))

    def regression_pct(self, baseline: "BenchReport") -> float:
        """Relative change of the p95 against ``baseline`` in percent (positive = slower)."""
        if baseline.p95_ns == 0:
            return 0.0
        return 100.0 * (self.p95_ns - baseline.p95_ns) / baseline.p95_ns


@dataclass
class E2EForensicsSummary:
    output_path: str
    log_entries: int
    failed_entries: int
    modes: List[ExecutionMode] = field(default_factory=list)


def _oracle_present(config: HarnessConfig) -> bool:
    if os.path.isdir(config.oracle_root):
        return True
    try:
        import torch  # noqa: F401  (the live oracle of the differential checks)
        return True
    except ImportError:
        return False


def run_smoke(config: HarnessConfig) -> HarnessReport:
    """Counts the fixture families and checks that the suite and the allow-list parse; runs no case."""
    suite = config.suite()
    with open(config.allowlist_path) as f:
        json.load(f)
    return HarnessReport("smoke", _oracle_present(config), len(suite), config.strict_mode, 0, 0)


def run_family_conformance(config: HarnessConfig, family: str, mode) -> Tuple[HarnessReport, List[CaseResult]]:
    if family not in FAMILIES:
        raise ValueError(f"unknown fixture family {family!r}")
    rep = run_family(family, ExecutionMode.parse(mode), config.suite())
    return (HarnessReport(family, _oracle_present(config), 1, ExecutionMode.parse(mode) is ExecutionMode.Strict,
                          rep.cases_total, rep.cases_passed), rep.results)


def _named(family: str):
    def run(config: HarnessConfig, mode) -> Tuple[HarnessReport, List[CaseResult]]:
        return run_family_conformance(config, family, mode)
    run.__name__ = f"run_{family}_conformance"
    run.__doc__ = f"Run the ``{family}`` fixture family in ``mode``; returns the summary and one result per case."
    return run


# one entry point per family under the reference's names
_REFERENCE_NAMES = {"scalar_autograd": "scalar", "dispatch_key": "dispatch"}
for _fam in FAMILIES:
    globals()[f"run_{_REFERENCE_NAMES.get(_fam, _fam)}_conformance"] = _named(_fam)


def emit_e2e_forensics_matrix_filtered(config: HarnessConfig, output_path: str, modes: Sequence = (),
                                       packet_filter: Optional[str] = None) -> E2EForensicsSummary:
    """One structured log record per case and mode, written as JSONL.  ``packet_filter`` keeps the families of
    that packet only; an empty ``modes`` means strict and hardened."""
    sel = [ExecutionMode.parse(m) for m in modes] or [ExecutionMode.Strict, ExecutionMode.Hardened]
    if packet_filter is not None and packet_filter not in PACKET_FAMILIES:
        raise ValueError(f"unknown packet {packet_filter!r}")
    fams = sorted(FAMILIES) if packet_filter is None else PACKET_FAMILIES[packet_filter]
    suite = config.suite()
    entries = failed = 0
    os.makedirs(os.path.dirname(os.path.abspath(output_path)) or ".", exist_ok=True)
    with open(output_path, "w") as out:
        for m in sel:
            for fam in fams:
                for r in run_family(fam, m, suite).results:
                    entries += 1
                    failed += not r.passed
                    out.write(json.dumps(structured_log(r, packet=packet_filter or packet_of(fam)), sort_keys=True) + "\n")
    return E2EForensicsSummary(output_path, entries, failed, sel)


def emit_e2e_forensics_matrix(config: HarnessConfig, output_path: str, modes: Sequence = ()) -> E2EForensicsSummary:
    return emit_e2e_forensics_matrix_filtered(config, output_path, modes, None)


def run_scalar_microbench(iterations: int, mode) -> BenchReport:
    """Session creation, ``(x + y) * x`` on the scalar tape and its backward, timed per iteration."""
    from ..session import FrankenTorchSession
    samples = []
    for _ in range(max(1, iterations)):
        t0 = time.perf_counter_ns()
        s = FrankenTorchSession(mode, ledger_dispatch=False)
        x, y = s.variable(2.0, True), s.variable(3.0, True)
        s.backward(s.mul(s.add(x, y), x))
        samples.append(time.perf_counter_ns() - t0)
    return BenchReport.from_samples(samples)


def run_packet_e2e_microbench(config: HarnessConfig, iterations: int, packet_id: str, tmp_dir: Optional[str] = None) -> BenchReport:
    """Time ``emit_e2e_forensics_matrix_filtered`` for one packet (both modes) ``iterations`` times."""
    import tempfile
    samples = []
    with tempfile.TemporaryDirectory(dir=tmp_dir) as d:
        path = os.path.join(d, f"e2e_{packet_id}_{os.getpid()}.jsonl")
        for _ in range(max(1, iterations)):
            t0 = time.perf_counter_ns()
            emit_e2e_forensics_matrix_filtered(config, path, (), packet_id)
            samples.append(time.perf_counter_ns() - t0)
    return BenchReport.from_samples(samples)
