"""The reliability gate topology, runnable on a CPU-only machine:

    python -m frankentorch_b200.conformance.gates [--only G2,G4] [--workdir DIR] [--json report.json]

The reference wires eight gates into its CI workflow
(.github/workflows/phase2c_reliability_gates.yml:48-240): G1 format + lint, G2 workspace tests,
G3 differential report, G4 fuzz corpus + e2e matrix + triage + reliability budgets, G5
microbenchmark, G6 artifact validator, G7 durability pipeline, G8 a manual readiness sign-off.
G1-G7 have the counterparts below; each is a command that exits non-zero on failure, run in
order, and the run stops at the first failing gate (G8 stays a human decision and is reported
as such).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path
from typing import Callable, Dict, List, Tuple

ROOT = Path(__file__).resolve().parent.parent.parent
PY = sys.executable


def _run(cmd: List[str], env=None) -> Tuple[int, str]:
    p = subprocess.run(cmd, cwd=str(ROOT), capture_output=True, text=True, env=env)
    return p.returncode, (p.stdout + p.stderr)[-4000:]


def _cli(*args: str) -> Tuple[int, str]:
    return _run([PY, "-m", "frankentorch_b200.conformance.cli", *args])


def g1_static(work: Path):
    """Byte-compile every module, build both native libraries for sm_100a / the host, scan the sources."""
    rc, out = _run([PY, "-m", "compileall", "-q", "frankentorch_b200", "bench.py", "__graft_entry__.py"])
    if rc:
        return rc, out
    rc, out = _run([PY, "-c", "import __graft_entry__ as g; g.build()"])
    if rc:
        return rc, out
    rc, out = _run([PY, "-m", "frankentorch_b200.conformance.source_scan"])
    if rc:
        return rc, out
    rc, out = _run(["sh", "hooks/pre-commit", "--self-test"])
    if rc:
        return rc, out
    return _run([PY, "-m", "pytest", "-q", "tests/test_metamorphic.py", "-k", "kernels or spin or multicast or "
                 "placeholders or closed_call"])


def g2_tests(work: Path):
    return _run([PY, "-m", "pytest", "-x", "-q", "-m", "not gpu", "tests"])


def g3_differential(work: Path):
    return _cli("run_differential_report", "--mode", "both", "--output", str(work / "differential.json"))


def g4_fuzz_e2e_budgets(work: Path):
    rc, out = _run([PY, "-m", "pytest", "-q", "tests/test_properties.py"])
    if rc:
        return rc, out
    e2e, tri = str(work / "e2e.jsonl"), str(work / "triage.json")
    for args in (("run_e2e_matrix", "--mode", "both", "--output", e2e),
                 ("triage_forensics_failures", "--input", e2e, "--output", tri),
                 ("build_failure_forensics_index", "--e2e", e2e, "--triage", tri, "--output", str(work / "index.json"))):
        rc, out = _cli(*args)
        if rc:
            return rc, out
    policy = work / "policy.json"
    policy.write_text(json.dumps({"min_cases_per_family": 1, "min_pass_ratio": 1.0, "flake_budget": 0}))
    return _cli("check_reliability_budgets", "--policy", str(policy), "--e2e", e2e)


def g5_microbench(work: Path):
    out = str(work / "perf.json")
    rc, log = _cli("run_perf_slos", "--profile", "smoke", "--iterations", "5", "--output", out)
    if rc:
        return rc, log
    return _cli("check_perf_slos", "--input", out)


def g6_artifacts(work: Path):
    root = work / "artifacts"
    root.mkdir(exist_ok=True)
    src = ROOT / "frankentorch_b200" / "conformance"
    for name in ("golden_suite.json", "HARDENED_DEVIATION_ALLOWLIST_V1.json"):
        (root / name).write_bytes((src / name).read_bytes())
    rc, log = _cli("run_raptorq_durability_pipeline", "--root", str(root))
    if rc:
        return rc, log
    return _cli("validate_phase2c_artifacts", str(root))


def g7_durability(work: Path):
    root = work / "durability"
    root.mkdir(exist_ok=True)
    (root / "state.bin").write_bytes(os.urandom(20000))
    rc, log = _cli("run_raptorq_durability_pipeline", "--root", str(root), "--repair-symbols", "6")
    if rc:
        return rc, log
    rc, log = _cli("validate_artifacts", str(root))
    if rc:
        return rc, log
    (root / "state.bin").write_bytes(b"tampered")
    rc2, log2 = _cli("validate_artifacts", str(root))
    return (0, log) if rc2 != 0 else (1, "a tampered artifact passed validation\n" + log2)


GATES: Dict[str, Tuple[str, Callable]] = {
    "G1": ("static checks: compile, build, source scan", g1_static),
    "G2": ("test suite (CPU)", g2_tests),
    "G3": ("differential report against live PyTorch", g3_differential),
    "G4": ("property / fuzz tier, e2e forensics matrix, triage, reliability budgets", g4_fuzz_e2e_budgets),
    "G5": ("microbenchmark and perf SLO gate", g5_microbench),
    "G6": ("artifact validator", g6_artifacts),
    "G7": ("durability pipeline (sidecar, proof, tamper detection)", g7_durability),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--only", default="", help="comma-separated gate ids (default: all, in order)")
    ap.add_argument("--workdir", default="")
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    want = [g.strip().upper() for g in args.only.split(",") if g.strip()] or list(GATES)
    unknown = [g for g in want if g not in GATES]
    if unknown:
        ap.error(f"unknown gate(s) {unknown}; have {list(GATES)}")
    work = Path(args.workdir or tempfile.mkdtemp(prefix="ft_gates_"))
    work.mkdir(parents=True, exist_ok=True)
    report, failed = [], None
    for gid in want:
        title, fn = GATES[gid]
        t0 = time.time()
        rc, log = fn(work)
        rec = {"gate": gid, "title": title, "passed": rc == 0, "seconds": round(time.time() - t0, 2)}
        if rc:
            rec["log_tail"] = log[-1500:]
        report.append(rec)
        print(f"{gid} {'PASS' if rc == 0 else 'FAIL'}  {title}  ({rec['seconds']} s)")
        if rc:
            print(log[-1500:])
            failed = gid
            break
    report.append({"gate": "G8", "title": "readiness sign-off", "passed": None, "note": "manual decision, not automated"})
    if args.json:
        Path(args.json).write_text(json.dumps({"schema": "ft-gates-v1", "gates": report}, indent=1))
    return 0 if failed is None else 1


if __name__ == "__main__":
    sys.exit(main())
