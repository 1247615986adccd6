"""Conformance command-line tools (mirror of the ft-conformance binaries, Appendix D of the
reference survey: ``run_e2e_matrix``, ``run_differential_report``, ``triage_forensics_failures``,
``build_failure_forensics_index``, ``check_reliability_budgets``, ``run_raptorq_durability_pipeline``,
``validate_phase2c_artifacts``, ``run_perf_slos``, ``check_perf_slos``, ``check_benchmark_regression``,
``emit_packet_sidecar``), plus ``emit_packet_contracts`` (per-packet contract table, fixture manifest and
parity report, the counterpart of artifacts/phase2c/FT-P2C-00X/ in the reference).

    python -m frankentorch_b200.conformance.cli run_e2e_matrix --mode both --output e2e.jsonl
    python -m frankentorch_b200.conformance.cli run_differential_report --output diff.json
    python -m frankentorch_b200.conformance.cli triage_forensics_failures --input e2e.jsonl --output triage.json
    python -m frankentorch_b200.conformance.cli check_reliability_budgets --e2e e2e.jsonl --output gate.json
    python -m frankentorch_b200.conformance.cli run_perf_slos --profile smoke --output perf.json
    python -m frankentorch_b200.conformance.cli check_perf_slos --input perf.json
    python -m frankentorch_b200.conformance.cli emit_packet_sidecar <artifact> [--repair-symbols N]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from collections import Counter, defaultdict
from typing import Dict, List

from ..runtime.ledger import ExecutionMode
from . import perf_slo
from .runner import structured_log
from .runner_more import FAMILIES, run_family

PACKETS = {"FT-P2C-001": ["tensor_meta"], "FT-P2C-002": ["dispatch_key"], "FT-P2C-003": ["op_schema"],
           "FT-P2C-004": ["autograd_scheduler", "scalar_autograd"], "FT-P2C-006": ["serialization"],
           "FT-P2C-007": ["dispatch_key"], "FT-P2C-008": ["nn_state"], "FT-P2C-009": ["optimizer"]}
RELIABILITY_POLICY = {"min_cases_per_family": 1, "min_pass_ratio": 1.0, "flake_budget": 0,
                      "required_families": sorted(FAMILIES)}


def _packet_of(family: str) -> str:
    for p, fams in PACKETS.items():
        if family in fams:
            return p
    return "FT-P2C-005"


def _modes(arg: str) -> List[ExecutionMode]:
    return [ExecutionMode.Strict, ExecutionMode.Hardened] if arg == "both" else [ExecutionMode.parse(arg)]


def run_e2e_matrix(args) -> int:
    fams = PACKETS[args.packet] if args.packet else ([args.family] if args.family else sorted(FAMILIES))
    lines, failed = [], 0
    for m in _modes(args.mode):
        for f in fams:
            for r in run_family(f, m).results:
                failed += not r.passed
                lines.append(json.dumps(structured_log(r, packet=_packet_of(f)), sort_keys=True))
    text = "\n".join(lines) + "\n"
    if args.output:
        with open(args.output, "w") as fh:
            fh.write(text)
    if args.print_full_log or not args.output:
        sys.stdout.write(text)
    print(f"e2e matrix: {len(lines)} scenarios, {failed} failed", file=sys.stderr)
    return 1 if failed else 0


def run_differential_report(args) -> int:
    """Differential check against live PyTorch as the oracle: the same random problems are run
    through the session (DAC tape, f64) and through ``torch.autograd`` and compared."""
    import torch

    from ..session import FrankenTorchSession
    checks = []
    ops = [("tanh", {}), ("sigmoid", {}), ("gelu", {}), ("softmax", {"dim": -1}), ("log_softmax", {"dim": -1}),
           ("cumsum", {"dim": 0}), ("exp", {}), ("silu", {}), ("softplus", {})]
    for m in _modes(args.mode):
        for name, kw in ops:
            s = FrankenTorchSession(m, ledger_dispatch=False)
            x = s.randn([4, 5], requires_grad=True)
            y = getattr(s, "tensor_" + name)(x, **kw)
            rep = s.tensor_backward(s.tensor_sum(s.tensor_square(y)))
            xt = s.tensor(x).detach().clone().requires_grad_(True)
            fn = {"gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu,
                  "softplus": torch.nn.functional.softplus}.get(name, getattr(torch, name, None))
            yt = fn(xt, **kw)
            (yt ** 2).sum().backward()
            d_out = float((s.tensor(y) - yt.detach()).abs().max())
            d_grad = float((rep.gradient(x) - xt.grad).abs().max())
            checks.append({"op": name, "mode": m.value, "max_abs_output_diff": d_out, "max_abs_grad_diff": d_grad,
                           "passed": d_out < 1e-12 and d_grad < 1e-10})
    report = {"schema_version": "ft-differential-report-v1", "oracle": f"torch {torch.__version__}",
              "checks": checks, "passed": all(c["passed"] for c in checks)}
    text = json.dumps(report, indent=2)
    if args.output:
        open(args.output, "w").write(text)
    if args.print_full_report or not args.output:
        print(text)
    return 0 if report["passed"] else 1


def _read_jsonl(path: str) -> List[dict]:
    return [json.loads(l) for l in open(path) if l.strip()]


def triage_forensics_failures(args) -> int:
    recs = [r for r in _read_jsonl(args.input) if r["outcome"] != "pass" and (not args.packet or r["packet_id"] == args.packet)]
    buckets: Dict[str, List[dict]] = defaultdict(list)
    for r in recs:
        buckets[f"{r['packet_id']}|{r['reason_code']}"].append(r)
    out = {"schema_version": "ft-triage-v1", "failures": len(recs),
           "buckets": [{"key": k, "count": len(v), "scenarios": [x["scenario_id"] for x in v][:20],
                        "replay": v[0]["replay_command"]} for k, v in sorted(buckets.items())]}
    open(args.output, "w").write(json.dumps(out, indent=2))
    return 0


def build_failure_forensics_index(args) -> int:
    idx = {"schema_version": "ft-forensics-index-v1", "sources": {}}
    for name in ("e2e", "triage", "differential"):
        p = getattr(args, name)
        if p and os.path.exists(p):
            idx["sources"][name] = {"path": p, "bytes": os.path.getsize(p)}
    if args.e2e:
        c = Counter(r["outcome"] for r in _read_jsonl(args.e2e))
        idx["e2e_outcomes"] = dict(c)
    open(args.output, "w").write(json.dumps(idx, indent=2))
    return 0


def check_reliability_budgets(args) -> int:
    policy = json.load(open(args.policy)) if args.policy else RELIABILITY_POLICY
    recs = _read_jsonl(args.e2e)
    per = defaultdict(lambda: [0, 0])
    for r in recs:
        fam = r["scenario_id"].split("/")[0]
        per[fam][0] += 1
        per[fam][1] += r["outcome"] == "pass"
    violations = []
    for fam in policy["required_families"]:
        tot, ok = per.get(fam, [0, 0])
        if tot < policy["min_cases_per_family"]:
            violations.append(f"{fam}: coverage {tot} below floor {policy['min_cases_per_family']}")
        elif ok / tot < policy["min_pass_ratio"]:
            violations.append(f"{fam}: pass ratio {ok}/{tot}")
    out = {"schema_version": "ft-reliability-gate-v1", "passed": not violations, "violations": violations,
           "flake_budget": policy["flake_budget"], "scenarios": len(recs)}
    text = json.dumps(out, indent=2)
    if args.output:
        open(args.output, "w").write(text)
    print(text)
    return 0 if out["passed"] else 1


def run_raptorq_durability_pipeline(args) -> int:
    """Sidecar + decode proof for every artifact file under a root; writes a manifest and a scrub report."""
    from ..serialize import decode_with_sidecar, generate_raptorq_sidecar, hash_bytes
    root = args.root
    manifest, events = [], []
    for dirpath, _, files in sorted(os.walk(root)):
        for f in sorted(files):
            if f.endswith((".sidecar.json", ".proof.json")):
                continue
            p = os.path.join(dirpath, f)
            payload = open(p, "rb").read()
            if not payload or len(payload) > (1 << 20):
                continue
            side, proof = generate_raptorq_sidecar(payload, args.repair_symbols)
            open(p + ".sidecar.json", "w").write(side.to_json())
            open(p + ".proof.json", "w").write(json.dumps(proof.__dict__))
            manifest.append({"artifact": os.path.relpath(p, root), "source_hash": side.source_hash, "k": side.k,
                             "repair_symbols": side.repair_symbols})
            events.append({"artifact": os.path.relpath(p, root), "scrub_status": "ok" if proof.recovered else "failed",
                           "proof_hash": proof.proof_hash})
    out = {"schema_version": "ft-durability-pipeline-v1", "manifest": manifest, "scrub_report": events,
           "passed": all(e["scrub_status"] == "ok" for e in events)}
    print(json.dumps(out, indent=2))
    return 0 if out["passed"] else 1


def emit_packet_sidecar(args) -> int:
    from ..serialize import generate_raptorq_sidecar
    payload = open(args.artifact, "rb").read()
    side, proof = generate_raptorq_sidecar(payload, args.repair_symbols)
    open(args.artifact + ".sidecar.json", "w").write(side.to_json())
    open(args.artifact + ".proof.json", "w").write(json.dumps(proof.__dict__))
    print(f"{args.artifact}: k={side.k} repair={side.repair_symbols} proof={proof.proof_hash}")
    return 0 if proof.recovered else 1


def validate_artifacts(args) -> int:
    """Every ``*.sidecar.json`` under the root must still recover (here: match) its artifact."""
    from ..serialize import hash_bytes
    bad = []
    for dirpath, _, files in os.walk(args.root):
        for f in files:
            if f.endswith(".sidecar.json"):
                art = os.path.join(dirpath, f[: -len(".sidecar.json")])
                side = json.load(open(os.path.join(dirpath, f)))
                if not os.path.exists(art) or hash_bytes(open(art, "rb").read()) != side["source_hash"]:
                    bad.append(art)
    from . import packets
    contract_problems = packets.validate(args.root)
    for sub in ("artifacts/phase2c", "phase2c"):
        if os.path.isdir(os.path.join(args.root, sub)):
            contract_problems += packets.validate(os.path.join(args.root, sub))
    ok = not bad and not contract_problems
    print(json.dumps({"passed": ok, "stale_or_missing": bad, "packet_contract_problems": contract_problems}, indent=2))
    return 0 if ok else 1


def emit_packet_contracts(args) -> int:
    """Write the per-packet contract table, fixture manifest and parity report (both modes are run now)."""
    from . import packets
    written = packets.emit(args.output)
    print(json.dumps({"written": len(written), "root": args.output, "problems": packets.validate(args.output)}, indent=2))
    return 0


def run_perf_slos_cmd(args) -> int:
    rep = perf_slo.run_perf_slos(args.profile, args.iterations, args.warmup_iterations, args.device)
    text = rep.to_json()
    if args.output:
        open(args.output, "w").write(text)
    else:
        print(text)
    if args.baseline and os.path.exists(args.baseline):
        print(json.dumps(perf_slo.check_benchmark_regression(json.load(open(args.baseline)), json.loads(text))))
    return 0


def check_perf_slos_cmd(args) -> int:
    gate = perf_slo.check_perf_slos(json.load(open(args.input)))
    print(json.dumps(gate, indent=2))
    return 0 if gate["passed"] else 1


def check_benchmark_regression_cmd(args) -> int:
    res = perf_slo.check_benchmark_regression(json.load(open(args.baseline)), json.load(open(args.input)), args.threshold_pct)
    text = json.dumps(res, indent=2)
    if args.output:
        open(args.output, "w").write(text)
    print(text)
    return 0 if res["passed"] else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="frankentorch_b200.conformance.cli")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("run_e2e_matrix")
    p.add_argument("--mode", default="both")
    p.add_argument("--packet")
    p.add_argument("--family")
    p.add_argument("--output")
    p.add_argument("--print-full-log", action="store_true")
    p.set_defaults(fn=run_e2e_matrix)
    p = sub.add_parser("run_differential_report")
    p.add_argument("--mode", default="both")
    p.add_argument("--output")
    p.add_argument("--print-full-report", action="store_true")
    p.set_defaults(fn=run_differential_report)
    p = sub.add_parser("triage_forensics_failures")
    p.add_argument("--input", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--packet")
    p.set_defaults(fn=triage_forensics_failures)
    p = sub.add_parser("build_failure_forensics_index")
    p.add_argument("--e2e")
    p.add_argument("--triage")
    p.add_argument("--differential")
    p.add_argument("--output", required=True)
    p.set_defaults(fn=build_failure_forensics_index)
    p = sub.add_parser("check_reliability_budgets")
    p.add_argument("--policy")
    p.add_argument("--e2e", required=True)
    p.add_argument("--output")
    p.set_defaults(fn=check_reliability_budgets)
    p = sub.add_parser("run_raptorq_durability_pipeline")
    p.add_argument("--root", required=True)
    p.add_argument("--repair-symbols", type=int, default=4)
    p.set_defaults(fn=run_raptorq_durability_pipeline)
    p = sub.add_parser("emit_packet_sidecar")
    p.add_argument("artifact")
    p.add_argument("--repair-symbols", type=int, default=4)
    p.set_defaults(fn=emit_packet_sidecar)
    for name in ("validate_artifacts", "validate_phase2c_artifacts"):   # the reference's binary carries the longer name
        p = sub.add_parser(name)
        p.add_argument("root", nargs="?", default=".")
        p.set_defaults(fn=validate_artifacts)
    p = sub.add_parser("emit_packet_contracts")
    p.add_argument("--output", default="artifacts/phase2c")
    p.set_defaults(fn=emit_packet_contracts)
    p = sub.add_parser("run_perf_slos")
    p.add_argument("--profile", default="smoke", choices=["smoke", "full"])
    p.add_argument("--iterations", type=int, default=10)
    p.add_argument("--warmup-iterations", type=int, default=1)
    p.add_argument("--device", default="cpu")
    p.add_argument("--output")
    p.add_argument("--baseline")
    p.set_defaults(fn=run_perf_slos_cmd)
    p = sub.add_parser("check_perf_slos")
    p.add_argument("--input", required=True)
    p.set_defaults(fn=check_perf_slos_cmd)
    p = sub.add_parser("check_benchmark_regression")
    p.add_argument("--baseline", required=True)
    p.add_argument("--input", required=True)
    p.add_argument("--threshold-pct", type=float, default=7.0)
    p.add_argument("--output")
    p.set_defaults(fn=check_benchmark_regression_cmd)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
