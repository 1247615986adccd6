"""Conformance tooling: forensics JSONL schema, gates, perf SLO report, durability pipeline."""
import json
import os

from frankentorch_b200.conformance import cli, perf_slo


def test_e2e_matrix_triage_and_reliability_gate(tmp_path):
    e2e = str(tmp_path / "e2e.jsonl")
    assert cli.main(["run_e2e_matrix", "--mode", "both", "--packet", "FT-P2C-004", "--output", e2e]) == 0
    recs = [json.loads(l) for l in open(e2e)]
    required = {"schema_version", "ts_unix_ms", "suite_id", "scenario_id", "fixture_id", "packet_id", "mode", "seed",
                "env_fingerprint", "artifact_refs", "replay_command", "outcome", "reason_code"}
    assert recs and all(required <= set(r) for r in recs)
    assert {r["mode"] for r in recs} == {"strict", "hardened"} and all(r["schema_version"] == "ft-conformance-log-v1" for r in recs)
    tri = str(tmp_path / "triage.json")
    assert cli.main(["triage_forensics_failures", "--input", e2e, "--output", tri]) == 0
    assert json.load(open(tri))["failures"] == 0
    idx = str(tmp_path / "index.json")
    assert cli.main(["build_failure_forensics_index", "--e2e", e2e, "--triage", tri, "--output", idx]) == 0
    pol = str(tmp_path / "policy.json")
    json.dump({"min_cases_per_family": 1, "min_pass_ratio": 1.0, "flake_budget": 0,
               "required_families": ["autograd_scheduler", "scalar_autograd"]}, open(pol, "w"))
    assert cli.main(["check_reliability_budgets", "--policy", pol, "--e2e", e2e]) == 0
    json.dump({"min_cases_per_family": 1, "min_pass_ratio": 1.0, "flake_budget": 0, "required_families": ["nn_state"]}, open(pol, "w"))
    assert cli.main(["check_reliability_budgets", "--policy", pol, "--e2e", e2e]) == 1    # coverage floor violated


def test_differential_report_against_live_torch(tmp_path):
    out = str(tmp_path / "diff.json")
    assert cli.main(["run_differential_report", "--mode", "both", "--output", out]) == 0
    rep = json.load(open(out))
    assert rep["passed"] and len(rep["checks"]) == 18


def test_perf_slo_report_and_gates(tmp_path):
    assert perf_slo.percentile([5.0, 1.0, 3.0, 2.0, 4.0], 50) == 3.0
    assert perf_slo.percentile([1.0, 2.0], 99) == 2.0
    out = str(tmp_path / "perf.json")
    assert cli.main(["run_perf_slos", "--profile", "smoke", "--iterations", "3", "--output", out]) == 0
    rep = json.load(open(out))
    assert rep["schema_version"] == "ft-perf-slo-report-v1" and rep["workloads"]["checkpoint"]["mb_per_s"] > 0
    assert cli.main(["check_perf_slos", "--input", out]) == 0
    worse = json.loads(json.dumps(rep))
    worse["workloads"]["matmul"]["p99"] *= 2
    w = str(tmp_path / "worse.json")
    json.dump(worse, open(w, "w"))
    assert cli.main(["check_benchmark_regression", "--baseline", out, "--input", w]) == 1
    assert cli.main(["check_benchmark_regression", "--baseline", out, "--input", out]) == 0


def test_durability_pipeline_and_validator(tmp_path):
    root = tmp_path / "artifacts"
    root.mkdir()
    (root / "contract.md").write_text("packet contract table\n" * 40)
    (root / "golden.json").write_text(json.dumps({"a": list(range(200))}))
    assert cli.main(["run_raptorq_durability_pipeline", "--root", str(root)]) == 0
    assert os.path.exists(root / "golden.json.sidecar.json") and os.path.exists(root / "golden.json.proof.json")
    assert cli.main(["validate_artifacts", str(root)]) == 0
    (root / "golden.json").write_text("tampered")
    assert cli.main(["validate_artifacts", str(root)]) == 1


def test_packet_contract_artifacts_are_emitted_and_validated(tmp_path):
    """Each packet gets a contract table, a manifest pinning its golden cases and an all-pass parity report; the
    validator notices a stale manifest and a missing contract row."""
    import json

    from frankentorch_b200.conformance import packets
    root = str(tmp_path / "phase2c")
    written = packets.emit(root)
    assert len(written) == 3 * len(packets.CONTRACTS)
    assert packets.validate(root) == []
    rep = json.load(open(f"{root}/FT-P2C-004/parity_report.json"))
    assert rep["passed"] and rep["modes"]["strict"]["cases"] == rep["modes"]["strict"]["passed"] > 0
    man_path = f"{root}/FT-P2C-001/fixture_manifest.json"
    man = json.load(open(man_path))
    man["fixtures"][0]["sha256"] = "0" * 64
    json.dump(man, open(man_path, "w"))
    table = f"{root}/FT-P2C-009/contract_table.md"
    open(table, "w").write(open(table).read().replace("`OPTIM-002`", "`OPTIM-00X`"))
    problems = packets.validate(root)
    assert any("FT-P2C-001" in p and "changed" in p for p in problems)
    assert any("FT-P2C-009" in p and "OPTIM-002" in p for p in problems)
    # the committed artifacts are current
    here = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    assert packets.validate(__import__("os").path.join(here, "artifacts", "phase2c")) == []


def test_conformance_harness_library_entry_points(tmp_path):
    """``HarnessConfig`` / ``HarnessReport`` / per-family runners / forensics matrix / micro-benchmarks
    (ft-conformance/src/lib.rs:38, :580, :1685, :1777-2680, :2682, :4834)."""
    import json
    from frankentorch_b200.conformance import harness as H
    from frankentorch_b200.conformance.runner_more import FAMILIES
    cfg = H.HarnessConfig.default_paths()
    smoke = H.run_smoke(cfg)
    assert smoke.suite == "smoke" and smoke.fixture_count == len(FAMILIES) and smoke.oracle_present and smoke.cases_total == 0
    for fam in FAMILIES:
        assert callable(getattr(H, f"run_{ {'scalar_autograd': 'scalar', 'dispatch_key': 'dispatch'}.get(fam, fam)}_conformance"))
    rep, cases = H.run_dispatch_conformance(cfg, "hardened")
    assert rep.ok() and rep.cases_total == len(cases) > 0 and not rep.strict_mode and all(c.mode == "hardened" for c in cases)
    rep, _ = H.run_tensor_sort_conformance(cfg, "strict")
    assert rep.ok() and rep.strict_mode and rep.suite == "tensor_sort"
    with __import__("pytest").raises(ValueError):
        H.run_family_conformance(cfg, "no_such_family", "strict")
    out = str(tmp_path / "sub" / "e2e.jsonl")
    summ = H.emit_e2e_forensics_matrix_filtered(cfg, out, (), "FT-P2C-004")
    lines = [json.loads(l) for l in open(out)]
    assert summ.log_entries == len(lines) > 0 and summ.failed_entries == 0 and [m.value for m in summ.modes] == ["strict", "hardened"]
    assert {l["packet_id"] for l in lines} == {"FT-P2C-004"} and {l["mode"] for l in lines} == {"strict", "hardened"}
    assert {l["scenario_id"].split("/")[0] for l in lines} == {"autograd_scheduler", "scalar_autograd"}
    one = H.emit_e2e_forensics_matrix_filtered(cfg, out, ["strict"], "FT-P2C-003")
    assert one.log_entries * 1 == sum(1 for _ in open(out)) and [m.value for m in one.modes] == ["strict"]
    with __import__("pytest").raises(ValueError):
        H.emit_e2e_forensics_matrix_filtered(cfg, out, (), "FT-P2C-042")
    assert sorted(sum(H.PACKET_FAMILIES.values(), [])) == sorted(list(FAMILIES) + ["dispatch_key"])     # every family has a packet
    b = H.BenchReport.from_samples([5, 1, 3, 2, 4, 100])
    assert (b.iterations, b.p50_ns, b.p95_ns, b.p99_ns, b.mean_ns) == (6, 3, 100, 100, 19)
    assert H.BenchReport.from_samples([]).iterations == 0
    assert H.BenchReport(1, 10, 110, 0, 0).regression_pct(H.BenchReport(1, 10, 100, 0, 0)) == 10.0
    mb = H.run_scalar_microbench(5, "strict")
    assert mb.iterations == 5 and 0 < mb.p50_ns <= mb.p95_ns <= mb.p99_ns
    pb = H.run_packet_e2e_microbench(cfg, 1, "FT-P2C-003", tmp_dir=str(tmp_path))
    assert pb.iterations == 1 and pb.p50_ns > 0
    assert H.mode_label("Strict") == "strict" and H.now_unix_ms() > 1_600_000_000_000
