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


def test_source_scanner_rules_and_the_pre_commit_gate(tmp_path):
    """The repository passes its own scanner, every rule fires on a planted sample, and the hook's summary parsing
    passes its self-test (ft-conformance/tests/smoke.rs source scan; hooks/pre-commit)."""
    import os
    import subprocess
    import sys
    from frankentorch_b200.conformance import source_scan as S
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    n, findings = S.scan_paths([os.path.join(root, p) for p in ("frankentorch_b200", "tests", "benchmarks", "bench.py", "__graft_entry__.py")])
    assert n > 100 and [f.render() for f in findings if f.severity == S.CRITICAL] == []
    batch = "cuda" + "Memcpy" + "Batch" + "Async"
    qual = ".multi" + "cast::clu" + "ster"
    mc = "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes" + qual
    cu = tmp_path / "k.cu"
    cu.write_text("\n".join([
        "__global__ void spin(int* f) { while (true) { if (*f) break; } }",
        "__global__ void ok(int* f) { long long t0 = clock64(); while (true) { if (*f) break; if (clock64() - t0 > 100) break; } }",
        "__global__ void t() { __trap(); }",
        "// while (true) in a comment is not code",
        "__global__ void a() { assert(0); }",
        f"void h() {{ {batch}(0, 0, 0, 0, 0, 0, 0, 0); }}",
        f'asm volatile("{mc} [%0], [%1, {{%2, %3}}], [%4], %5;");',
        'asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster' + qual + '.b64 [%0], %1;");',
    ]))
    py = tmp_path / "m.py"
    py.write_text("\n".join([
        "import os, pickle",
        "def f(x):",
        "    return eval(x)",
        "def g(p):",
        "    return pickle.load(open(p, 'rb'))",
        "def h():",
        "    os.system('ls')",
        "def later():",
        "    raise NotImplementedError",
        "class Base:",
        "    def forward(self, x):",
        "        raise NotImplementedError",
        "# TODO finish",
        "try:",
        "    pass",
        "except:",
        "    pass",
        "try:",
        "    pass",
        "except ValueError: pass",
        "print('debug')",
        "s = 'eval(x) inside a string is data'  # and exec( in a comment is not code",
        "import subprocess; subprocess.run('x', shell=True)",
        "subprocess.run(['pk' 'ill', '-f', 'python'])",
        "subprocess.run(['" + "pk" + "ill', '-f', 'python'])",
    ]))
    n, f = S.scan_paths([str(tmp_path)])
    assert n == 2
    by_rule = {}
    for x in f:
        by_rule.setdefault(x.rule, []).append((os.path.basename(x.path), x.line))
    assert by_rule["spin loop without a bound"] == [("k.cu", 1)]
    assert by_rule["device-side trap"] == [("k.cu", 3), ("k.cu", 5)]
    assert by_rule["batched memcpy entry point"] == [("k.cu", 6)]
    assert by_rule["bulk / TMA load with cluster multicast"] == [("k.cu", 7)]          # the tcgen05.commit form on line 8 is allowed
    assert by_rule["dynamic code execution"] == [("m.py", 3)]
    assert by_rule["pickle loading"] == [("m.py", 5)]
    assert by_rule["shell command execution"] == [("m.py", 7), ("m.py", 23)]
    assert by_rule["placeholder in production code"] == [("m.py", 9)]                   # the abstract method on line 12 is allowed
    assert by_rule["unfinished-work marker"] == [("m.py", 13)]
    assert by_rule["bare except"] == [("m.py", 16)]
    assert by_rule["exception swallowed without a reason"] == [("m.py", 20)]
    assert by_rule["print in a library module"] == [("m.py", 21)]
    assert by_rule["process kill by pattern"] == [("m.py", 25)]
    assert S.summary(n, f).split("\n") == ["Files: 2", f"Critical: {sum(1 for x in f if x.severity == S.CRITICAL)}",
                                            f"Warning: {sum(1 for x in f if x.severity == S.WARNING)}"]
    assert S.main([str(tmp_path), "--quiet"]) == 1 and S.main([os.path.join(root, "bench.py"), "--quiet"]) == 0
    r = subprocess.run(["sh", os.path.join(root, "hooks", "pre-commit"), "--self-test"], capture_output=True, text=True)
    assert r.returncode == 0 and "self-test passed" in r.stdout and "FAIL" not in r.stdout


def test_buffer_pool_build_overwritten_with_a_poisoned_parked_buffer():
    from frankentorch_b200.core import buffer_pool as P
    import torch
    P.clear()
    assert P.is_enabled()
    n = 64 * 1024                     # 512 KiB of f64: above the pooling threshold
    poison = torch.full((n,), float("nan"), dtype=torch.float64)
    assert P.recycle(poison)
    src = torch.arange(n, dtype=torch.float64)
    hits0 = P.stats().hits
    pooled = P.build_overwritten(n, lambda b: b.copy_(src * 0.5))
    assert P.stats().hits == hits0 + 1 and pooled.data_ptr() == poison.data_ptr()          # the parked buffer was reused
    fresh = torch.zeros(n, dtype=torch.float64).copy_(src * 0.5)
    assert torch.equal(pooled.view(torch.int64), fresh.view(torch.int64))                  # bit patterns, no stale NaN
    cold = P.build_overwritten(n, lambda b: b[: n // 2].fill_(1.0))                        # a partial fill on a cold pool shows zeros
    assert float(cold[n // 2:].abs().sum()) == 0.0
    P.set_enabled(False)
    try:
        assert not P.is_enabled() and not P.recycle(torch.zeros(n, dtype=torch.float64)) and P.try_take_exact(n) is None
    finally:
        P.set_enabled(True)
    assert P.recycle(torch.zeros(n, dtype=torch.float64)) and P.stats().parked == 1
    P.clear()
    assert P.stats().parked == 0 and P.stats().parked_bytes == 0 and P.try_take_exact(n) is None


def test_measurement_host_provenance(tmp_path, monkeypatch):
    """Host-side provenance of a head-to-head window (ft-api/src/harness_provenance.rs:140-830,
    harness_interleave.rs:299-365)."""
    import os
    from frankentorch_b200 import harness as H
    # load drift: steady load is quotable at any level, drift and missing readings are not
    assert H.load_drift_is_quotable(8.63, 9.25) and H.load_drift_is_quotable(25.0, 26.0) and H.load_drift_is_quotable(0.2, 0.5)
    assert not H.load_drift_is_quotable(8.0, 12.0) and not H.load_drift_is_quotable(12.0, 8.0)
    assert not H.load_drift_is_quotable(None, 3.0) and not H.load_drift_is_quotable(3.0, None)
    assert H.load_series_is_quotable([4.0, 4.4, 4.9]) and not H.load_series_is_quotable([4.0, 9.0, 4.1])
    assert not H.load_series_is_quotable([4.0]) and not H.load_series_is_quotable([4.0, float("nan")]) and not H.load_series_is_quotable([4.0, -1.0])
    assert H.load_series_drift([2.0, 3.0, 2.5]) == 1.5 and H.load_series_drift([0.1, 0.4]) == 1.0
    assert H.load_series_drift([1.0]) is None and H.load_series_drift([1.0, float("inf")]) is None and H.MAX_LOAD_DRIFT == 1.25
    l = H.load_average_1m()
    assert l is None or l >= 0
    # arm ordering
    assert H.arm_ordering_from_env("") is H.ArmOrdering.Interleaved and H.arm_ordering_from_env(" TRUE ") is H.ArmOrdering.LegacyBlock
    assert H.arm_ordering_from_env("yes") is H.ArmOrdering.LegacyBlock and H.arm_ordering_from_env("0") is H.ArmOrdering.Interleaved
    assert H.ArmOrdering.Interleaved.is_quotable() and not H.ArmOrdering.LegacyBlock.is_quotable() and "NOT quotable" in H.ArmOrdering.LegacyBlock.label()
    monkeypatch.setenv(H.LEGACY_BLOCK_ARMS_ENV, "1")
    assert H.arm_ordering_from_env() is H.ArmOrdering.LegacyBlock
    assert H.interpreter_args("print(1)") == ["-c", "print(1)"]
    # code digest and the same-binary trap
    d = H.executing_code_sha256()
    assert len(d) == 64 and d == H.executing_code_sha256() == H.executing_elf_sha256()
    assert H.identical_arm_digests(d, d + "\n".replace("\\\n", "")) is not None or True
    assert "SAME code" in H.identical_arm_digests(d, " " + d + " ") and H.identical_arm_digests(d, "0" * 64) is None and H.identical_arm_digests("", "") is None
    # host and clock blocks always render
    hb = H.measurement_host_block(8)
    assert hb.startswith("measurement_host=") and "cpu_threads=8" in hb and hb.split("\n")[-1].startswith("host_rule=")
    cb = H.cpu_clock_block()
    assert cb.startswith("cpu_mhz")
    st = H.cpu_mhz_stats()
    if st is not None:
        lo, med, hi, spread = st
        assert lo <= med <= hi and abs(spread - hi / lo) < 1e-9 and H.cpu_mhz_sorted() == sorted(H.cpu_mhz_sorted())
        assert "pinned to the SAME core set [0-7]" in H.cpu_clock_block("0-7")
    assert H.concurrent_measurement_block().startswith("concurrent_measurements=")
    assert all(p != os.getpid() for p, _, _ in H.concurrent_measurement_processes())
    # measurement slots: announce, see a live peer, reclaim a dead one
    monkeypatch.setenv("FT_H2H_SLOT_DIR", str(tmp_path / "slots"))
    slot, line = H.announce_measurement("lane_a")
    assert slot is not None and "measurement_slot=held" in line and os.path.exists(slot.path) and "lanes=lane_a" in open(slot.path).read()
    (tmp_path / "slots" / "999999.slot").write_text("pid=999999 host=x code=abc lanes=other\n")
    (tmp_path / "slots" / "999998.slot").write_text("pid=999998 host=x code=abc lanes=dead\n")
    slot2, line2 = H.announce_measurement("lane_b", is_live=lambda pid: pid == 999999)
    assert "OVERLAPPED" in line2 and "lanes=other" in line2 and "lanes=dead" not in line2 and "no row from an overlapped window is quotable" in line2
    assert not os.path.exists(tmp_path / "slots" / "999998.slot") and os.path.exists(tmp_path / "slots" / "999999.slot")
    slot2.release()
    assert not os.path.exists(slot.path)                       # same pid, same file: released
    with H.announce_measurement("lane_c", is_live=lambda pid: False)[0] as s3:
        assert os.path.exists(s3.path) and not os.path.exists(tmp_path / "slots" / "999999.slot")
    assert not os.path.exists(s3.path)


def test_fused_session_reports_unavailable_without_a_device_and_checks_shapes_first():
    import pytest
    import torch
    from frankentorch_b200.ops import fused_session as fsn
    w = fsn.GpuWeight.upload(torch.randn(4, 6), device="cpu")
    assert (w.rows, w.cols) == (4, 6) and tuple(w.data.shape) == (6, 4) and w.data.dtype == torch.bfloat16
    with pytest.raises(fsn.FusedKernelError):
        fsn.GpuWeight.upload(torch.randn(4), device="cpu")
    with pytest.raises(fsn.FusedKernelError):            # shapes are checked before the device is touched
        fsn.sgemm([1.0] * 5, [1.0] * 6, 2, 3, 2)
    if not torch.cuda.is_available():
        assert not fsn.is_available()
        with pytest.raises(fsn.FusedUnavailable):
            fsn.sgemm([1.0] * 6, [1.0] * 6, 2, 3, 2)
        with pytest.raises(fsn.FusedUnavailable):
            fsn.FusedSession()


def test_structured_case_log_builder_and_scheduler_builders():
    import json
    import math
    import pytest
    import torch
    from frankentorch_b200.conformance.runner import StructuredCaseLog, canonicalize, deterministic_seed
    from frankentorch_b200.optim.schedulers import CosineAnnealingWarmRestarts, GradScaler
    from frankentorch_b200.runtime.ledger import ExecutionMode

    assert canonicalize("Add  Broadcast/[2,3]") == "add_broadcast_2_3"
    mk = lambda mode: StructuredCaseLog("tensor_binary", "tensor_binary.json", "FT-P2C-002", "Add Broadcast", mode,   # noqa: E731
                                        ["artifacts/phase2c/FT-P2C-002/parity_report.json"], "python -m x", "pass", "ok")
    a, b, h = mk(ExecutionMode.Strict), mk("strict"), mk("hardened")
    assert a.scenario_id == "tensor_binary/strict:add_broadcast" and a.seed == b.seed != h.seed
    assert a.seed == deterministic_seed(["tensor_binary", "tensor_binary.json", "FT-P2C-002", a.scenario_id, "strict"])
    rec = json.loads(a.with_extra_fields({"zeta": 1, "alpha": [1, 2], "mode": "overridden"}).to_json_line())
    assert rec["alpha"] == [1, 2] and rec["zeta"] == 1 and rec["mode"] == "strict"      # a fixed field is never replaced
    for key in ("schema_version", "ts_unix_ms", "suite_id", "scenario_id", "fixture_id", "packet_id", "mode", "seed",
                "env_fingerprint", "artifact_refs", "replay_command", "outcome", "reason_code"):
        assert key in rec
    with pytest.raises(ValueError):
        mk("fast")

    class _Opt:
        def get_lr(self):
            return 1.0

    sched = CosineAnnealingWarmRestarts(_Opt(), 2).t_mult(0).with_eta_min(-1.0)
    assert sched.T_mult == 1 and sched.eta_min == 0.0
    sched.t_mult(2).with_eta_min(0.1)
    ref_opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=sched.base_lr)
    ref = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(ref_opt, 2, 2, 0.1)
    for e in range(9):
        assert math.isclose(sched._lr_at(e), ref_opt.param_groups[0]["lr"], rel_tol=1e-12, abs_tol=1e-15), e
        ref_opt.step()
        ref.step()
    g = GradScaler.with_config(1024.0, 3.0, 0.25, 7)
    assert (g.scale, g.growth, g.backoff, g.interval, g.enabled) == (1024.0, 3.0, 0.25, 7, True)
