"""Configuration, metrics and profiling helpers (CPU)."""
import json

import pytest
import torch

from frankentorch_b200.runtime.ledger import EvidenceKind, EvidenceLedger
from frankentorch_b200.utils import config as cfgmod
from frankentorch_b200.utils import metrics, profiling


def test_percentile_is_nearest_rank():
    xs = [15.0, 20.0, 35.0, 40.0, 50.0]
    # nearest rank: ceil(p/100 * n)
    assert metrics.percentile_nearest_rank(xs, 30) == 20.0
    assert metrics.percentile_nearest_rank(xs, 40) == 20.0
    assert metrics.percentile_nearest_rank(xs, 50) == 35.0
    assert metrics.percentile_nearest_rank(xs, 100) == 50.0
    assert metrics.percentile_nearest_rank([7.0], 99) == 7.0
    with pytest.raises(ValueError):
        metrics.percentile_nearest_rank([], 50)
    s = metrics.summarize(list(range(1, 101)))
    assert (s["p50"], s["p95"], s["p99"], s["min"], s["max"]) == (50.0, 95.0, 99.0, 1.0, 100.0)


def test_roofline_fraction_picks_the_slowest_bound():
    pk = metrics.Peaks(hbm_gbs=1000.0, bf16_tflops=100.0, bf16_tflops_sustained=80.0, nvlink_gbs=100.0)
    r = metrics.roofline_fraction(us=200.0, flops=1e10, hbm_bytes=1e8, nvlink_bytes=1e6, peaks=pk)
    # 1e10 / 1e14 = 100 us; 1e8 / 1e12 = 100 us... flops first on a tie
    assert r["bound_us"] == pytest.approx(100.0) and r["fraction"] == pytest.approx(0.5)
    r = metrics.roofline_fraction(us=50.0, nvlink_bytes=4e6, peaks=pk)
    assert r["limiter"] == "nvlink" and r["fraction"] == pytest.approx(0.8)
    r = metrics.roofline_fraction(us=125.0, flops=1e10, peaks=pk, sustained=True)
    assert r["fraction"] == pytest.approx(1.0)


def test_load_peaks_reads_measured_file_and_falls_back(tmp_path):
    f = tmp_path / "peaks.json"
    f.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1300.0}))
    pk = metrics.load_peaks(str(f))
    assert pk.source == "measured" and pk.hbm_gbs == 6000.0 and pk.bf16_tflops_sustained == 1300.0
    assert metrics.load_peaks(str(tmp_path / "missing.json")) is metrics.FALLBACK_PEAKS


def test_gpt_step_flops_matches_hand_count():
    # one layer, d = 4, ff = 8, vocab = 16, seq = 2, one token, dense attention
    per_tok = (2 * 4 * 12 + 2 * 4 * 4 + 4 * 4 * 8) + 2 * 4 * 16
    attn = 4 * 2 * 4
    assert metrics.gpt_step_flops(1, 4, 8, 16, 2, 1, causal=False) == 3.0 * (per_tok + attn)


def test_run_config_round_trip_and_validation():
    c = cfgmod.RunConfig()
    c.model.n_expert, c.parallel.layout, c.parallel.world = 8, "ep", 8
    c.validate()
    again = cfgmod.RunConfig.from_json(c.to_json())
    assert again == c and again.to_json() == c.to_json()
    with pytest.raises(ValueError):
        cfgmod.RunConfig.from_dict({"model": {"n_heads": 3}})
    with pytest.raises(ValueError):
        cfgmod.RunConfig.from_dict({"bogus": 1})
    bad = cfgmod.RunConfig()
    bad.model.n_head = 7
    with pytest.raises(ValueError):
        bad.validate()
    tp = cfgmod.RunConfig()
    tp.parallel.layout, tp.parallel.world = "tp", 5
    with pytest.raises(ValueError):
        tp.validate()


def test_env_switches_parse_once_and_echo_to_the_ledger(monkeypatch):
    cfgmod.reset_flags()
    monkeypatch.setenv("FT_COMM_CTAS", "12")
    monkeypatch.setenv("FT_MODE", "hardened")
    monkeypatch.setenv("FT_NVTX", "1")
    assert cfgmod.env_flag("FT_COMM_CTAS") == 12 and cfgmod.env_flag("FT_NVTX") is True
    monkeypatch.setenv("FT_COMM_CTAS", "99")          # read once per process
    assert cfgmod.env_flag("FT_COMM_CTAS") == 12
    c = cfgmod.RunConfig().with_env_overrides()
    assert c.mode == "hardened" and c.parallel.comm_ctas == 12
    with pytest.raises(KeyError):
        cfgmod.env_flag("FT_NOT_A_SWITCH")
    led = EvidenceLedger()
    cfgmod.echo_to_ledger(led, c)
    kinds = [e.kind for e in led.entries()]
    assert kinds == [EvidenceKind.Policy, EvidenceKind.Policy]
    assert led[0].summary.startswith("run_config {") and '"FT_COMM_CTAS":12' in led[1].summary
    cfgmod.set_flag("FT_COMM_CTAS", 8)
    assert cfgmod.env_flag("FT_COMM_CTAS") == 8
    cfgmod.reset_flags()
    monkeypatch.setenv("FT_GEMM_PAIR_COST", "abc")
    with pytest.raises(ValueError):
        cfgmod.env_flag("FT_GEMM_PAIR_COST")
    cfgmod.reset_flags()


def test_session_mode_follows_ft_mode(monkeypatch):
    from frankentorch_b200.runtime.ledger import ExecutionMode
    from frankentorch_b200.session import FrankenTorchSession
    cfgmod.reset_flags()
    monkeypatch.setenv("FT_MODE", "hardened")
    assert FrankenTorchSession().runtime.mode == ExecutionMode.Hardened
    assert FrankenTorchSession(ExecutionMode.Strict).runtime.mode == ExecutionMode.Strict
    cfgmod.reset_flags()


def test_tape_ranges_wrap_every_backward_rule():
    import contextlib
    from frankentorch_b200.session import FrankenTorchSession
    s = FrankenTorchSession()
    seen = []

    @contextlib.contextmanager
    def rec(name):
        seen.append(name)
        yield

    assert profiling.install_tape_ranges(s.tensor_tape, enabled=True, range_fn=rec)
    x = s.tensor_variable([1.0, 2.0, 3.0], [3], requires_grad=True)
    y = s.tensor_sum(s.tensor_mul(x, x))
    s.tensor_backward(y)
    assert len(seen) == 2 and all(n.startswith("bwd:") for n in seen)
    assert not profiling.install_tape_ranges(s.tensor_tape, enabled=False)
    assert s.tensor_tape.range_fn is None


def test_stage_profile_on_cpu():
    prof = profiling.StageProfile(torch.device("cpu"))
    with prof.stage("a"):
        torch.ones(10).sum()
    with prof.stage("a"):
        pass
    out = prof.summary()
    assert out["a"]["n"] == 2 and out["a"]["ms"] >= 0.0


def test_training_log_record_has_the_contract_fields():
    line = {"value": 638000.0, "ms_per_step": 12.8, "step_ms_p50": 12.8, "step_ms_p99": 12.9, "n_gpus": 8, "steps": 20,
            "warmup": 5, "gpu_launches": 5600, "e2e": {"value": 636000.0}, "clocks": {"sm_mhz": 1965.0},
            "config": {"model": "gpt2-small", "parallelism": "dp8"}}
    rec = metrics.training_log_record(line, roofline={"gemm_reduce_scatter": 0.5})
    required = ["schema_version", "ts_unix_ms", "suite_id", "scenario_id", "fixture_id", "packet_id", "mode", "seed",
                "env_fingerprint", "artifact_refs", "replay_command", "outcome", "reason_code"]
    assert all(k in rec for k in required) and rec["artifact_refs"]
    assert rec["schema_version"] == "ft-conformance-log-v1" and rec["outcome"] == "pass"
    assert rec["scenario_id"] == "train/strict:gpt2-small/dp8"
    assert "--nproc-per-node 8" in rec["replay_command"] and "--gpus 8" in rec["replay_command"]
    assert rec["metrics"]["step_ms_p99"] == 12.9 and rec["metrics"]["roofline_fraction"] == {"gemm_reduce_scatter": 0.5}
    assert metrics.training_log_record({"value": 0})["outcome"] == "fail"
