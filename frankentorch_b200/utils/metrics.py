"""Training metrics: step-time percentiles, tokens/s, roofline fractions.

Percentiles follow the reference's perf reports: nearest-rank on the sorted samples
(crates/ft-conformance/src/perf_slo.rs:177-186), with p50/p95/p99/mean/min/max as in ``:43-83``.
Roofline fractions are taken against peaks measured on the machine (a copy bandwidth and a
library bf16 GEMM rate stored in a JSON file), never against nominal figures.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

import torch


def percentile_nearest_rank(samples: Sequence[float], pct: float) -> float:
    """Nearest-rank percentile: the value at rank ceil(pct/100 * n) of the sorted samples."""
    if not samples:
        raise ValueError("percentile of an empty sample")
    if not 0.0 < pct <= 100.0:
        raise ValueError("pct must be in (0, 100]")
    s = sorted(samples)
    rank = max(1, math.ceil(pct / 100.0 * len(s)))
    return float(s[rank - 1])


def summarize(samples: Sequence[float]) -> Dict[str, float]:
    return {"n": len(samples), "p50": percentile_nearest_rank(samples, 50), "p95": percentile_nearest_rank(samples, 95),
            "p99": percentile_nearest_rank(samples, 99), "mean": float(sum(samples) / len(samples)),
            "min": float(min(samples)), "max": float(max(samples))}


class StepTimer:
    """One CUDA event per step boundary; durations are read after the loop, so the timed region
    carries no synchronisation of its own."""

    def __init__(self):
        self.marks: List[torch.cuda.Event] = []

    def mark(self) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.marks.append(e)

    def step_ms(self) -> List[float]:
        torch.cuda.synchronize()
        return [self.marks[i].elapsed_time(self.marks[i + 1]) for i in range(len(self.marks) - 1)]

    def total_ms(self) -> float:
        torch.cuda.synchronize()
        return self.marks[0].elapsed_time(self.marks[-1])


def max_over_ranks(value: float, device, group=None) -> float:
    """The slowest rank's figure: multi-GPU times are reported as the maximum over ranks."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


@dataclass(frozen=True)
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    nvlink_gbs: float = 770.0
    source: str = "fallback"


FALLBACK_PEAKS = Peaks(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def load_peaks(path: Optional[str] = None) -> Peaks:
    """Measured peaks from ``MEASURED_PEAKS.json`` beside the package root, else the fallback."""
    p = Path(path) if path else Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return Peaks(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                     bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    except (OSError, KeyError, ValueError):
        return FALLBACK_PEAKS


def roofline_fraction(*, us: float, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
                      peaks: Optional[Peaks] = None, sustained: bool = False) -> Dict[str, float]:
    """Achieved / attainable for one launch: the bound is the slowest of FLOPs / GEMM peak,
    HBM bytes / copy bandwidth and NVLink bytes / link bandwidth."""
    pk = peaks or load_peaks()
    tf = pk.bf16_tflops_sustained if sustained else pk.bf16_tflops
    t_flop = flops / (tf * 1e12) * 1e6
    t_hbm = hbm_bytes / (pk.hbm_gbs * 1e9) * 1e6
    t_link = nvlink_bytes / (pk.nvlink_gbs * 1e9) * 1e6
    bound = max(t_flop, t_hbm, t_link)
    which = "flops" if bound == t_flop else ("hbm" if bound == t_hbm else "nvlink")
    return {"bound_us": bound, "fraction": (bound / us) if us > 0 else 0.0, "limiter": which, "peaks": pk.source}


def gpt_step_flops(n_layer: int, d: int, ff: int, vocab: int, seq: int, tokens: int, causal: bool = True) -> float:
    """Model FLOPs of one training step (forward + backward = 3 x forward GEMM work; attention
    scores and context counted at half density when causal)."""
    per_tok = n_layer * (2 * d * 3 * d + 2 * d * d + 2 * 2 * d * ff) + 2 * d * vocab
    attn = n_layer * 2 * 2 * seq * d * (0.5 if causal else 1.0)
    return 3.0 * tokens * (per_tok + attn)


def training_log_record(bench_line: Dict, *, mode: str = "strict", seed: int = 1234,
                        roofline: Optional[Dict[str, float]] = None) -> Dict:
    """One ``ft-conformance-log-v1`` record for a training benchmark: the 13 required fields of the
    structured log contract (artifacts/phase2c/TEST_LOG_CONTRACT_V1.md) plus the training metrics
    (tokens/s max over ranks, step-time p50 / p99, roofline fraction per fused path)."""
    import time

    from ..conformance.runner import LOG_SCHEMA, env_fingerprint
    cfg = bench_line.get("config", {})
    scenario = f"train/{mode}:{cfg.get('model', '?')}/{cfg.get('parallelism', '?')}"
    n = int(bench_line.get("n_gpus", 1))
    launch = "python bench.py" if n == 1 else (
        f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {n} --master-addr 127.0.0.1 bench.py")
    return {
        "schema_version": LOG_SCHEMA, "ts_unix_ms": int(time.time() * 1000), "suite_id": "training",
        "scenario_id": scenario, "fixture_id": "synthetic-uniform-tokens", "packet_id": "FT-B200-TRAIN",
        "mode": mode, "seed": int(seed), "env_fingerprint": env_fingerprint(),
        "artifact_refs": ["bench.py"],
        "replay_command": f"{launch} --gpus {n} --model {cfg.get('model', 'gpt2-small')} "
                          f"--steps {bench_line.get('steps', 20)} --warmup {bench_line.get('warmup', 5)}",
        "outcome": "pass" if bench_line.get("value", 0) > 0 else "fail",
        "reason_code": "ok" if bench_line.get("value", 0) > 0 else "no_throughput",
        "metrics": {
            "tokens_per_s_max_over_ranks": bench_line.get("value"),
            "ms_per_step": bench_line.get("ms_per_step"),
            "step_ms_p50": bench_line.get("step_ms_p50"), "step_ms_p99": bench_line.get("step_ms_p99"),
            "e2e_tokens_per_s": (bench_line.get("e2e") or {}).get("value"),
            "gpu_launches": bench_line.get("gpu_launches"), "n_gpus": n,
            "clocks": bench_line.get("clocks"), "roofline_fraction": dict(roofline or {}),
        },
    }
