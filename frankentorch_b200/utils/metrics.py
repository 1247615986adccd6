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
