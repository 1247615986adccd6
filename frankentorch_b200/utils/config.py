"""Typed run configuration and the ``FT_*`` environment switches.

The reference has no config file or CLI parser in its libraries: it is configured through
constructor arguments, the session's ``ExecutionMode`` and a set of environment variables read
once behind ``OnceLock`` (``FT_RAYON_WIDTH`` crates/ft-kernel-cpu/src/pool.rs:168,
``FT_SDPA_BR`` crates/ft-kernel-cpu/src/lib.rs:4962, ``FT_METAL_FLASH_V1``
crates/ft-kernel-metal/src/fused.rs:871, ...).  Here the same three mechanisms are kept, with one
dataclass that names everything a training job needs and one registry of environment switches;
both are echoed into the evidence ledger when a job starts, so a replay can see how it ran.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional

from ..runtime.ledger import EvidenceKind, EvidenceLedger, ExecutionMode


# ------------------------------------------------------------------------------ env switches
@dataclass(frozen=True)
class EnvFlag:
    name: str
    default: Any
    parse: Callable[[str], Any]
    doc: str


def _bool(s: str) -> bool:
    return s.strip().lower() not in ("", "0", "false", "off", "no")


ENV_FLAGS: Dict[str, EnvFlag] = {f.name: f for f in (
    EnvFlag("FT_NO_AUTOBUILD", False, _bool,
            "do not compile the kernel library on first use; raise if it is missing"),
    EnvFlag("FT_GEMM_PAIR_COST", 0.92, float,
            "relative cost of a 256x256 CTA-pair GEMM tile against two 128x256 tiles in the tile model"),
    EnvFlag("FT_NVTX", False, _bool, "emit an NVTX range per tape node and per engine phase"),
    EnvFlag("FT_DP_IMPL", "fused", str, "data-parallel gradient path: fused (peer memory) or nccl"),
    EnvFlag("FT_COMM_CTAS", 20, int, "copy CTAs of the gather-fused GEMMs"),
    EnvFlag("FT_MODE", "strict", str, "execution mode of new sessions: strict or hardened"),
    EnvFlag("FT_ENC_CHUNK", 8, int, "encoder inference: layers per CUDA graph (models/encoder.py)"),
    EnvFlag("FT_CPU_THREADS", "", str,
            "thread width of the CPU reference kernels: unset = serial, 'auto' = min(16, physical cores), or a count"),
    EnvFlag("FT_DP_OVERLAP", True, _bool, "start each gradient bucket's reduction under the backward pass"),
    EnvFlag("FT_DP_DEFER", True, _bool, "run the sharded AdamW + parameter all-gather under the next forward pass"),
    EnvFlag("FT_SDPA_BR", "64", str, "query-row tile of the blocked CPU attention kernel (8..512; set_sdpa_br(0) = adaptive)"),
    EnvFlag("FT_GATHER_TRANSPORT", "sm", str, "push-form gathers of the fused GEMMs: copy CTAs (sm) or copy engines (ce)"),
    EnvFlag("FT_DP_NVLS", "0", str, "data-parallel parameter all-gather through NVSwitch multimem stores: 0, 1, or "
            "auto (jobs of eight or more ranks, where the system offers a multicast object)"),
    EnvFlag("FT_DP_WIRE", "bf16", str, "gradient type on NVLink for the fused data-parallel path: bf16 or fp32"),
    EnvFlag("FT_DP_BUCKET_MB", 0.0, float, "gradient bucket size in MB of bf16 (0 = 32)"),
    EnvFlag("FT_DP_CTAS", 296, int, "CTAs of a bucket's push / reduce kernels while the backward pass runs"),
    EnvFlag("FT_DP_UPDATE_CTAS", 592, int, "CTAs of the per-bucket AdamW + all-gather kernels under the forward pass"),
    EnvFlag("FT_SIDE_STREAM", True, _bool, "bias column sums and split-K reductions of a backward rule on a second stream"),
    EnvFlag("FT_DP_TAIL_CTAS", 592, int, "CTAs of the buckets that finish with the backward pass"),
)}

_cache: Dict[str, Any] = {}


def env_flag(name: str) -> Any:
    """Value of a registered switch; parsed once per process like the reference's ``OnceLock``s."""
    if name not in ENV_FLAGS:
        raise KeyError(f"unregistered environment switch {name}")
    if name not in _cache:
        f = ENV_FLAGS[name]
        raw = os.environ.get(name)
        try:
            _cache[name] = f.default if raw is None else f.parse(raw)
        except ValueError as e:
            raise ValueError(f"{name}={raw!r}: {e}") from None
    return _cache[name]


def set_flag(name: str, value: Any) -> None:
    """Programmatic setter (the reference pairs each variable with one, e.g. ``set_sdpa_br``)."""
    if name not in ENV_FLAGS:
        raise KeyError(f"unregistered environment switch {name}")
    _cache[name] = value


def reset_flags() -> None:
    _cache.clear()


def env_snapshot() -> Dict[str, Any]:
    return {n: env_flag(n) for n in sorted(ENV_FLAGS)}


# ------------------------------------------------------------------------------ run config
@dataclass
class ModelSpec:
    name: str = "gpt2-small"
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    d_ff: int = 3072
    vocab: int = 50257
    seq_len: int = 1024
    n_expert: int = 0
    top_k: int = 2
    capacity_factor: float = 1.25


@dataclass
class ParallelSpec:
    layout: str = "dp"          # dp | zero3 | tp | ep | pp
    world: int = 1
    sequence_parallel: bool = True
    dp_impl: str = "fused"      # fused | nccl
    comm_ctas: int = 20
    pipeline_micro_batches: int = 1

    def validate(self) -> None:
        if self.layout not in ("dp", "zero3", "tp", "ep", "pp"):
            raise ValueError(f"unknown parallel layout {self.layout!r}")
        if self.world < 1 or self.world > 8 and self.layout != "dp":
            raise ValueError("fused collectives support 1..8 ranks on one node")
        if self.dp_impl not in ("fused", "nccl"):
            raise ValueError(f"unknown dp_impl {self.dp_impl!r}")


@dataclass
class PrecisionSpec:
    compute: str = "bf16"       # parameters / activations on the GPU
    master: str = "fp32"
    grad_reduce: str = "fp32"   # accumulation dtype of the rank-ordered reductions
    loss_scale: Optional[float] = None


@dataclass
class OptimSpec:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip_norm: float = 1.0


@dataclass
class RunConfig:
    """Everything that determines a training job: model, layout, precision, optimizer, mode."""
    model: ModelSpec = field(default_factory=ModelSpec)
    parallel: ParallelSpec = field(default_factory=ParallelSpec)
    precision: PrecisionSpec = field(default_factory=PrecisionSpec)
    optim: OptimSpec = field(default_factory=OptimSpec)
    micro_batch: int = 8
    seed: int = 1234
    mode: str = "strict"
    cuda_graph: bool = True

    def validate(self) -> "RunConfig":
        self.parallel.validate()
        ExecutionMode.parse(self.mode)
        m = self.model
        if m.d_model % m.n_head:
            raise ValueError("d_model must be a multiple of n_head")
        if m.d_model // m.n_head not in (64, 128):
            raise ValueError("the attention kernels support head sizes 64 and 128")
        if self.parallel.layout == "tp" and m.n_head % self.parallel.world:
            raise ValueError("tensor parallel needs n_head divisible by the world size")
        if self.parallel.layout == "ep" and (m.n_expert == 0 or m.n_expert % self.parallel.world):
            raise ValueError("expert parallel needs n_expert divisible by the world size")
        if self.micro_batch < 1:
            raise ValueError("micro_batch must be positive")
        return self

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True, separators=(",", ":"))

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RunConfig":
        d = dict(d)
        sub = {"model": ModelSpec, "parallel": ParallelSpec, "precision": PrecisionSpec, "optim": OptimSpec}
        kw = {}
        for k, v in d.items():
            if k in sub:
                known = {f.name for f in dataclasses.fields(sub[k])}
                bad = set(v) - known
                if bad:
                    raise ValueError(f"unknown {k} field(s): {sorted(bad)}")
                kw[k] = sub[k](**v)
            elif k in {f.name for f in dataclasses.fields(cls)}:
                kw[k] = v
            else:
                raise ValueError(f"unknown config field {k!r}")
        return cls(**kw).validate()

    @classmethod
    def from_json(cls, s: str) -> "RunConfig":
        return cls.from_dict(json.loads(s))

    def with_env_overrides(self) -> "RunConfig":
        """Apply the environment switches that shadow config fields."""
        out = dataclasses.replace(self, parallel=dataclasses.replace(self.parallel))
        if "FT_DP_IMPL" in os.environ:
            out.parallel.dp_impl = env_flag("FT_DP_IMPL")
        if "FT_COMM_CTAS" in os.environ:
            out.parallel.comm_ctas = env_flag("FT_COMM_CTAS")
        if "FT_MODE" in os.environ:
            out.mode = env_flag("FT_MODE")
        return out.validate()


def echo_to_ledger(ledger: EvidenceLedger, cfg: Optional[RunConfig] = None) -> None:
    """Record the configuration and every environment switch as ``Policy`` evidence."""
    if cfg is not None:
        ledger.record(EvidenceKind.Policy, "run_config " + cfg.to_json())
    ledger.record(EvidenceKind.Policy,
                  "env_flags " + json.dumps(env_snapshot(), sort_keys=True, separators=(",", ":")))
