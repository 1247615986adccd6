"""Thread-width policy of the CPU reference kernels.

Mirrors ft-kernel-cpu/src/pool.rs (:119 ``auto_width``, :139 ``resolve_width``, :166
``configure_global_pool``): the width is opt-in through ``FT_CPU_THREADS`` (``FT_RAYON_WIDTH`` is
accepted as an alias for users of the reference), ``auto`` means ``min(16, physical cores)``, the
decision is made once per process and echoed into the evidence ledger by the session that made it.
The parallel kernels never split a reduction, so results are bit-identical at every width.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

from . import native


@dataclass(frozen=True)
class PoolOutcome:
    width: int
    changed: bool          # this call decided the width
    spec: str              # what was asked for ("" = nothing)
    physical_cores: int

    def summary(self) -> str:
        how = "configured" if self.changed else "in force"
        return f"cpu pool width={self.width} ({how}; spec={self.spec or 'unset'}; physical_cores={self.physical_cores})"


def resolve_spec(spec: Optional[str] = None) -> str:
    if spec is not None:
        return str(spec).strip()
    return (os.environ.get("FT_CPU_THREADS") or os.environ.get("FT_RAYON_WIDTH") or "").strip()


def configure_cpu_threads(spec: Optional[str] = None, ledger=None) -> PoolOutcome:
    """Decide the process-wide width (first caller wins).  Raises ``ValueError`` on a malformed spec."""
    import ctypes as C
    lib = native.load()
    s = resolve_spec(spec)
    changed = C.c_int(0)
    w = lib.ftc_pool_configure(s.encode(), C.byref(changed))
    if w < 0:
        raise ValueError(f"FT_CPU_THREADS={s!r}: expected 'auto' or a positive integer")
    out = PoolOutcome(int(w), bool(changed.value), s, int(lib.ftc_pool_physical_cores()))
    if ledger is not None:
        from .ledger import EvidenceKind
        ledger.record(EvidenceKind.Policy, out.summary())
    return out


def pool_width() -> int:
    return int(native.load().ftc_pool_width())


def auto_width() -> int:
    return int(native.load().ftc_pool_auto_width())


# ---- runtime toggles of the CPU reference kernels (ft-kernel-cpu/src/lib.rs:4912-4990) -----------------------
def set_sdpa_br(br: int) -> int:
    """Query-row tile of the blocked CPU attention kernel: clamped to [8, 512]; 0 selects the adaptive rule
    (128 rows when heads x blocks keeps the pool busy, else 64).  Returns the value stored.  The environment
    variable ``FT_SDPA_BR`` sets the initial value (read once).  Results are bit-identical for every value."""
    return int(native.load().ftc_set_sdpa_br(int(br)))


def set_parallel_target_workers(workers: int) -> int:
    """Number of chunks the row-parallel CPU kernels are cut into (0 = one per pool thread); returns the previous
    value so a paired measurement can restore it (ft-kernel-cpu/src/lib.rs:2758).  Each row is computed by one
    thread whatever the split: results do not change."""
    return int(native.load().ftc_pool_set_target_workers(int(workers)))


def parallel_target_workers() -> int:
    return int(native.load().ftc_pool_target_workers())


def set_par_min_work(elems: int) -> int:
    """Elements of work below which a kernel stays serial; returns the previous gate."""
    return int(native.load().ftc_pool_set_min_work(int(elems)))


def set_sdpa_br_auto() -> int:
    return set_sdpa_br(0)


def sdpa_br() -> int:
    return int(native.load().ftc_get_sdpa_br())


def sdpa_br_for(seq_q: int, num_bh: int) -> int:
    """The tile the kernel uses for ``num_bh`` (batch x head) problems of ``seq_q`` query rows."""
    return int(native.load().ftc_sdpa_br_for(int(seq_q), int(num_bh)))


def sdpa_blocked(q, k, v, *, causal: bool = False, scale=None):
    """Blocked, pool-parallel f64 attention: ``q`` ``[..., sq, d]``, ``k`` / ``v`` ``[..., sk, d]`` CPU tensors."""
    import math

    import torch
    lead = q.shape[:-2]
    sq, d = q.shape[-2:]
    sk = k.shape[-2]
    q2, k2, v2 = (t.to(torch.float64).reshape(-1, t.shape[-2], d).contiguous() for t in (q, k, v))
    out = torch.empty_like(q2)
    native.load().ftc_sdpa_f64_blocked(q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), out.data_ptr(), q2.shape[0], sq, sk,
                                       d, float(scale if scale is not None else 1.0 / math.sqrt(d)), int(causal))
    return out.reshape(*lead, sq, d)
