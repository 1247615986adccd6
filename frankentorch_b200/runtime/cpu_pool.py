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
