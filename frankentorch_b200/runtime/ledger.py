"""Evidence ledger, runtime context and durability envelope.

Behaviour follows the reference runtime crate (ft-runtime/src/lib.rs): four evidence
kinds (:9), entries ``{ts_unix_ms, kind, summary}`` (:17), a bounded ledger that keeps
entry 0 (the policy-init anchor) plus the newest half once the soft cap of 32,768 is
exceeded (:46-55), ``RuntimeContext.new`` recording the initial mode (:94),
``set_mode`` recording a policy entry (:105), decode failures recorded as durability
evidence (:120), and the ``DurabilityEnvelope`` / ``ScrubStatus`` model (:132-197).
The ledger storage is native (``libftcore``).
"""
from __future__ import annotations

import ctypes as C
import enum
import time
from dataclasses import dataclass, field
from typing import List, Optional

from . import native


class ExecutionMode(enum.Enum):
    Strict = "strict"
    Hardened = "hardened"

    @staticmethod
    def parse(v) -> "ExecutionMode":
        if isinstance(v, ExecutionMode):
            return v
        s = str(v).lower()
        if s == "strict":
            return ExecutionMode.Strict
        if s == "hardened":
            return ExecutionMode.Hardened
        raise ValueError(f"unknown execution mode {v!r}")


class EvidenceKind(enum.IntEnum):
    Dispatch = 0
    Backward = 1
    Policy = 2
    Durability = 3


@dataclass(frozen=True)
class EvidenceEntry:
    ts_unix_ms: int
    kind: EvidenceKind
    summary: str


class EvidenceLedger:
    SOFT_CAP = 32768

    def __init__(self, soft_cap: int = SOFT_CAP):
        self._lib = native.load()
        self._h = self._lib.ftc_ledger_new(soft_cap)
        self.soft_cap = soft_cap

    def __del__(self):
        try:
            if self._h:
                self._lib.ftc_ledger_free(self._h)
                self._h = None
        except Exception:
            pass

    def record(self, kind: EvidenceKind, summary: str, ts_unix_ms: int = -1) -> None:
        self._lib.ftc_ledger_record(self._h, int(kind), summary.encode("utf-8"), ts_unix_ms)

    def __len__(self) -> int:
        return int(self._lib.ftc_ledger_len(self._h))

    @property
    def total_recorded(self) -> int:
        return int(self._lib.ftc_ledger_total(self._h))

    def __getitem__(self, i: int) -> EvidenceEntry:
        n = len(self)
        if i < 0:
            i += n
        ts, kind = C.c_int64(), C.c_int()
        buf = C.create_string_buffer(512)
        ln = self._lib.ftc_ledger_get(self._h, i, C.byref(ts), C.byref(kind), buf, 512)
        if ln < 0:
            raise IndexError(i)
        if ln >= 512:
            buf = C.create_string_buffer(ln + 1)
            self._lib.ftc_ledger_get(self._h, i, C.byref(ts), C.byref(kind), buf, ln + 1)
        return EvidenceEntry(ts.value, EvidenceKind(kind.value), buf.value.decode("utf-8", "replace"))

    def entries(self) -> List[EvidenceEntry]:
        return [self[i] for i in range(len(self))]

    def clear(self) -> None:
        self._lib.ftc_ledger_clear(self._h)


class RuntimeContext:
    """Mode policy plus the provenance ledger of one session."""

    def __init__(self, mode: ExecutionMode = ExecutionMode.Strict, soft_cap: int = EvidenceLedger.SOFT_CAP):
        self._mode = ExecutionMode.parse(mode)
        self.ledger = EvidenceLedger(soft_cap)
        self.ledger.record(EvidenceKind.Policy, f"mode initialized to {self._mode.name}")

    @property
    def mode(self) -> ExecutionMode:
        return self._mode

    def set_mode(self, mode: ExecutionMode) -> None:
        self._mode = ExecutionMode.parse(mode)
        self.ledger.record(EvidenceKind.Policy, f"mode switched to {self._mode.name}")

    def record_checkpoint_decode_failure(self, reason: str) -> None:
        self.ledger.record(EvidenceKind.Durability, f"checkpoint decode failure: {reason}")

    def evidence(self) -> List[EvidenceEntry]:
        return self.ledger.entries()

    def ledger_mut(self) -> EvidenceLedger:
        """The ledger itself, for callers that record their own evidence (ft-runtime/src/lib.rs:116)."""
        return self.ledger


class ScrubStatus(enum.Enum):
    Ok = "ok"
    Recovered = "recovered"
    Failed = "failed"


@dataclass
class DecodeProof:
    ts_unix_ms: int
    reason: str
    recovered_blocks: int
    proof_hash: str


@dataclass
class DurabilityEnvelope:
    artifact_id: str
    artifact_type: str
    source_hash: str
    k: int = 0
    repair_symbols: int = 0
    overhead_ratio: float = 0.0
    symbol_hashes: List[str] = field(default_factory=list)
    scrub_status: ScrubStatus = ScrubStatus.Ok
    last_ok_unix_ms: Optional[int] = None
    decode_proofs: List[DecodeProof] = field(default_factory=list)

    def mark_scrub_status(self, status: ScrubStatus) -> None:
        """Result of the latest scrub; an ``Ok`` scrub also stamps ``last_ok_unix_ms``."""
        self.scrub_status = status
        if status is ScrubStatus.Ok:
            self.last_ok_unix_ms = int(time.time() * 1000)

    def add_decode_proof(self, reason: str, proof_hash: str, recovered_blocks: int = 0) -> None:
        self.decode_proofs.append(DecodeProof(int(time.time() * 1000), str(reason), int(recovered_blocks), str(proof_hash)))
