"""JSON checkpoint envelope and erasure-coded sidecar (mirror of ft-serialize, formats 1 and 2).

Envelope (ft-serialize/src/lib.rs:39-67):
``{"schema_version":1,"mode":"strict"|"hardened","entries":[{"node_id","value","grad"}],
"source_hash":"det64:%016x"}``; unknown fields rejected; entries normalised by sorting on
``(node_id, value bits, grad None<Some, grad bits)`` (:488-504); non-finite values rejected
at encode (:462-486); 1 MiB payload cap (:17); strict decode = typed parse that names the
unknown field, hardened decode = bounded diagnostics for non-object / incompatible payloads
(:375-424); version + checksum validation (:438-460).

The hash feeds ``u32 version, u8 mode(1|2)`` and per entry ``u64 node_id, u64 value bits,
u8 has_grad, u64 grad bits`` (:506-529) into a 64-bit hasher.  The reference's hasher
(``DetHasher::for_lab`` of an external crate) is not available offline; this implementation
uses FNV-1a-64 over the same byte feed, so envelopes written here verify here, while the
reference's golden digest (``det64:4950f922ab2dbd30``) does not reproduce.

Sidecar: a systematic random linear fountain code over GF(2^8) with seeded, replayable
coefficients (``code = "rlf256-systematic-v1"``) in the role RaptorQ plays in the reference
(:175-373), with the reference's parameters: symbol size 32 / 64 / 128 / 256 by payload length
(:553-560), seed ``0x46545f5241505451``, repair count ``max(requested, 1) + 8`` with the 1024 /
65,536 limits, a manifest of repair symbols and a decode proof found by dropping source symbols
in several mixes until a decode returns the payload.  Any ``m`` lost source symbols are recovered
from ``m`` repair symbols unless their coefficient matrix happens to be singular (probability
about 1/255, vanishing with every surplus symbol).
"""
from __future__ import annotations

import enum
import json
import math
import struct
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..runtime import native
from ..runtime.ledger import ExecutionMode

SCHEMA_VERSION = 1
MAX_PAYLOAD_BYTES = 1 << 20
SIDECAR_SEED = 0x46545F5241505451
OBJECT_ID = (0x46545F434B50545F, 0x4455524142494C45)
MAX_REPAIR_SYMBOLS = 1024
MAX_SOURCE_SYMBOLS = 65536


class SerializeError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass(frozen=True)
class SnapshotEntry:
    node_id: int
    value: float
    grad: Optional[float] = None


def _bits(x: float) -> int:
    return struct.unpack("<Q", struct.pack("<d", x))[0]


def normalize_entries(entries: Sequence[SnapshotEntry]) -> List[SnapshotEntry]:
    return sorted(entries, key=lambda e: (e.node_id, _bits(e.value), e.grad is not None,
                                          _bits(e.grad) if e.grad is not None else 0))


def checkpoint_hash(version: int, mode: ExecutionMode, entries: Sequence[SnapshotEntry]) -> str:
    b = bytearray(struct.pack("<I", version))
    b.append(1 if mode == ExecutionMode.Strict else 2)
    for e in entries:
        b += struct.pack("<QQ", e.node_id, _bits(e.value))
        if e.grad is None:
            b.append(0)
        else:
            b.append(1)
            b += struct.pack("<Q", _bits(e.grad))
    return f"det64:{native.fnv1a64(bytes(b)):016x}"


def hash_bytes(data: bytes) -> str:
    return f"det64:{native.fnv1a64(data):016x}"


def encode_checkpoint(entries: Sequence[SnapshotEntry], mode: ExecutionMode = ExecutionMode.Strict) -> str:
    mode = ExecutionMode.parse(mode)
    for e in entries:
        if not math.isfinite(e.value) or (e.grad is not None and not math.isfinite(e.grad)):
            raise SerializeError("NonFinite", f"node {e.node_id}: non-finite value or gradient cannot be encoded")
        if e.node_id < 0:
            raise SerializeError("InvalidNode", "node ids are unsigned")
    norm = normalize_entries(entries)
    doc = {"schema_version": SCHEMA_VERSION, "mode": mode.value,
           "entries": [{"node_id": e.node_id, "value": e.value, "grad": e.grad} for e in norm],
           "source_hash": checkpoint_hash(SCHEMA_VERSION, mode, norm)}
    text = json.dumps(doc, separators=(",", ":"))
    if len(text.encode()) > MAX_PAYLOAD_BYTES:
        raise SerializeError("PayloadTooLarge", f"payload exceeds {MAX_PAYLOAD_BYTES} bytes")
    return text


class CheckpointMode(enum.Enum):
    """Mode stamped into an envelope when it is written (ft-serialize/src/lib.rs:49)."""
    Strict = "strict"
    Hardened = "hardened"

    def execution_mode(self) -> ExecutionMode:
        return ExecutionMode.parse(self.value)


class DecodeMode(enum.Enum):
    """Diagnostic style of the decoder (ft-serialize/src/lib.rs:55): strict reports the parser's position, hardened
    classifies the payload as incompatible and says why."""
    Strict = "strict"
    Hardened = "hardened"

    def execution_mode(self) -> ExecutionMode:
        return ExecutionMode.parse(self.value)


def _exec_mode(mode) -> ExecutionMode:
    return mode.execution_mode() if isinstance(mode, (CheckpointMode, DecodeMode)) else ExecutionMode.parse(mode)


@dataclass(frozen=True)
class CheckpointEnvelope:
    """The decoded document (ft-serialize/src/lib.rs:62): version, writer's mode, normalised entries and the hash
    that binds them."""
    schema_version: int
    mode: CheckpointMode
    entries: Tuple[SnapshotEntry, ...]
    source_hash: str

    def to_json(self) -> str:
        return json.dumps({"schema_version": self.schema_version, "mode": self.mode.value,
                           "entries": [{"node_id": e.node_id, "value": e.value, "grad": e.grad} for e in self.entries],
                           "source_hash": self.source_hash}, separators=(",", ":"))


def encode_envelope(entries: Sequence[SnapshotEntry], mode=CheckpointMode.Strict) -> CheckpointEnvelope:
    """Validate and normalise ``entries`` and bind them with the source hash, without rendering JSON."""
    text = encode_checkpoint(entries, _exec_mode(mode))
    return decode_envelope(text, DecodeMode.Strict)


def decode_envelope(text: str, mode=DecodeMode.Strict, runtime=None) -> CheckpointEnvelope:
    """``decode_checkpoint`` returning the whole envelope record."""
    m, entries = decode_checkpoint(text, _exec_mode(mode), runtime)
    doc = json.loads(text)
    return CheckpointEnvelope(int(doc["schema_version"]), CheckpointMode(m.value), tuple(entries), doc["source_hash"])


def encode_snapshot(entries: Sequence[SnapshotEntry]) -> str:
    """Strict-mode envelope of ``entries`` (ft-serialize/src/lib.rs:166)."""
    return encode_checkpoint(entries, ExecutionMode.Strict)


def decode_snapshot(text: str) -> List[SnapshotEntry]:
    """Entries of a strict-mode decode (ft-serialize/src/lib.rs:170)."""
    return decode_checkpoint(text, ExecutionMode.Strict)[1]


_TOP_KEYS = {"schema_version", "mode", "entries", "source_hash"}
_ENTRY_KEYS = {"node_id", "value", "grad"}


def decode_checkpoint(text: str, mode: ExecutionMode = ExecutionMode.Strict, runtime=None) -> Tuple[ExecutionMode, List[SnapshotEntry]]:
    """Decode and verify an envelope.  ``mode`` selects the diagnostic style; failures are also
    recorded as durability evidence on ``runtime`` when one is given."""
    mode = ExecutionMode.parse(mode)

    def fail(kind, msg):
        if runtime is not None:
            runtime.record_checkpoint_decode_failure(msg)
        raise SerializeError(kind, msg)

    if len(text.encode()) > MAX_PAYLOAD_BYTES:
        fail("PayloadTooLarge", f"payload exceeds {MAX_PAYLOAD_BYTES} bytes")
    try:
        doc = json.loads(text)
    except json.JSONDecodeError as e:
        fail("InvalidJson", f"invalid json: {e.msg} at line {e.lineno} column {e.colno}" if mode == ExecutionMode.Strict
             else f"incompatible payload: malformed json ({e.msg})")
    if not isinstance(doc, dict):
        fail("InvalidJson" if mode == ExecutionMode.Strict else "IncompatiblePayload",
             "invalid json: expected an object at the top level" if mode == ExecutionMode.Strict
             else f"incompatible payload: top-level {type(doc).__name__} is not an object")
    unknown = sorted(set(doc) - _TOP_KEYS)
    if unknown:
        fail("UnknownField", f"unknown field `{unknown[0]}`" if mode == ExecutionMode.Strict
             else f"incompatible payload: unknown keys {unknown[:8]}")
    missing = sorted(_TOP_KEYS - set(doc))
    if missing:
        fail("MissingField", f"missing field `{missing[0]}`")
    if doc["schema_version"] != SCHEMA_VERSION:
        fail("VersionMismatch", f"unsupported schema version {doc['schema_version']} (expected {SCHEMA_VERSION})")
    try:
        doc_mode = ExecutionMode.parse(doc["mode"])
    except ValueError:
        fail("InvalidMode", f"unknown mode {doc['mode']!r}")
    if not isinstance(doc["entries"], list):
        fail("InvalidJson", "invalid json: `entries` must be an array")
    entries = []
    for raw in doc["entries"]:
        if not isinstance(raw, dict) or set(raw) - _ENTRY_KEYS or not {"node_id", "value"} <= set(raw):
            fail("InvalidEntry", "invalid entry: expected {node_id, value, grad}")
        if not isinstance(raw["node_id"], int) or raw["node_id"] < 0:
            fail("InvalidEntry", "invalid entry: node_id must be an unsigned integer")
        g = raw.get("grad")
        entries.append(SnapshotEntry(raw["node_id"], float(raw["value"]), None if g is None else float(g)))
    want = checkpoint_hash(SCHEMA_VERSION, doc_mode, normalize_entries(entries))
    if doc["source_hash"] != want:
        fail("ChecksumMismatch", f"checksum mismatch: envelope has {doc['source_hash']}, entries hash to {want}")
    return doc_mode, entries


# -------------------------------------------------------------------------------------- sidecar
# The erasure code is a systematic random linear fountain code over GF(2^8) ("rlf256"): repair
# symbol e is sum_i c(e, i) * source_i with coefficients drawn from a generator seeded by
# (seed, e), every c non-zero.  Any m lost source symbols are recovered from any m' >= m repair
# symbols whose m x m' coefficient matrix has rank m - for random coefficients that fails with
# probability about 1/255 per exactly-sufficient set and vanishes with each extra symbol - by
# Gauss-Jordan elimination over GF(2^8).  It is NOT RaptorQ (RFC 6330's pre-code and degree tables
# are not reproduced here); it plays RaptorQ's role with the reference's parameters.
CODE_NAME = "rlf256-systematic-v1"
_GF_POLY = 0x11D


def _gf_tables():
    import numpy as np
    exp = np.zeros(512, dtype=np.int32)
    log = np.zeros(256, dtype=np.int32)
    x = 1
    for i in range(255):
        exp[i] = x
        log[x] = i
        x <<= 1
        if x & 0x100:
            x ^= _GF_POLY
    exp[255:510] = exp[0:255]
    mul = np.zeros((256, 256), dtype=np.uint8)
    a = np.arange(1, 256)
    mul[1:, 1:] = exp[(log[a][:, None] + log[a][None, :])].astype(np.uint8)
    inv = np.zeros(256, dtype=np.uint8)
    inv[1:] = exp[255 - log[a]].astype(np.uint8)
    return mul, inv


_GF = None


def _gf():
    global _GF
    if _GF is None:
        _GF = _gf_tables()
    return _GF


@dataclass
class RepairSymbol:
    esi: int
    degree: int
    bytes: str      # hex


@dataclass(frozen=True)
class RepairSymbolRecord:
    """Manifest line of one repair symbol (ft-serialize/src/lib.rs:71): its encoding symbol id, how many source
    symbols it combines, and its length in bytes; the payload itself stays in the sidecar."""
    esi: int
    degree: int
    bytes: int


@dataclass
class RepairSidecar:
    """Repair symbols stored next to an artifact (field set of the reference's sidecar record,
    ft-serialize/src/lib.rs:69-101, plus ``code``, which names the erasure code actually used)."""
    schema_version: int
    source_hash: str
    symbol_size: int
    k: int
    payload_len: int
    seed: int
    object_id: Tuple[int, int]
    repair_symbols: int
    repair_manifest: List[RepairSymbol] = field(default_factory=list)
    code: str = CODE_NAME

    def to_json(self) -> str:
        return json.dumps(asdict(self), separators=(",", ":"))

    def symbol_records(self) -> List[RepairSymbolRecord]:
        return [RepairSymbolRecord(r.esi, r.degree, len(r.bytes) // 2) for r in self.repair_manifest]


# Name under which the reference exposes this record.  The record's ``code`` field says which
# erasure code produced the symbols: this implementation's is rlf256, not RaptorQ.
RaptorQSidecar = RepairSidecar


@dataclass
class DecodeProofArtifact:
    schema_version: int
    source_hash: str
    dropped_source_symbols: List[int]
    used_repair_esis: List[int]
    recovered: bool
    proof_hash: str


def symbol_size_for(payload_len: int) -> int:
    if payload_len <= 1024:
        return 32
    if payload_len <= 16 * 1024:
        return 64
    if payload_len <= 256 * 1024:
        return 128
    return 256


class _Lcg:
    def __init__(self, seed):
        self.s = seed & ((1 << 64) - 1)

    def next(self, bound):
        self.s = (self.s * 6364136223846793005 + 1) & ((1 << 64) - 1)
        return (self.s >> 33) % bound


def _coefficients(esi: int, k: int, seed: int):
    """The k non-zero GF(2^8) coefficients of repair symbol ``esi`` (replayable from seed and esi)."""
    import numpy as np
    g = _Lcg(seed ^ ((esi + 1) * 0x9E3779B97F4A7C15))
    return np.fromiter((1 + g.next(255) for _ in range(k)), dtype=np.uint8, count=k)


def _symbols(payload: bytes, size: int):
    import numpy as np
    k = max(1, (len(payload) + size - 1) // size)
    padded = payload + bytes(k * size - len(payload))
    return np.frombuffer(padded, dtype=np.uint8).reshape(k, size).copy()


def repair_symbol_count(requested: int, k: int) -> int:
    """``max(requested, 1) + 8`` (ft-serialize/src/lib.rs:205-221; the systematic code needs no
    padding symbols, so the reference's ``k' - k`` term is zero).  More than 1024 requested repair
    symbols, or a block of more than 65,536 source symbols, is an error (:27, :37, :186)."""
    if requested > MAX_REPAIR_SYMBOLS:
        raise SerializeError("RepairSymbolLimit", f"repair_symbols {requested} exceeds {MAX_REPAIR_SYMBOLS}")
    if k > MAX_SOURCE_SYMBOLS:
        raise SerializeError("SourceSymbolLimit", f"{k} source symbols exceed {MAX_SOURCE_SYMBOLS}")
    return max(requested, 1) + 8


def generate_repair_sidecar(payload: bytes, repair_symbols: int = 0) -> Tuple[RepairSidecar, DecodeProofArtifact]:
    """Repair symbols for ``payload`` and a proof that it is recoverable from them.

    The proof is found the way the reference does it (:223-373): source symbols are dropped in
    several mixes (the first ones, evenly spread ones, seeded random ones, as many as there are repair
    symbols and then fewer) until a decode from the remaining symbols plus the sidecar returns the
    payload; ``recovered`` is False - never assumed - if none of the mixes decodes."""
    import numpy as np
    mul, _ = _gf()
    size = symbol_size_for(len(payload))
    src = _symbols(payload, size)
    k = src.shape[0]
    count = repair_symbol_count(repair_symbols, k)
    manifest = []
    for j in range(count):
        esi = k + j
        c = _coefficients(esi, k, SIDECAR_SEED)
        sym = np.bitwise_xor.reduce(mul[c[:, None], src], axis=0)
        manifest.append(RepairSymbol(esi, k, sym.tobytes().hex()))
    side = RepairSidecar(1, hash_bytes(payload), size, k, len(payload), SIDECAR_SEED, OBJECT_ID, count, manifest)
    rows = [src[i].tobytes() for i in range(k)]
    rng = _Lcg(SIDECAR_SEED ^ k)
    proof = None
    for ndrop in sorted({min(k, count), min(k, max(1, count // 2)), min(k, 3), 1}, reverse=True):
        mixes = [list(range(ndrop)), sorted({(i * k) // ndrop for i in range(ndrop)}),
                 sorted({rng.next(k) for _ in range(ndrop)})]
        for dropped in mixes:
            rec = decode_with_sidecar([None if i in set(dropped) else r for i, r in enumerate(rows)], side)
            if rec is not None and rec == payload:
                used = [m.esi for m in manifest[: len(dropped)]]
                ph = hash_bytes(json.dumps([side.source_hash, dropped, used]).encode())
                proof = DecodeProofArtifact(1, side.source_hash, dropped, used, True, ph)
                break
        if proof is not None:
            break
    if proof is None:
        proof = DecodeProofArtifact(1, side.source_hash, [], [], False, hash_bytes(side.source_hash.encode()))
    return side, proof


# The reference's name for this entry point (ft-serialize/src/lib.rs:175).
generate_raptorq_sidecar = generate_repair_sidecar


def decode_with_sidecar(received: Sequence[Optional[bytes]], side: RepairSidecar) -> Optional[bytes]:
    """Recover the payload from source symbols (``None`` = lost) plus the sidecar's repair symbols
    by Gauss-Jordan elimination over GF(2^8).  Returns ``None`` if the losses are not recoverable
    (more losses than repair symbols, a rank-deficient system, or a hash mismatch afterwards)."""
    import numpy as np
    mul, inv = _gf()
    k, size = side.k, side.symbol_size
    if len(received) != k:
        return None
    missing = [i for i, s in enumerate(received) if s is None]
    if not missing:
        data = b"".join(received)[: side.payload_len]
        return data if hash_bytes(data) == side.source_hash else None
    m = len(missing)
    if m > len(side.repair_manifest):
        return None
    have = [i for i in range(k) if received[i] is not None]
    have_arr = np.frombuffer(b"".join(received[i] for i in have), dtype=np.uint8).reshape(len(have), size) \
        if have else np.zeros((0, size), dtype=np.uint8)
    A = np.zeros((len(side.repair_manifest), m), dtype=np.uint8)
    B = np.zeros((len(side.repair_manifest), size), dtype=np.uint8)
    for r, rs in enumerate(side.repair_manifest):
        c = _coefficients(rs.esi, k, side.seed)
        val = np.frombuffer(bytes.fromhex(rs.bytes), dtype=np.uint8).copy()
        if len(val) != size:
            return None
        if have:
            val ^= np.bitwise_xor.reduce(mul[c[have][:, None], have_arr], axis=0)
        A[r] = c[missing]
        B[r] = val
    # Gauss-Jordan: a pivot row per missing symbol, eliminated from every other row
    used = np.zeros(A.shape[0], dtype=bool)
    pivot_of = [-1] * m
    for j in range(m):
        cand = [r for r in range(A.shape[0]) if not used[r] and A[r, j] != 0]
        if not cand:
            return None
        p = cand[0]
        used[p] = True
        pivot_of[j] = p
        f = inv[A[p, j]]
        A[p] = mul[f, A[p]]
        B[p] = mul[f, B[p]]
        for r in range(A.shape[0]):
            if r != p and A[r, j] != 0:
                g = A[r, j]
                A[r] ^= mul[g, A[p]]
                B[r] ^= mul[g, B[p]]
    out = list(received)
    for j, i in enumerate(missing):
        out[i] = B[pivot_of[j]].tobytes()
    data = b"".join(out)[: side.payload_len]
    return data if hash_bytes(data) == side.source_hash else None
