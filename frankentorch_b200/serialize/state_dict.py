"""FTSV native state-dict format, SafeTensors and single-Linear ONNX export.

FTSV (ft-serialize/src/lib.rs:594-604, writer :711-861, loader :996-1163): magic ``"FTSV"``,
``u32 LE version = 1``, ``u64 LE num_tensors``, then per tensor in sorted key order:
``u64 key_len, key bytes (UTF-8), u64 ndim, ndim x u64 dims, u8 dtype tag (0=F64, 1=F32,
2=F16, 3=BF16), raw little-endian values``.  The loader rejects bad magic, versions above 1,
duplicate keys, truncated data, shape overflow and trailing bytes, and bounds ``num_tensors``
by ``remaining_bytes / 17`` before allocating.  The format has no hash and is fully
specified, so files are byte-identical to the reference's for the same tensors.

SafeTensors (:1936-2285): F64 / F32 / F16 / BF16, optional string metadata, header-only
metadata read.  ONNX (:1496-1651): hand-rolled protobuf, IR version 8, opset 17,
``MatMul`` + ``Add`` (or ``Identity`` without bias) for one Linear layer.

Sharded checkpoints: ``save_sharded`` writes ``<stem>.rank{r}.ftsv`` per rank and
``consolidate_shards`` reproduces the single-file byte stream.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .checkpoint import SerializeError

FTSV_MAGIC = b"FTSV"
FTSV_VERSION = 1
_TAG = {torch.float64: 0, torch.float32: 1, torch.float16: 2, torch.bfloat16: 3}
_UNTAG = {v: k for k, v in _TAG.items()}
_ESIZE = {0: 8, 1: 4, 2: 2, 3: 2}


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().to("cpu").contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def state_dict_to_bytes(sd: Dict[str, torch.Tensor]) -> bytes:
    for k, t in sd.items():
        if t.dtype not in _TAG:
            raise SerializeError("UnsupportedDType", f"{k}: dtype {t.dtype} is not storable (F64/F32/F16/BF16 only)")
    out = [FTSV_MAGIC, struct.pack("<IQ", FTSV_VERSION, len(sd))]
    for k in sorted(sd):
        t = sd[k]
        kb = k.encode("utf-8")
        out.append(struct.pack("<Q", len(kb)))
        out.append(kb)
        out.append(struct.pack("<Q", t.dim()))
        out.append(struct.pack(f"<{t.dim()}Q", *t.shape) if t.dim() else b"")
        out.append(bytes([_TAG[t.dtype]]))
        out.append(_raw_bytes(t))
    return b"".join(out)


def save_state_dict(sd: Dict[str, torch.Tensor], path: str) -> int:
    data = state_dict_to_bytes(sd)
    tmp = path + ".tmp"
    with open(tmp, "wb", buffering=1 << 20) as f:
        f.write(data)
    os.replace(tmp, path)
    return len(data)


def load_state_dict_from_bytes(data: bytes) -> Dict[str, torch.Tensor]:
    n = len(data)
    if n < 4 or data[:4] != FTSV_MAGIC:
        raise SerializeError("InvalidMagic", f"invalid magic: expected 'FTSV', found {data[:4]!r}")
    if n < 16:
        raise SerializeError("Truncated", "truncated header")
    version, count = struct.unpack_from("<IQ", data, 4)
    if version > FTSV_VERSION:
        raise SerializeError("UnsupportedVersion", f"unsupported version {version} (max {FTSV_VERSION})")
    off = 16
    if count > (n - off) // 17:
        raise SerializeError("Truncated", f"tensor count {count} exceeds what {n - off} remaining bytes can hold")
    out: Dict[str, torch.Tensor] = {}

    def need(k, what):
        if off + k > n:
            raise SerializeError("Truncated", f"truncated {what}")

    for _ in range(count):
        need(8, "key length")
        (klen,) = struct.unpack_from("<Q", data, off)
        off += 8
        need(klen, "key bytes")
        try:
            key = data[off: off + klen].decode("utf-8")
        except UnicodeDecodeError:
            raise SerializeError("InvalidKey", "key is not valid UTF-8")
        off += klen
        if key in out:
            raise SerializeError("DuplicateKey", f"duplicate key '{key}'")
        need(8, "rank")
        (ndim,) = struct.unpack_from("<Q", data, off)
        off += 8
        if ndim > 64:
            raise SerializeError("ShapeOverflow", f"rank {ndim} is not plausible")
        need(8 * ndim, "shape dims")
        dims = struct.unpack_from(f"<{ndim}Q", data, off) if ndim else ()
        off += 8 * ndim
        numel, span = 1, 1
        for d in dims:
            numel *= d
            span *= max(d, 1)           # strides are built from the non-zero extents: a zero extent elsewhere
            if span > (1 << 62):        # must not hide an extent (or a product of extents) beyond the index range
                raise SerializeError("ShapeOverflow", "shape volume overflows")
        need(1, "dtype tag")
        tag = data[off]
        off += 1
        if tag not in _UNTAG:
            raise SerializeError("InvalidDType", f"unknown dtype tag {tag}")
        nbytes = numel * _ESIZE[tag]
        need(nbytes, f"values of '{key}'")
        buf = bytes(data[off: off + nbytes])
        off += nbytes
        if tag == 3:
            t = torch.frombuffer(bytearray(buf), dtype=torch.int16).view(torch.bfloat16) if nbytes else torch.empty(0, dtype=torch.bfloat16)
        else:
            t = torch.frombuffer(bytearray(buf), dtype=_UNTAG[tag]) if nbytes else torch.empty(0, dtype=_UNTAG[tag])
        out[key] = t.reshape(tuple(dims)).clone()
    if off != n:
        raise SerializeError("TrailingBytes", f"{n - off} trailing bytes after the last tensor")
    return out


def load_state_dict(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        return load_state_dict_from_bytes(f.read())


# -------------------------------------------------------------------------------------- sharded
def save_sharded(sd: Dict[str, torch.Tensor], stem: str, rank: int) -> str:
    path = f"{stem}.rank{rank}.ftsv"
    save_state_dict(sd, path)
    return path


def consolidate_shards(stem: str, world: int, out_path: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """Merge per-rank shards: disjoint key sets, row-sharded tensors named ``key@shard{r}``
    (concatenated in rank order), and bucket-sharded flat tensors named ``key@bshard{r}`` with
    their bucket table ``key@layout`` (rows ``lo, hi, shard, off``: rank ``r`` holds elements
    ``[lo + r*shard, min(lo + (r+1)*shard, hi))`` of every bucket at ``off`` of its piece)."""
    merged: Dict[str, torch.Tensor] = {}
    parts: Dict[str, List[Tuple[int, torch.Tensor]]] = {}
    bparts: Dict[str, Dict[int, torch.Tensor]] = {}
    layouts: Dict[str, torch.Tensor] = {}
    for r in range(world):
        for k, t in load_state_dict(f"{stem}.rank{r}.ftsv").items():
            if k.endswith("@layout"):
                layouts[k[: -len("@layout")]] = t
            elif "@bshard" in k:
                base, idx = k.rsplit("@bshard", 1)
                bparts.setdefault(base, {})[int(idx)] = t
            elif "@shard" in k:
                base, idx = k.rsplit("@shard", 1)
                parts.setdefault(base, []).append((int(idx), t))
            elif k in merged:
                if not torch.equal(merged[k], t):
                    raise SerializeError("ShardConflict", f"replicated key '{k}' differs between ranks")
            else:
                merged[k] = t
    for base, lst in parts.items():
        merged[base] = torch.cat([t for _, t in sorted(lst, key=lambda x: x[0])], 0)
    for base, by_rank in bparts.items():
        if base not in layouts or sorted(by_rank) != list(range(world)):
            raise SerializeError("ShardLayout", f"'{base}': bucket table or a rank's piece is missing")
        table = layouts[base].to(torch.int64).reshape(-1, 4).tolist()
        numel = max(hi for _, hi, _, _ in table)
        full = torch.zeros(numel, dtype=by_rank[0].dtype)
        for lo, hi, shard, off in table:
            for r in range(world):
                a = lo + r * shard
                b = max(a, min(a + shard, hi))
                if b > a:
                    full[a:b] = by_rank[r].reshape(-1)[off: off + (b - a)]
        merged[base] = full
    if out_path:
        save_state_dict(merged, out_path)
    return merged


# -------------------------------------------------------------------------------------- safetensors
_ST_NAME = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16"}
_ST_DTYPE = {v: k for k, v in _ST_NAME.items()}


class TensorIOError(SerializeError):
    """Failure of a tensor file operation (ft-serialize/src/lib.rs:608).  ``kind`` is one of ``Io`` (with ``path``),
    ``InvalidMagic``, ``UnsupportedVersion`` (with ``found`` / ``max``), ``Corrupt`` (with ``reason``) and
    ``TensorError``; decoders of this module raise the parent class with finer kinds, and ``classify`` maps those
    onto this set."""

    KINDS = ("Io", "InvalidMagic", "UnsupportedVersion", "Corrupt", "TensorError")

    def __init__(self, kind: str, message: str, **fields):
        if kind not in self.KINDS:
            raise ValueError(f"unknown TensorIOError kind {kind!r}")
        super().__init__(kind, message)
        self.fields = fields

    @staticmethod
    def classify(err: Exception, path: Optional[str] = None) -> "TensorIOError":
        if isinstance(err, TensorIOError):
            return err
        if isinstance(err, OSError):
            return TensorIOError("Io", f"I/O error at '{path}': {err.strerror or err}", path=path, detail=str(err))
        if isinstance(err, SerializeError):
            if err.kind in ("InvalidMagic", "UnsupportedVersion"):
                return TensorIOError(err.kind, str(err))
            if err.kind in ("InvalidShape", "ShapeOverflow", "InvalidDType", "UnsupportedDType"):
                return TensorIOError("TensorError", str(err))
            return TensorIOError("Corrupt", f"corrupt file: {err}", reason=str(err))
        return TensorIOError("Corrupt", f"corrupt file: {err}", reason=str(err))


def load_tensor_file(path: str) -> Dict[str, torch.Tensor]:
    """Load an FTSV or SafeTensors file (told apart by the magic bytes); every failure is a ``TensorIOError``."""
    try:
        with open(path, "rb") as f:
            data = f.read()
        return load_state_dict_from_bytes(data) if data[:4] == b"FTSV" else load_safetensors_from_bytes(data)
    except (OSError, SerializeError, ValueError, KeyError, struct.error) as e:
        raise TensorIOError.classify(e, path) from e


def save_safetensors_to_bytes(sd: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> bytes:
    header, chunks, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for k in sorted(sd):
        t = sd[k]
        if t.dtype not in _ST_NAME:
            raise SerializeError("UnsupportedDType", f"{k}: dtype {t.dtype} is not storable")
        b = _raw_bytes(t)
        header[k] = {"dtype": _ST_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        chunks.append(b)
        off += len(b)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    return struct.pack("<Q", len(hb)) + hb + b"".join(chunks)


def save_safetensors(sd: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    data = save_safetensors_to_bytes(sd, metadata)
    with open(path, "wb") as f:
        f.write(data)


def _st_header(data: bytes):
    if len(data) < 8:
        raise SerializeError("Truncated", "safetensors file shorter than its length prefix")
    (hl,) = struct.unpack_from("<Q", data, 0)
    if hl > len(data) - 8 or hl > (100 << 20):
        raise SerializeError("Truncated", "safetensors header length exceeds the file")
    try:
        return json.loads(data[8: 8 + hl]), 8 + hl
    except json.JSONDecodeError as e:
        raise SerializeError("InvalidJson", f"safetensors header is not valid json: {e.msg}")
    except (UnicodeDecodeError, RecursionError) as e:
        raise SerializeError("InvalidJson", f"safetensors header is not valid json: {type(e).__name__}")


def load_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        return load_safetensors_from_bytes(f.read())


def load_safetensors_from_bytes(data: bytes) -> Dict[str, torch.Tensor]:
    """Every malformed input ends in a ``SerializeError``: the header must be an object of tensor records with a
    known dtype, integer offsets inside the file, a shape of non-negative integers whose volume fits the index
    range, and exactly ``volume * element size`` bytes of data."""
    header, base = _st_header(data)
    if not isinstance(header, dict):
        raise SerializeError("InvalidJson", "safetensors header is not an object")
    out = {}
    for k, info in header.items():
        if k == "__metadata__":
            continue
        if not isinstance(info, dict) or not {"dtype", "shape", "data_offsets"} <= set(info):
            raise SerializeError("InvalidJson", f"{k}: a tensor record needs dtype, shape and data_offsets")
        if not isinstance(info["dtype"], str) or info["dtype"] not in _ST_DTYPE:
            raise SerializeError("UnsupportedDType", f"{k}: dtype {info['dtype']!r} is not supported")
        offs, shape = info["data_offsets"], info["shape"]
        if not (isinstance(offs, list) and len(offs) == 2 and all(type(o) is int for o in offs)):
            raise SerializeError("InvalidJson", f"{k}: data_offsets must be two integers")
        a, b = offs
        if not (0 <= a <= b <= len(data) - base):
            raise SerializeError("Truncated", f"{k}: data offsets outside the file")
        if not (isinstance(shape, list) and all(type(d) is int and d >= 0 for d in shape)) or len(shape) > 64:
            raise SerializeError("InvalidShape", f"{k}: shape must be a list of non-negative integers")
        numel, span = 1, 1
        for d in shape:
            numel *= d
            span *= max(d, 1)
            if span > (1 << 62):
                raise SerializeError("ShapeOverflow", f"{k}: shape volume overflows")
        dt = _ST_DTYPE[info["dtype"]]
        esize = torch.empty(0, dtype=dt).element_size()
        if b - a != numel * esize:
            raise SerializeError("Truncated", f"{k}: {b - a} bytes of data for {numel} elements of {esize} bytes")
        raw = bytearray(data[base + a: base + b])
        if dt == torch.bfloat16:
            t = torch.frombuffer(raw, dtype=torch.int16).view(torch.bfloat16) if raw else torch.empty(0, dtype=dt)
        else:
            t = torch.frombuffer(raw, dtype=dt) if raw else torch.empty(0, dtype=dt)
        out[k] = t.reshape(shape).clone()
    return out


def load_safetensors_metadata(path: str) -> Dict[str, str]:
    with open(path, "rb") as f:
        header, _ = _st_header(f.read())
    meta = header.get("__metadata__", {}) if isinstance(header, dict) else {}
    if not isinstance(meta, dict):
        raise SerializeError("InvalidJson", "__metadata__ is not an object")
    return {str(k): str(v) for k, v in meta.items()}


# -------------------------------------------------------------------------------------- ONNX (one Linear)
def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + (_varint(len(payload)) + payload if wire == 2 else payload)


def _str(num, s):
    return _field(num, 2, s.encode())


def _int(num, v):
    return _field(num, 0, _varint(v))


def _tensor_proto(name: str, arr: np.ndarray) -> bytes:
    body = b"".join(_int(1, d) for d in arr.shape) + _int(2, 1) + _str(8, name) + _field(9, 2, arr.astype("<f4").tobytes())
    return body


def _value_info(name: str, shape) -> bytes:
    dims = b"".join(_field(1, 2, (_int(1, d) if isinstance(d, int) else _str(2, d))) for d in shape)
    tensor_type = _int(1, 1) + _field(2, 2, dims)
    return _str(1, name) + _field(2, 2, _field(1, 2, tensor_type))


def _node(op: str, inputs, outputs, name: str) -> bytes:
    return b"".join(_str(1, i) for i in inputs) + b"".join(_str(2, o) for o in outputs) + _str(3, name) + _str(4, op)


def export_linear_onnx_to_bytes(weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                                producer: str = "frankentorch_b200") -> bytes:
    """``y = x @ W^T (+ b)`` as an ONNX ModelProto (IR 8, opset 17)."""
    if weight.dim() != 2:
        raise SerializeError("InvalidShape", "Linear weight must be 2-D [out, in]")
    out_f, in_f = weight.shape
    if bias is not None and tuple(bias.shape) != (out_f,):
        raise SerializeError("InvalidShape", "bias must be [out]")
    wt = weight.detach().float().t().contiguous().numpy()
    nodes = [_field(1, 2, _node("MatMul", ["x", "weight_t"], ["mm"], "linear_matmul"))]
    inits = [_field(5, 2, _tensor_proto("weight_t", wt))]
    if bias is not None:
        nodes.append(_field(1, 2, _node("Add", ["mm", "bias"], ["y"], "linear_add")))
        inits.append(_field(5, 2, _tensor_proto("bias", bias.detach().float().numpy())))
    else:
        nodes.append(_field(1, 2, _node("Identity", ["mm"], ["y"], "linear_identity")))
    graph = (b"".join(nodes) + _str(2, "linear") + b"".join(inits)
             + _field(11, 2, _value_info("x", ["batch", in_f])) + _field(12, 2, _value_info("y", ["batch", out_f])))
    model = _int(1, 8) + _str(2, producer) + _field(7, 2, graph) + _field(8, 2, _str(1, "") + _int(2, 17))
    return model


def save_linear_onnx(weight: torch.Tensor, bias: Optional[torch.Tensor], path: str, producer: str = "frankentorch_b200") -> int:
    """Write ``export_linear_onnx_to_bytes`` to ``path``; returns the byte count (ft-serialize/src/lib.rs:1539)."""
    data = export_linear_onnx_to_bytes(weight, bias, producer)
    with open(path, "wb") as f:
        f.write(data)
    return len(data)
