"""Scalar tensors and typed storage (ft-core/src/lib.rs:827 ``ScalarTensor``, :915 ``TensorStorage``).

``ScalarTensor`` is the value type of the scalar tape and of the scalar dispatch entry points: one f64
value with its own tensor id, a storage id shared by alias views, a version counter that every in-place
write and every ``with_value`` derivative bumps, and an evidence fingerprint over all of these.

``TensorStorage`` is a flat, dtype-tagged buffer: the variants of the reference's enum (F32, F64, F16, BF16,
QInt8, QUInt8, Complex64, Complex128) are the element types it admits.  It wraps a contiguous
``torch.Tensor`` on either device, so a result of the GPU backend is a storage without a host copy; the
``as_<dtype>()`` accessors answer ``None`` for a different variant (the reference returns ``Option``) and
``to_f64_vec`` / ``to_f32_vec`` convert on the host.
"""
from __future__ import annotations

import itertools
import struct
from typing import List, Optional, Sequence

import torch

from ..runtime import native
from .dtype import DType
from .meta import Device, TensorMeta, TensorMetaError

_NEXT_TENSOR_ID = itertools.count(1 << 32)      # distinct from the dense tensors' id range
_NEXT_STORAGE_ID = itertools.count(1 << 32)
_U64 = (1 << 64) - 1


class ScalarTensor:
    __slots__ = ("_id", "_storage_id", "_meta", "_value", "_version")

    def __init__(self, value: float, dtype: DType = DType.F64, device: Device = Device.Cpu, *, _storage_id=None,
                 _meta: Optional[TensorMeta] = None, _version: int = 0):
        self._id = next(_NEXT_TENSOR_ID)
        self._storage_id = next(_NEXT_STORAGE_ID) if _storage_id is None else _storage_id
        self._meta = _meta if _meta is not None else TensorMeta.from_shape_and_strides((), (), 0, dtype, Device.parse(device))
        self._value = float(value)
        self._version = _version

    def with_value(self, value: float) -> "ScalarTensor":
        """A new tensor (new id, new storage) with this one's metadata and the next version."""
        return ScalarTensor(value, _meta=self._meta, _version=min(self._version + 1, _U64))

    def alias_view(self, storage_offset: int) -> "ScalarTensor":
        """A view on the same storage at ``storage_offset`` (validated by the metadata)."""
        if storage_offset < 0:
            raise TensorMetaError("storage offset must be non-negative")
        meta = self._meta.with_storage_offset(storage_offset)
        return ScalarTensor(self._value, _storage_id=self._storage_id, _meta=meta, _version=self._version)

    def set_in_place(self, value: float) -> None:
        self._value = float(value)
        self._version = min(self._version + 1, _U64)

    id = property(lambda self: self._id)
    storage_id = property(lambda self: self._storage_id)
    value = property(lambda self: self._value)
    meta = property(lambda self: self._meta)
    version = property(lambda self: self._version)

    def evidence_fingerprint64(self) -> int:
        buf = struct.pack("<QQQQd", self._id & _U64, self._storage_id & _U64, self._version & _U64,
                          self._meta.fingerprint64(), self._value)
        return native.fnv1a64(buf)

    def __eq__(self, other):
        return (isinstance(other, ScalarTensor) and other._value == self._value and other._meta == self._meta
                and other._id == self._id)

    def __repr__(self):
        return f"ScalarTensor(id={self._id}, value={self._value}, dtype={self._meta.dtype.value}, version={self._version})"


_VARIANTS = (DType.F32, DType.F64, DType.F16, DType.BF16, DType.QInt8, DType.QUInt8, DType.Complex64, DType.Complex128)
_QTORCH = {DType.QInt8: torch.int8, DType.QUInt8: torch.uint8}


class TensorStorage:
    """Flat typed buffer.  ``data`` is a contiguous 1-D ``torch.Tensor``; quantized variants hold the raw
    integer codes (scale and zero point live in the tensor metadata)."""
    __slots__ = ("dtype", "data")

    def __init__(self, dtype: DType, data: torch.Tensor):
        if dtype not in _VARIANTS:
            raise ValueError(f"TensorStorage has no {dtype.value} variant")
        want = _QTORCH.get(dtype) or dtype.to_torch()
        if data.dtype != want:
            raise ValueError(f"storage variant {dtype.value} needs {want}, got {data.dtype}")
        self.dtype = dtype
        self.data = data.reshape(-1) if data.is_contiguous() else data.contiguous().reshape(-1)

    @staticmethod
    def from_tensor(t: torch.Tensor) -> "TensorStorage":
        if t.dtype in (torch.int8, torch.uint8):
            return TensorStorage(DType.QInt8 if t.dtype == torch.int8 else DType.QUInt8, t)
        return TensorStorage(DType.from_torch(t.dtype), t)

    @staticmethod
    def from_values(values: Sequence[float], dtype: DType = DType.F64) -> "TensorStorage":
        return TensorStorage(dtype, torch.tensor(list(values), dtype=_QTORCH.get(dtype) or dtype.to_torch()))

    def __len__(self) -> int:
        return self.data.numel()

    def is_empty(self) -> bool:
        return self.data.numel() == 0

    def _as(self, dtype: DType) -> Optional[torch.Tensor]:
        return self.data if self.dtype == dtype else None

    def as_f64(self): return self._as(DType.F64)                    # noqa: E704
    def as_f32(self): return self._as(DType.F32)                    # noqa: E704
    def as_f16(self): return self._as(DType.F16)                    # noqa: E704
    def as_bf16(self): return self._as(DType.BF16)                  # noqa: E704
    def as_qint8(self): return self._as(DType.QInt8)                # noqa: E704
    def as_quint8(self): return self._as(DType.QUInt8)              # noqa: E704
    def as_complex64(self): return self._as(DType.Complex64)        # noqa: E704
    def as_complex128(self): return self._as(DType.Complex128)      # noqa: E704

    def to_f64_vec(self) -> List[float]:
        """Host list in f64 (complex variants give their real parts, as the reference does)."""
        d = self.data.detach()
        if d.is_complex():
            d = d.real
        return d.to("cpu", torch.float64).tolist()

    def to_f32_vec(self) -> List[float]:
        d = self.data.detach()
        if d.is_complex():
            d = d.real
        return d.to("cpu", torch.float32).tolist()

    def __eq__(self, other):
        return isinstance(other, TensorStorage) and other.dtype == self.dtype and torch.equal(other.data, self.data)

    def __repr__(self):
        return f"TensorStorage.{self.dtype.value}(len={len(self)}, device={self.data.device})"
