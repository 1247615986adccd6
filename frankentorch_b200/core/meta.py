"""Tensor metadata, device identity and deterministic fingerprints.

Reference: ft-core/src/lib.rs - ``Device`` :176, ``QuantizationParams`` :188, ``TensorMeta`` :340
(validation of rank/stride agreement and offset overflow), ``is_contiguous`` :580 (size-1 dims
ignored), ``storage_index_for`` :609, ``fingerprint64`` :648 over an FNV-1a hasher :660-679;
ft-device/src/lib.rs - ``DeviceGuard`` :35, ``ensure_same_device`` :62.
"""
from __future__ import annotations

import enum
import math
import struct
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

from ..runtime import native
from .dtype import DType

U64_MAX = (1 << 64) - 1


class Device(enum.Enum):
    Cpu = "Cpu"
    Cuda = "Cuda"

    @staticmethod
    def parse(name) -> "Device":
        if isinstance(name, Device):
            return name
        s = str(name).lower()
        if s == "cpu":
            return Device.Cpu
        if s == "cuda":
            return Device.Cuda
        raise DeviceError(f"unknown device {name!r}")


class TensorMetaError(ValueError):
    pass


class TensorCompatError(ValueError):
    pass


class DeviceError(ValueError):
    pass


class QuantizationParams:
    """Affine quantization parameters of a tensor (ft-core/src/lib.rs:188): one ``(scale, zero_point)`` for the whole
    tensor, or one per slice of ``axis``.  Scales must be finite and positive; equality and hashing use the scales'
    bit patterns."""
    __slots__ = ("_scales", "_zero_points", "_axis")

    def __init__(self, scale: float = 1.0, zero_point: int = 0):
        self._scales = (self._check(scale),)
        self._zero_points = (int(zero_point),)
        self._axis: Optional[int] = None

    @staticmethod
    def _check(scale: float) -> float:
        scale = float(scale)
        if not math.isfinite(scale) or scale <= 0.0:
            raise TensorMetaError(f"invalid quantization scale {scale!r}: must be finite and > 0")
        return scale

    @staticmethod
    def per_channel(scales: Sequence[float], zero_points: Sequence[int], axis: int) -> "QuantizationParams":
        if len(scales) == 0:
            raise TensorMetaError("per-channel quantization needs at least one channel")
        if len(scales) != len(zero_points):
            raise TensorMetaError(f"quantization vector length mismatch: {len(scales)} scales vs {len(zero_points)} zero points")
        q = QuantizationParams.__new__(QuantizationParams)
        q._scales = tuple(QuantizationParams._check(s) for s in scales)
        q._zero_points = tuple(int(z) for z in zero_points)
        q._axis = int(axis)
        return q

    scale = property(lambda self: self._scales[0])
    zero_point = property(lambda self: self._zero_points[0])
    axis = property(lambda self: self._axis)

    def scales(self):
        return list(self._scales)

    def zero_points(self):
        return list(self._zero_points)

    def __len__(self) -> int:
        return len(self._scales)

    def is_per_channel(self) -> bool:
        return self._axis is not None

    def validate_for_shape(self, shape: Sequence[int]) -> None:
        if self._axis is None:
            if len(self._scales) != 1:
                raise TensorMetaError("per-tensor quantization carries exactly one scale")
            return
        if not 0 <= self._axis < len(shape):
            raise TensorMetaError(f"quantization axis {self._axis} out of range for rank {len(shape)}")
        if shape[self._axis] != len(self._scales):
            raise TensorMetaError(f"{len(self._scales)} quantization channels for extent {shape[self._axis]} of axis {self._axis}")

    def _key(self):
        return (tuple(struct.pack("<d", s) for s in self._scales), self._zero_points, self._axis)

    def __eq__(self, other):
        return isinstance(other, QuantizationParams) and other._key() == self._key()

    def __hash__(self):
        return hash(self._key())

    def __repr__(self):
        if self._axis is None:
            return f"QuantizationParams(scale={self.scale}, zero_point={self.zero_point})"
        return f"QuantizationParams.per_channel(scales={list(self._scales)}, zero_points={list(self._zero_points)}, axis={self._axis})"


def contiguous_strides(shape: Sequence[int]) -> Tuple[int, ...]:
    strides, acc = [], 1
    for s in reversed(shape):
        strides.append(acc)
        acc *= max(int(s), 1) if s == 0 else int(s)
    return tuple(reversed(strides))


@dataclass(frozen=True)
class TensorMeta:
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    storage_offset: int = 0
    dtype: DType = DType.F64
    device: Device = Device.Cpu
    quantization: Optional[QuantizationParams] = None

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_shape(shape: Sequence[int], dtype: DType = DType.F64, device: Device = Device.Cpu) -> "TensorMeta":
        return TensorMeta.from_shape_and_strides(shape, contiguous_strides(shape), 0, dtype, device)

    @staticmethod
    def from_shape_and_strides(shape, strides, storage_offset=0, dtype=DType.F64, device=Device.Cpu) -> "TensorMeta":
        shape, strides = tuple(int(s) for s in shape), tuple(int(s) for s in strides)
        if len(shape) != len(strides):
            raise TensorMetaError(f"rank/stride mismatch: shape rank {len(shape)} vs {len(strides)} strides")
        if any(s < 0 for s in shape) or any(s < 0 for s in strides) or storage_offset < 0:
            raise TensorMetaError("negative extent, stride or offset")
        numel = 1
        for s in shape:
            numel *= s
            if numel > U64_MAX:
                raise TensorMetaError("shape volume overflows")
        # largest reachable linear offset must fit in 64 bits
        span = 0
        for size, stride in zip(shape, strides):
            if size == 0:
                continue
            step = (size - 1) * stride
            if step > U64_MAX:
                raise TensorMetaError(f"stride overflow: size {size} stride {stride}")
            span += step
        if storage_offset + span > U64_MAX:
            raise TensorMetaError(f"storage offset overflow: offset {storage_offset} + span {span}")
        return TensorMeta(shape, strides, int(storage_offset), dtype, device)

    @staticmethod
    def quantized_from_shape(shape, dtype: DType, device: Device, scale: float, zero_point: int) -> "TensorMeta":
        return TensorMeta.from_shape(shape, dtype, device).with_quantization(QuantizationParams(scale, zero_point)).validated()

    @staticmethod
    def quantized_per_channel_from_shape(shape, dtype: DType, device: Device, scales, zero_points, axis: int) -> "TensorMeta":
        q = QuantizationParams.per_channel(scales, zero_points, axis)
        return TensorMeta.from_shape(shape, dtype, device).with_quantization(q).validated()

    @staticmethod
    def quantized_from_shape_and_strides(shape, strides, storage_offset, dtype: DType, device: Device, scale: float,
                                         zero_point: int) -> "TensorMeta":
        m = TensorMeta.from_shape_and_strides(shape, strides, storage_offset, dtype, device)
        return m.with_quantization(QuantizationParams(scale, zero_point)).validated()

    @staticmethod
    def quantized_per_channel_from_shape_and_strides(shape, strides, storage_offset, dtype: DType, device: Device, scales,
                                                     zero_points, axis: int) -> "TensorMeta":
        m = TensorMeta.from_shape_and_strides(shape, strides, storage_offset, dtype, device)
        return m.with_quantization(QuantizationParams.per_channel(scales, zero_points, axis)).validated()

    def with_quantization(self, quantization: QuantizationParams) -> "TensorMeta":
        return TensorMeta(self.shape, self.strides, self.storage_offset, self.dtype, self.device, quantization)

    def with_dtype(self, dtype: DType) -> "TensorMeta":
        """Same layout with another element type; quantization parameters survive only on a quantized dtype."""
        return TensorMeta(self.shape, self.strides, self.storage_offset, dtype, self.device,
                          self.quantization if dtype.is_quantized() else None)

    def validate(self) -> None:
        """A quantized dtype needs quantization parameters that fit the shape; any other dtype must carry none."""
        if self.dtype.is_quantized():
            if self.quantization is None:
                raise TensorMetaError(f"dtype {self.dtype.value} needs quantization parameters")
            self.quantization.validate_for_shape(self.shape)
        elif self.quantization is not None:
            raise TensorMetaError(f"dtype {self.dtype.value} must not carry quantization parameters")
        TensorMeta.from_shape_and_strides(self.shape, self.strides, self.storage_offset, self.dtype, self.device)

    def validated(self) -> "TensorMeta":
        self.validate()
        return self

    # ------------------------------------------------------------------ queries
    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def rank(self) -> int:
        return len(self.shape)

    def is_contiguous(self) -> bool:
        if len(self.shape) != len(self.strides):
            return False
        expected = 1
        for size, stride in zip(reversed(self.shape), reversed(self.strides)):
            if size == 1:
                continue
            if stride != expected:
                return False
            expected *= size
        return True

    def storage_index_for(self, index: Sequence[int]) -> int:
        if len(index) != len(self.shape):
            raise TensorMetaError(f"index rank mismatch: expected {len(self.shape)}, got {len(index)}")
        linear = self.storage_offset
        for dim, (idx, size, stride) in enumerate(zip(index, self.shape, self.strides)):
            if idx >= size or idx < 0:
                raise TensorMetaError(f"index {idx} out of bounds for dim {dim} of size {size}")
            linear += idx * stride
            if linear > U64_MAX:
                raise TensorMetaError("storage offset overflow")
        return linear

    def with_storage_offset(self, offset: int) -> "TensorMeta":
        return TensorMeta.from_shape_and_strides(self.shape, self.strides, offset, self.dtype, self.device)

    def fingerprint64(self) -> int:
        """FNV-1a over (shape, strides, offset, dtype, device, quantization), little-endian u64 words."""
        buf = bytearray()
        for seq in (self.shape, self.strides):
            buf += struct.pack("<Q", len(seq))
            for v in seq:
                buf += struct.pack("<Q", v & U64_MAX)
        buf += struct.pack("<Q", self.storage_offset)
        buf += struct.pack("<Q", list(DType).index(self.dtype))
        buf += struct.pack("<Q", list(Device).index(self.device))
        if self.quantization is None:
            buf += struct.pack("<Q", 0)
        else:
            q = self.quantization
            if not q.is_per_channel():           # the per-tensor encoding is unchanged
                buf += struct.pack("<Qdq", 1, q.scale, q.zero_point)
            else:
                buf += struct.pack("<QQQ", 2, q.axis, len(q))
                for sc, zp in zip(q.scales(), q.zero_points()):
                    buf += struct.pack("<dq", sc, zp)
        return native.fnv1a64(bytes(buf))


def ensure_compatible(lhs: TensorMeta, rhs: TensorMeta) -> None:
    if lhs.dtype != rhs.dtype:
        raise TensorCompatError(f"dtype mismatch: lhs={lhs.dtype.value}, rhs={rhs.dtype.value}")
    if lhs.device != rhs.device:
        raise TensorCompatError(f"device mismatch: lhs={lhs.device.value}, rhs={rhs.device.value}")


class DeviceGuard:
    """Asserts that tensors handed to a scope live on the guard's device (identity guard only)."""

    def __init__(self, device: Device):
        self.device = Device.parse(device)

    def ensure_tensor_device(self, meta: TensorMeta) -> None:
        if meta.device != self.device:
            raise DeviceError(f"device mismatch: expected {self.device.value}, got {meta.device.value}")

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def ensure_same_device(lhs: TensorMeta, rhs: TensorMeta) -> Device:
    if lhs.device != rhs.device:
        raise DeviceError(f"device mismatch: lhs={lhs.device.value}, rhs={rhs.device.value}")
    return lhs.device
