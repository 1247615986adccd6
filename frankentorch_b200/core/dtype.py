"""Dtype model and promotion rules (reference: ft-core/src/lib.rs:23-170)."""
from __future__ import annotations

import enum
from typing import Optional

import torch


class DType(enum.Enum):
    F64 = "F64"
    F32 = "F32"
    F16 = "F16"
    BF16 = "BF16"
    QInt8 = "QInt8"
    QUInt8 = "QUInt8"
    I64 = "I64"
    I32 = "I32"
    Bool = "Bool"
    Complex64 = "Complex64"
    Complex128 = "Complex128"

    # ------------------------------------------------------------------ predicates
    def element_size(self) -> int:
        return {DType.Complex128: 16, DType.F64: 8, DType.I64: 8, DType.Complex64: 8, DType.F32: 4, DType.I32: 4,
                DType.F16: 2, DType.BF16: 2, DType.QInt8: 1, DType.QUInt8: 1, DType.Bool: 1}[self]

    def is_floating_point(self) -> bool:
        return self in (DType.F64, DType.F32, DType.F16, DType.BF16)

    def is_half(self) -> bool:
        return self in (DType.F16, DType.BF16)

    def is_integer(self) -> bool:
        return self in (DType.I32, DType.I64)

    def is_quantized(self) -> bool:
        return self in (DType.QInt8, DType.QUInt8)

    def is_bool(self) -> bool:
        return self is DType.Bool

    def is_complex(self) -> bool:
        return self in (DType.Complex64, DType.Complex128)

    # ------------------------------------------------------------------ promotion
    def promote(self, other: "DType") -> Optional["DType"]:
        """Strict promotion among float / complex types only; ``None`` for everything else."""
        a, b = self, other
        C128, C64, F64, F32, F16, BF16 = (DType.Complex128, DType.Complex64, DType.F64, DType.F32, DType.F16, DType.BF16)
        floats = (F64, F32, F16, BF16)
        if a.is_complex() and b.is_complex():
            return C128 if C128 in (a, b) else C64
        if (a is C128 and b in floats) or (b is C128 and a in floats):
            return C128
        if {a, b} == {C64, F64}:
            return C128
        if (a is C64 and b in (F32, F16, BF16)) or (b is C64 and a in (F32, F16, BF16)):
            return C64
        if a in floats and b in floats:
            if a is b:
                return a
            if {a, b} == {F16, BF16}:
                return F32
            if F64 in (a, b):
                return F64
            return F32
        return None

    def promote_types(self, other: "DType") -> "DType":
        """Total promotion following PyTorch's hierarchy (bool < quantized < ints < halves < floats < complex)."""
        if self is other:
            return self
        if {self, other} == {DType.F16, DType.BF16}:
            return DType.F32
        if {self, other} == {DType.Complex64, DType.F64}:
            return DType.Complex128
        rank = {DType.Bool: 0, DType.QInt8: 1, DType.QUInt8: 1, DType.I32: 2, DType.I64: 3, DType.F16: 4,
                DType.BF16: 4, DType.F32: 5, DType.F64: 6, DType.Complex64: 7, DType.Complex128: 8}
        return self if rank[self] >= rank[other] else other

    # ------------------------------------------------------------------ torch bridge
    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        return _FROM_TORCH[dt]

    @staticmethod
    def parse(name) -> "DType":
        if isinstance(name, DType):
            return name
        for d in DType:
            if d.value.lower() == str(name).lower():
                return d
        raise ValueError(f"unknown dtype {name!r}")


_TO_TORCH = {DType.F64: torch.float64, DType.F32: torch.float32, DType.F16: torch.float16, DType.BF16: torch.bfloat16,
             DType.QInt8: torch.qint8, DType.QUInt8: torch.quint8, DType.I64: torch.int64, DType.I32: torch.int32,
             DType.Bool: torch.bool, DType.Complex64: torch.complex64, DType.Complex128: torch.complex128}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}
