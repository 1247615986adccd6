"""Option enums of the ``nn`` layer (ft-nn/src/lib.rs: ``Reduction`` :15589, ``CTCReduction`` :16159,
``DistanceKind`` :15936, ``EmbeddingBagMode`` :3162, ``PaddingMode`` :7279, ``TransformerActivation`` :14559,
``UpsampleMode`` :10210).

Every member is also the string that the modules and the session operators take (``Reduction.Mean == "mean"``),
so a module accepts either spelling; ``parse`` turns a string (any case, ``-`` or ``_``) into the member.
"""
from __future__ import annotations

import enum


class _StrEnum(str, enum.Enum):
    def __str__(self) -> str:
        return self.value

    def __format__(self, spec) -> str:
        return format(self.value, spec)

    @classmethod
    def parse(cls, v):
        if isinstance(v, cls):
            return v
        key = str(v).lower().replace("_", "-")
        for m in cls:
            if m.value.replace("_", "-") == key or m.name.lower() == key.replace("-", ""):
                return m
        raise ValueError(f"unknown {cls.__name__} {v!r}")


class Reduction(_StrEnum):
    NoReduction = "none"      # the reference's ``None`` variant
    Mean = "mean"
    Sum = "sum"


class CTCReduction(_StrEnum):
    NoReduction = "none"      # per-sample losses [N]
    Sum = "sum"
    Mean = "mean"             # per-sample loss / target length, then the batch mean


class DistanceKind(_StrEnum):
    L2 = "l2"
    L1 = "l1"
    Cosine = "cosine"


class EmbeddingBagMode(_StrEnum):
    Sum = "sum"
    Mean = "mean"
    Max = "max"


class PaddingMode(_StrEnum):
    Zeros = "zeros"
    Reflect = "reflect"
    Replicate = "replicate"
    Circular = "circular"

    def pad_mode(self) -> str:
        """Mode string of ``tensor_pad_mode`` (zero padding is its ``constant`` mode)."""
        return "constant" if self is PaddingMode.Zeros else self.value


class TransformerActivation(_StrEnum):
    Relu = "relu"
    Gelu = "gelu"


class UpsampleMode(_StrEnum):
    Nearest = "nearest"
    NearestExact = "nearest-exact"
    Linear = "linear"
    Bilinear = "bilinear"
    Bicubic = "bicubic"
    Trilinear = "trilinear"
    Area = "area"
