"""Dispatch keys, key sets, strict / hardened resolution and decision records.

Reference: ft-dispatch/src/lib.rs - ``DispatchKey`` :493, ``TYPE_PRIORITY`` :520,
``DispatchKeySet`` :538 (``from_bits_checked`` :557, ``validate_for_scalar_binary`` :629),
``DispatchKeyError`` :650, ``DispatchDecision`` :680, ``resolve_dispatch_keys`` :1361-1393,
``dispatch_scalar_binary[_with_keyset]`` :1395.  The resolution itself runs in the native
runtime (``ftc_dispatch_resolve``).

This framework has ONE accelerator backend, ``SM100`` (+ ``AutogradSM100``): hand-written
sm_100a kernels.  ``CPU`` / ``AutogradCPU`` remain for the f64 reference path used by the
conformance suite; composite and backend-select keys only ever resolve through the hardened
fallback, exactly as in the reference.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Iterable, List, Optional, Tuple

from ..core.dtype import DType
from ..core.meta import Device, TensorCompatError
from ..runtime import native
from ..runtime.ledger import ExecutionMode


class DispatchKey(enum.IntEnum):
    Undefined = 0
    BackendSelect = 1
    CompositeImplicitAutograd = 2
    CompositeExplicitAutograd = 3
    CPU = 4
    AutogradCPU = 5
    SM100 = 6
    AutogradSM100 = 7

    def bit(self) -> int:
        return 1 << int(self)

    @staticmethod
    def all() -> List["DispatchKey"]:
        return [k for k in DispatchKey if k is not DispatchKey.Undefined]

    @staticmethod
    def parse(name: str) -> "DispatchKey":
        for k in DispatchKey:
            if k.name == name:
                return k
        raise DispatchKeyError("unknown", f"unknown dispatch key {name!r}")


class DispatchKeyError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


class DispatchError(ValueError):
    pass


_RESOLVE_ERRORS = {
    1: ("EmptySet", "dispatch keyset is empty"),
    2: ("NoTypeKey", "dispatch keyset has no resolvable type key"),
    3: ("NoBackendKey", "dispatch keyset has no backend key"),
    4: ("UnknownBits", "dispatch keyset has unknown bitmask"),
    5: ("IncompatibleSet", "incompatible dispatch keyset: an Autograd key requires its backend key"),
    6: ("IncompatibleSet", "incompatible dispatch keyset: strict mode forbids composite/backend fallback routing"),
    7: ("IncompatibleSet", "incompatible dispatch keyset: resolved key/backend key drifted to incompatible pair"),
}


class DispatchKeySet:
    __slots__ = ("bits",)

    def __init__(self, bits: int = 0):
        self.bits = int(bits)

    @staticmethod
    def empty() -> "DispatchKeySet":
        return DispatchKeySet(0)

    @staticmethod
    def from_keys(keys: Iterable[DispatchKey]) -> "DispatchKeySet":
        ks = DispatchKeySet(0)
        for k in keys:
            ks.add(k)
        return ks

    @staticmethod
    def from_bits_checked(bits: int) -> "DispatchKeySet":
        known = 0
        for k in DispatchKey.all():
            known |= k.bit()
        unknown = bits & ~known
        if unknown:
            raise DispatchKeyError("UnknownBits", f"dispatch keyset has unknown bitmask 0x{unknown:016x}")
        return DispatchKeySet(bits)

    def add(self, key: DispatchKey) -> None:
        self.bits |= key.bit()

    def remove(self, key: DispatchKey) -> None:
        self.bits &= ~key.bit()

    def has(self, key: DispatchKey) -> bool:
        return bool(self.bits & key.bit())

    def is_empty(self) -> bool:
        return self.bits == 0

    def union(self, other: "DispatchKeySet") -> "DispatchKeySet":
        return DispatchKeySet(self.bits | other.bits)

    def intersection(self, other: "DispatchKeySet") -> "DispatchKeySet":
        return DispatchKeySet(self.bits & other.bits)

    def validate_for_scalar_binary(self) -> None:
        resolve(ExecutionMode.Hardened, self)   # hardened accepts every valid set

    def __eq__(self, other):
        return isinstance(other, DispatchKeySet) and other.bits == self.bits

    def __repr__(self):
        return "DispatchKeySet(" + "|".join(k.name for k in DispatchKey.all() if self.has(k)) + ")"


def resolve(mode: ExecutionMode, keyset: DispatchKeySet) -> Tuple[DispatchKey, DispatchKey, DispatchKey, bool]:
    """``(selected_key, backend_key, effective_key, fallback_used)`` or a typed error."""
    out = (C.c_int * 4)()
    rc = native.load().ftc_dispatch_resolve(keyset.bits & ((1 << 64) - 1), int(mode == ExecutionMode.Hardened), out)
    if rc != 0:
        kind, msg = _RESOLVE_ERRORS[rc]
        raise DispatchKeyError(kind, msg)
    return DispatchKey(out[0]), DispatchKey(out[1]), DispatchKey(out[2]), bool(out[3])


def keyset_for(device: Device, requires_grad: bool) -> DispatchKeySet:
    ks = DispatchKeySet.from_keys([DispatchKey.BackendSelect])
    if device == Device.Cpu:
        ks.add(DispatchKey.CPU)
        if requires_grad:
            ks.add(DispatchKey.AutogradCPU)
    elif device == Device.Cuda:
        ks.add(DispatchKey.SM100)
        if requires_grad:
            ks.add(DispatchKey.AutogradSM100)
    return ks


@dataclass(frozen=True)
class DispatchDecision:
    op: str
    mode: ExecutionMode
    kernel: str
    selected_key: DispatchKey
    backend_key: DispatchKey
    keyset_bits: int
    fallback_used: bool
    deviation: Optional[str] = None      # allow-list id of the hardened-mode deviation that fired, if any

    def summary(self) -> str:
        s = (f"op={self.op} mode={self.mode.value} kernel={self.kernel} dispatch_key={self.selected_key.name} "
             f"backend_key={self.backend_key.name} keyset_bits=0x{self.keyset_bits:x} "
             f"fallback_path={str(self.fallback_used).lower()}")
        return s + (f" deviation={self.deviation}" if self.deviation else "")


_KERNEL_NS = {DispatchKey.AutogradCPU: "autograd_cpu", DispatchKey.CPU: "cpu",
              DispatchKey.AutogradSM100: "autograd_sm100", DispatchKey.SM100: "sm100"}


def decide(op: str, mode: ExecutionMode, keyset: DispatchKeySet, kernel_suffix: str, *,
           kernel: Optional[str] = None, deviation: Optional[str] = None) -> DispatchDecision:
    """Resolve the key set and name the kernel.  ``kernel`` (a full name such as
    ``ftk::norm_fwd_kernel<layer_norm>``) replaces the default ``<namespace>::<suffix>`` string when the
    caller knows which kernel it launched; ``deviation`` marks a hardened-mode fallback."""
    selected, backend, effective, fallback = resolve(mode, keyset)
    name = kernel if kernel is not None else f"{_KERNEL_NS[effective]}::{kernel_suffix}"
    return DispatchDecision(op, mode, name, selected, backend, keyset.bits, fallback or deviation is not None,
                            deviation)


def ensure_meta_compatible(lhs_dtype: DType, rhs_dtype: DType, lhs_device: Device, rhs_device: Device) -> None:
    if lhs_dtype != rhs_dtype:
        raise TensorCompatError(f"dtype mismatch: lhs={lhs_dtype.value}, rhs={rhs_dtype.value}")
    if lhs_device != rhs_device:
        raise TensorCompatError(f"device mismatch: lhs={lhs_device.value}, rhs={rhs_device.value}")


_SCALAR_OPS = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
    "min": min, "max": max,
}


def dispatch_scalar_binary(op: str, mode: ExecutionMode, lhs: float, rhs: float, requires_grad: bool = False,
                           keyset: Optional[DispatchKeySet] = None, lhs_dtype: DType = DType.F64,
                           rhs_dtype: DType = DType.F64, lhs_device=Device.Cpu, rhs_device=Device.Cpu):
    """Scalar binary op with full key resolution; returns ``(value, DispatchDecision)``."""
    lhs_device, rhs_device = Device.parse(lhs_device), Device.parse(rhs_device)
    ensure_meta_compatible(lhs_dtype, rhs_dtype, lhs_device, rhs_device)
    if keyset is None:
        keyset = keyset_for(lhs_device, requires_grad)
    if op not in _SCALAR_OPS:
        if op in ("matmul", "dot", "outer", "bmm"):
            raise DispatchKeyError("IncompatibleSet", "matmul/dot/outer/bmm is unsupported for scalar tensors")
        raise DispatchError(f"unknown scalar binary op {op!r}")
    decision = decide(op, mode, keyset, f"{op}_scalar")
    if decision.backend_key is not DispatchKey.CPU:
        raise DispatchKeyError("NoBackendKey", "scalar tensors live on the CPU backend")
    return float(_SCALAR_OPS[op](lhs, rhs)), decision
