"""``FrankenTorchSession``: the public API facade.

A session owns a scalar tape, a tensor tape (the Deterministic Autograd Contract), a runtime
context (execution mode + evidence ledger) and a deterministic PRNG.  All tensors are handled
through integer node ids; every method that creates a tensor returns the id of a new tape
node, every op records a dispatch decision in the ledger and every backward records its
scheduler telemetry.

The surface mirrors the reference session (ft-api; reconstructed from its call sites in
ft-nn / ft-optim / ft-data / ft-conformance): ``tensor_variable``, ``tensor_values``,
``tensor_<op>`` for the operator families, ``tensor_backward[_with_options]``,
``tensor_gradient``, ``tensor_accumulated_gradient``, ``no_grad_enter/exit``,
``tensor_apply_function``, ``checkpoint``, ``evidence`` and the scalar DAC calls
``variable/value/add/sub/mul/div/backward/gradient``.  Index and label tensors may be passed
as float-valued tensors (ft-conformance/tests/e2e_training.rs:289).

``device="cpu"`` (default) is the f64 reference path on PyTorch CPU operators.  ``device="cuda"``
is the sm_100a backend: the operator entry point looks each call up in the kernel registry
(:mod:`frankentorch_b200.dispatch.sm100`).  linear / matmul / bmm / layer_norm / rms_norm / softmax /
gelu / add / embedding / sdpa / cross_entropy / dropout on bf16 operands run the hand-written
kernels and the ledger names the kernel that was launched; layout operators are recorded as such;
any other operator is refused in strict mode and runs the PyTorch CUDA operator in hardened mode,
recorded with ``fallback_path=true`` and an allow-listed deviation id.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import math
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .autograd import functions as _f1  # noqa: F401  (populate the rule table)
from .autograd import functions_nn as _f3  # noqa: F401
from .autograd import functions_shape as _f2  # noqa: F401
from .autograd import functions_extra as _f4  # noqa: F401
from .autograd import functions_sparse as _f5  # noqa: F401
from .autograd import functions_parity as _f6  # noqa: F401
from .autograd.functions import OPS, OpDef
from .autograd.scalar_tape import BackwardReport, Tape
from .autograd.tape import (BackwardOptions, BorrowedInputVersionMismatch, TensorBackwardReport, TensorHookHandle,
                            TensorTape)
from .core.dtype import DType
from .core.meta import Device, TensorMeta
from .dispatch.keys import DispatchDecision, decide, keyset_for
from .runtime import native
from .runtime.ledger import EvidenceEntry, EvidenceKind, ExecutionMode, RuntimeContext

DEFAULT_SEED = 42


class SessionError(RuntimeError):
    pass


class Xoshiro256pp:
    """xoshiro256++ seeded through splitmix64; uniforms use the top 53 bits (native core)."""

    def __init__(self, seed: int = DEFAULT_SEED):
        self._lib = native.load()
        self.state = (C.c_uint64 * 4)()
        self.seed(seed)

    def seed(self, seed: int) -> None:
        self._lib.ftc_xoshiro_seed(self.state, int(seed) & ((1 << 64) - 1))

    def next_u64(self) -> int:
        return int(self._lib.ftc_xoshiro_next_u64(self.state))

    def uniform(self, n: int) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float64)
        if n:
            self._lib.ftc_xoshiro_fill_uniform(self.state, out.data_ptr(), n)
        return out

    def normal(self, n: int) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float64)
        if n:
            self._lib.ftc_xoshiro_fill_normal(self.state, out.data_ptr(), n)
        return out

    def get_state(self) -> List[int]:
        return [int(x) for x in self.state]

    def set_state(self, st: Sequence[int]) -> None:
        for i in range(4):
            self.state[i] = int(st[i])


class FunctionCtx:
    """Context handed to custom autograd functions (ft-autograd/src/lib.rs:1451-1489)."""

    def __init__(self, needs_input_grad: Sequence[bool]):
        self.needs_input_grad = tuple(needs_input_grad)
        self._saved: List[torch.Tensor] = []

    def save_for_backward(self, *tensors: torch.Tensor) -> None:
        self._saved = [t for t in tensors]

    @property
    def saved_tensors(self) -> List[torch.Tensor]:
        return self._saved

    @property
    def saved_shapes(self) -> List[Tuple[int, ...]]:
        return [tuple(t.shape) for t in self._saved]


class FrankenTorchSession:
    def __init__(self, mode: Optional[ExecutionMode] = None, device: str = "cpu", seed: int = DEFAULT_SEED,
                 default_dtype: Optional[DType] = None, ledger_dispatch: bool = True):
        if mode is None:   # the FT_MODE switch picks the mode of sessions that do not name one
            from .utils.config import env_flag
            mode = env_flag("FT_MODE")
        self.runtime = RuntimeContext(ExecutionMode.parse(mode))
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        self.default_dtype = default_dtype or (DType.BF16 if self.is_cuda else DType.F64)
        # gradient space: f64 on the CPU reference path, native kernel dtypes on the GPU
        self.tensor_tape = TensorTape(grad_dtype=None if self.is_cuda else torch.float64)
        if self.is_cuda:
            from .ops import kernels as K
            self.tensor_tape.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
        self.tape = Tape(self.runtime.mode)
        self.rng = Xoshiro256pp(seed)
        self._seed = int(seed)
        self._no_grad_depth = 0
        self._autocast: Optional[DType] = None
        self._ledger_dispatch = ledger_dispatch
        self.last_decision: Optional[DispatchDecision] = None
        # typed record of the last operator run through autograd/events.py; set ``operation_events`` to a list to keep all
        self.last_operation_event = None
        self.operation_events: Optional[list] = None
        self._dropout_calls = 0          # Philox offset of the next dropout on the GPU backend
        self._device_enum = Device.Cuda if self.is_cuda else Device.Cpu
        self.runtime.ledger.record(EvidenceKind.Policy,
                                   f"session device={self.device} default_dtype={self.default_dtype.value} seed={seed}")
        if not self.is_cuda:
            # thread width of the CPU reference kernels (FT_CPU_THREADS), decided once per process
            from .runtime.cpu_pool import configure_cpu_threads, resolve_spec
            if resolve_spec():
                configure_cpu_threads(ledger=self.runtime.ledger)

    # ------------------------------------------------------------------ mode / evidence
    @property
    def mode(self) -> ExecutionMode:
        return self.runtime.mode

    def set_mode(self, mode: ExecutionMode) -> None:
        self.runtime.set_mode(mode)
        self.tape.mode = self.runtime.mode

    def evidence(self) -> List[EvidenceEntry]:
        return self.runtime.evidence()

    def _record_dispatch(self, op: str, requires_grad: bool, kernel: Optional[str] = None, *,
                         launched: Optional[str] = None, deviation: Optional[str] = None) -> DispatchDecision:
        """One Dispatch entry per operator call.  ``launched`` is the full name of the kernel that ran
        (sm_100a routes); ``deviation`` the allow-list id of a hardened-mode fallback."""
        decision = decide(op, self.runtime.mode, keyset_for(self._device_enum, requires_grad), kernel or op,
                          kernel=launched, deviation=deviation)
        if self._ledger_dispatch:
            self.runtime.ledger.record(EvidenceKind.Dispatch, decision.summary())
        self.last_decision = decision
        return decision

    # ------------------------------------------------------------------ scalar DAC
    def variable(self, value: float, requires_grad: bool = False) -> int:
        return self.tape.leaf(value, requires_grad)

    def value(self, nid: int) -> float:
        return self.tape.value(nid)

    def _scalar_binary(self, op: str, a: int, b: int) -> int:
        nid, decision = self.tape.binary(op, a, b)
        if self._ledger_dispatch:
            self.runtime.ledger.record(EvidenceKind.Dispatch, decision.summary())
        return nid

    def add(self, a: int, b: int) -> int:
        return self._scalar_binary("add", a, b)

    def sub(self, a: int, b: int) -> int:
        return self._scalar_binary("sub", a, b)

    def mul(self, a: int, b: int) -> int:
        return self._scalar_binary("mul", a, b)

    def div(self, a: int, b: int) -> int:
        return self._scalar_binary("div", a, b)

    def backward(self, root: int, options: Optional[BackwardOptions] = None) -> BackwardReport:
        rep = self.tape.backward(root, options or BackwardOptions.for_mode(self.runtime.mode))
        self.runtime.ledger.record(EvidenceKind.Backward, "scalar " + rep.telemetry.render(self.runtime.mode.value).replace("\n", " "))
        return rep

    @staticmethod
    def gradient(report: BackwardReport, nid: int) -> Optional[float]:
        return report.gradient(nid)

    # ------------------------------------------------------------------ grad mode
    def no_grad_enter(self) -> None:
        self._no_grad_depth += 1
        self.tensor_tape.grad_enabled = False

    def no_grad_exit(self) -> None:
        if self._no_grad_depth == 0:
            raise SessionError("no_grad_exit without a matching no_grad_enter")
        self._no_grad_depth -= 1
        self.tensor_tape.grad_enabled = self._no_grad_depth == 0

    def is_grad_enabled(self) -> bool:
        return self._no_grad_depth == 0

    def with_no_grad(self, fn: Callable[["FrankenTorchSession"], Any]) -> Any:
        self.no_grad_enter()
        try:
            return fn(self)
        finally:
            self.no_grad_exit()

    @contextlib.contextmanager
    def no_grad(self):
        self.no_grad_enter()
        try:
            yield self
        finally:
            self.no_grad_exit()

    @contextlib.contextmanager
    def autocast(self, dtype: DType = DType.BF16):
        """Inside the context matmul-class ops run with operands narrowed to ``dtype``."""
        prev, self._autocast = self._autocast, dtype
        self.runtime.ledger.record(EvidenceKind.Policy, f"autocast enter {dtype.value}")
        try:
            yield self
        finally:
            self._autocast = prev
            self.runtime.ledger.record(EvidenceKind.Policy, "autocast exit")

    # ------------------------------------------------------------------ tensor creation / reading
    def _as_tensor(self, values, shape, dtype: DType) -> torch.Tensor:
        t = values if isinstance(values, torch.Tensor) else torch.tensor(list(values), dtype=torch.float64)
        if shape is not None:
            n = 1
            for s in shape:
                n *= s
            if t.numel() != n:
                raise SessionError(f"{t.numel()} values do not fill shape {tuple(shape)}")
            t = t.reshape(tuple(shape))
        return t.to(device=self.device, dtype=dtype.to_torch())

    def tensor_variable(self, values, shape=None, requires_grad: bool = False, dtype: Optional[DType] = None) -> int:
        dt = dtype or (DType.F64 if not self.is_cuda else self.default_dtype)
        return self.tensor_tape.leaf(self._as_tensor(values, shape, dt), requires_grad)

    def tensor_variable_f32(self, values, shape=None, requires_grad: bool = False) -> int:
        return self.tensor_variable(values, shape, requires_grad, DType.F32)

    def tensor_variable_from_storage(self, tensor, requires_grad: bool = False) -> int:
        data = tensor.data if hasattr(tensor, "meta") else tensor
        return self.tensor_tape.leaf(data.to(self.device), requires_grad)

    def tensor(self, nid: int) -> torch.Tensor:
        """The ``torch.Tensor`` behind a node (storage layer access)."""
        return self.tensor_tape.value(nid)

    def tensor_values(self, nid: int) -> List[float]:
        return self.tensor(nid).detach().to("cpu", torch.float64).reshape(-1).tolist()

    def tensor_values_f32(self, nid: int) -> List[float]:
        return self.tensor(nid).detach().to("cpu", torch.float32).reshape(-1).tolist()

    tensor_values_lossy_f64 = tensor_values

    def tensor_values_meta(self, nid: int) -> Tuple[List[float], TensorMeta]:
        return self.tensor_values(nid), self.tensor_meta(nid)

    def tensor_meta(self, nid: int) -> TensorMeta:
        t = self.tensor(nid)
        return TensorMeta.from_shape_and_strides(t.shape, t.stride(), t.storage_offset(), DType.from_torch(t.dtype),
                                                 self._device_enum)

    def tensor_shape(self, nid: int) -> List[int]:
        return list(self.tensor(nid).shape)

    def tensor_dtype(self, nid: int) -> DType:
        return DType.from_torch(self.tensor(nid).dtype)

    def tensor_numel(self, nid: int) -> int:
        return self.tensor(nid).numel()

    tensor_values_len = tensor_numel

    def tensor_item(self, nid: int) -> float:
        t = self.tensor(nid)
        if t.numel() != 1:
            raise SessionError("tensor_item needs a one-element tensor")
        return float(t.reshape(()).item())

    def tensor_requires_grad(self, nid: int) -> bool:
        return self.tensor_tape.nodes[nid].requires_grad

    def tensor_requires_grad_(self, nid: int, flag: bool = True) -> None:
        self.tensor_tape.requires_grad_(nid, flag)

    def tensor_detach(self, nid: int) -> int:
        return self.tensor_tape.leaf(self.tensor(nid).detach(), False)

    def tensor_version(self, nid: int) -> int:
        return self.tensor_tape.version(nid)


from . import _session_ops as _ops_install  # noqa: E402
from . import _session_factories as _fac_install  # noqa: E402

_ops_install.install(FrankenTorchSession)
_fac_install.install(FrankenTorchSession)

from . import _session_extras as _extra_install  # noqa: E402

_extra_install.install(FrankenTorchSession)

from . import _session_parity as _parity_install  # noqa: E402

_parity_install.install(FrankenTorchSession)
