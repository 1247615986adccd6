"""Module system (reference: ft-nn/src/lib.rs:316-899).

A ``Module`` registers parameters / buffers / children by name; ``state_dict`` returns dotted
hierarchical keys in sorted order (a ``BTreeMap`` in the reference, :168); ``load_state_dict``
validates every key, shape and dtype before mutating anything (all-or-nothing, :700-731) and
reports ``missing_keys`` / ``unexpected_keys``; ``strict`` turns those into errors.
Free functions: ``named_parameters``, ``named_modules``, ``named_buffers``, ``clip_grad_norm_``
(:740), ``clip_grad_value_``, ``parameters_to_vector`` / ``vector_to_parameters`` (:823-899).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

StateDict = Dict[str, torch.Tensor]


class ModuleError(RuntimeError):
    def __init__(self, reason_code: str, message: str):
        super().__init__(message)
        self.reason_code = reason_code


class ModuleRegistrationError(ModuleError):
    """Refused registration of a parameter, buffer or child (ft-nn/src/lib.rs:133).  ``kind`` is ``InvalidName``
    (with ``what``: parameter / buffer / module), ``NameConflict`` (with ``name``) or ``Unsupported`` (with
    ``module_type`` and ``operation``)."""

    def __init__(self, kind: str, reason_code: str, message: str, **fields):
        super().__init__(reason_code, message)
        self.kind, self.fields = kind, fields


class StateDictError(ModuleError):
    """Failure to build or load a state dict (ft-nn/src/lib.rs:177).  ``kind`` is ``DuplicateStateKey``,
    ``UnsupportedDType``, ``StrictKeyMismatch`` (with ``missing_keys`` / ``unexpected_keys``), ``ShapeMismatch``
    (with ``key``, ``expected``, ``found``) or ``DTypeMismatch``."""

    def __init__(self, kind: str, reason_code: str, message: str, **fields):
        super().__init__(reason_code, message)
        self.kind, self.fields = kind, fields


@dataclass
class LoadStateDictReport:
    missing_keys: List[str] = field(default_factory=list)
    unexpected_keys: List[str] = field(default_factory=list)


def _valid_name(name: str) -> bool:
    return bool(name) and "." not in name


class Module:
    def __init__(self):
        object.__setattr__(self, "_parameters", OrderedDict())     # name -> node id
        object.__setattr__(self, "_buffers", OrderedDict())        # name -> (node id, persistent)
        object.__setattr__(self, "_modules", OrderedDict())
        object.__setattr__(self, "training", True)
        object.__setattr__(self, "_forward_hooks", [])

    # ------------------------------------------------------------------ registration
    def register_parameter(self, name: str, node_id: Optional[int]) -> None:
        if not _valid_name(name):
            raise ModuleRegistrationError("InvalidName", "invalid_parameter_name", f"invalid parameter name {name!r}", what="parameter")
        if name in self._buffers or name in self._modules:
            raise ModuleRegistrationError("NameConflict", "name_collision", f"{name!r} is already registered as a buffer or child", name=name)
        self._parameters[name] = node_id

    def register_buffer(self, name: str, node_id: Optional[int], persistent: bool = True) -> None:
        if not _valid_name(name):
            raise ModuleRegistrationError("InvalidName", "invalid_buffer_name", f"invalid buffer name {name!r}", what="buffer")
        if name in self._parameters or name in self._modules:
            raise ModuleRegistrationError("NameConflict", "name_collision", f"{name!r} is already registered as a parameter or child", name=name)
        self._buffers[name] = (node_id, persistent)

    def add_module(self, name: str, module: Optional["Module"]) -> None:
        if not _valid_name(name):
            raise ModuleRegistrationError("InvalidName", "invalid_module_name", f"invalid child name {name!r}", what="module")
        self._modules[name] = module

    def __setattr__(self, name, value):
        if isinstance(value, Module):
            self._modules[name] = value
        object.__setattr__(self, name, value)

    # ------------------------------------------------------------------ traversal
    def named_children(self) -> List[Tuple[str, "Module"]]:
        return [(n, m) for n, m in self._modules.items() if m is not None]

    def children(self) -> List["Module"]:
        return [m for _, m in self.named_children()]

    def named_modules(self, prefix: str = "") -> List[Tuple[str, "Module"]]:
        out = [(prefix, self)]
        for n, m in self.named_children():
            out += m.named_modules(f"{prefix}.{n}" if prefix else n)
        return out

    def modules(self) -> List["Module"]:
        return [m for _, m in self.named_modules()]

    def named_parameters_own(self) -> List[Tuple[str, int]]:
        return [(n, p) for n, p in self._parameters.items() if p is not None]

    def named_parameters(self, prefix: str = "") -> List[Tuple[str, int]]:
        out = [(f"{prefix}.{n}" if prefix else n, p) for n, p in self.named_parameters_own()]
        for n, m in self.named_children():
            out += m.named_parameters(f"{prefix}.{n}" if prefix else n)
        return out

    def parameters(self) -> List[int]:
        seen, out = set(), []
        for _, p in self.named_parameters():
            if p not in seen:      # shared (tied) parameters appear once
                seen.add(p)
                out.append(p)
        return out

    def named_buffers(self, prefix: str = "", persistent_only: bool = False) -> List[Tuple[str, int]]:
        out = [(f"{prefix}.{n}" if prefix else n, b) for n, (b, pers) in self._buffers.items()
               if b is not None and (pers or not persistent_only)]
        for n, m in self.named_children():
            out += m.named_buffers(f"{prefix}.{n}" if prefix else n, persistent_only)
        return out

    def named_persistent_buffers(self, prefix: str = ""):
        return self.named_buffers(prefix, True)

    def buffers(self) -> List[int]:
        return [b for _, b in self.named_buffers()]

    # ------------------------------------------------------------------ mode
    def train(self, mode: bool = True) -> "Module":
        object.__setattr__(self, "training", bool(mode))
        for m in self.children():
            m.train(mode)
        return self

    def eval(self) -> "Module":
        return self.train(False)

    def is_training(self) -> bool:
        return self.training

    # ------------------------------------------------------------------ call
    def forward(self, session, *args, **kw):
        raise NotImplementedError

    def register_forward_hook(self, fn: Callable) -> int:
        self._forward_hooks.append(fn)
        return len(self._forward_hooks) - 1

    def __call__(self, session, *args, **kw):
        out = self.forward(session, *args, **kw)
        for h in self._forward_hooks:
            r = h(self, args, out)
            if r is not None:
                out = r
        return out

    # ------------------------------------------------------------------ state dict
    def state_dict(self, session, prefix: str = "") -> StateDict:
        sd = {}
        for name, nid in self.named_parameters(prefix) + self.named_buffers(prefix, persistent_only=True):
            if name in sd:
                raise StateDictError("DuplicateStateKey", "state_dict_duplicate_key", f"duplicate state key '{name}'", key=name)
            sd[name] = session.tensor(nid).detach().clone()
        return dict(sorted(sd.items()))

    def load_state_dict(self, session, state: StateDict, strict: bool = True) -> LoadStateDictReport:
        targets = dict(self.named_parameters() + self.named_buffers(persistent_only=True))
        report = LoadStateDictReport(sorted(k for k in targets if k not in state),
                                     sorted(k for k in state if k not in targets))
        if strict and (report.missing_keys or report.unexpected_keys):
            raise StateDictError("StrictKeyMismatch", "state_dict_key_mismatch",
                                 f"missing keys {report.missing_keys}, unexpected keys {report.unexpected_keys}",
                                 missing_keys=report.missing_keys, unexpected_keys=report.unexpected_keys)
        # validate everything before touching anything
        for k, src in state.items():
            if k not in targets:
                continue
            dst = session.tensor(targets[k])
            if tuple(dst.shape) != tuple(src.shape):
                raise StateDictError("ShapeMismatch", "state_dict_shape_mismatch",
                                     f"shape mismatch for {k}: expected {tuple(dst.shape)}, got {tuple(src.shape)}",
                                     key=k, expected=tuple(dst.shape), found=tuple(src.shape))
            if strict and dst.dtype != src.dtype and dst.is_floating_point() != src.is_floating_point():
                raise StateDictError("DTypeMismatch", "state_dict_dtype_mismatch", f"dtype mismatch for {k}: {dst.dtype} vs {src.dtype}", key=k)
        with session.no_grad():
            for k, src in state.items():
                if k in targets:
                    session.tensor(targets[k]).copy_(src.to(session.tensor(targets[k]).dtype))
                    session.tensor_tape.bump_version(targets[k])
        return report

    def zero_grad(self, session) -> None:
        session.tensor_zero_grads(self.parameters())


# -------------------------------------------------------------------------------------- containers
class Sequential(Module):
    def __init__(self, *layers: Module):
        super().__init__()
        for i, l in enumerate(layers):
            self.add_module(str(i), l)

    def forward(self, session, x):
        for m in self.children():
            x = m(session, x)
        return x

    def __len__(self):
        return len(self._modules)

    def __getitem__(self, i):
        return list(self._modules.values())[i]


class ModuleList(Module):
    def __init__(self, modules: Sequence[Module] = ()):
        super().__init__()
        for m in modules:
            self.append(m)

    def append(self, m: Module) -> None:
        self.add_module(str(len(self._modules)), m)

    def __iter__(self) -> Iterator[Module]:
        return iter(self._modules.values())

    def __len__(self):
        return len(self._modules)

    def __getitem__(self, i):
        return list(self._modules.values())[i]


class ModuleDict(Module):
    def __init__(self, modules: Optional[Dict[str, Module]] = None):
        super().__init__()
        for k, m in (modules or {}).items():
            self.add_module(k, m)

    def __getitem__(self, k):
        return self._modules[k]

    def __setitem__(self, k, m):
        self.add_module(k, m)

    def keys(self):
        return self._modules.keys()

    def items(self):
        return self._modules.items()


class ParameterList(Module):
    def __init__(self, params: Sequence[int] = ()):
        super().__init__()
        for p in params:
            self.append(p)

    def append(self, p: int) -> None:
        self.register_parameter(str(len(self._parameters)), p)

    def __iter__(self):
        return iter(self._parameters.values())

    def __len__(self):
        return len(self._parameters)


class ParameterDict(Module):
    def __init__(self, params: Optional[Dict[str, int]] = None):
        super().__init__()
        for k, p in (params or {}).items():
            self.register_parameter(k, p)

    def __getitem__(self, k):
        return self._parameters[k]


# -------------------------------------------------------------------------------------- free functions
def named_parameters(module: Module, prefix: str = ""):
    return module.named_parameters(prefix)


def named_modules(module: Module, prefix: str = ""):
    return module.named_modules(prefix)


def named_buffers(module: Module, prefix: str = ""):
    return module.named_buffers(prefix)


def module_state_dict(session, module: Module) -> StateDict:
    return module.state_dict(session)


def module_load_state_dict(session, module: Module, state: StateDict, strict: bool = True):
    return module.load_state_dict(session, state, strict)


def clip_grad_norm_(session, params: Sequence[int], max_norm: float, norm_type: float = 2.0) -> float:
    """Scale the accumulated gradients so their global norm is at most ``max_norm``; returns the norm."""
    grads = [session.tensor_tape.accumulated_gradient(p) for p in params]
    grads = [g for g in grads if g is not None]
    if not grads:
        return 0.0
    if math.isinf(norm_type):
        total = max(float(g.abs().max()) for g in grads)
    else:
        total = float(sum(float((g.double().abs() ** norm_type).sum()) for g in grads) ** (1.0 / norm_type))
    coef = max_norm / (total + 1e-6)
    if coef < 1.0:
        for g in grads:
            g.mul_(coef)
    return total


def clip_grad_value_(session, params: Sequence[int], clip_value: float) -> None:
    for p in params:
        g = session.tensor_tape.accumulated_gradient(p)
        if g is not None:
            g.clamp_(-clip_value, clip_value)


def parameters_to_vector(session, params: Sequence[int]) -> torch.Tensor:
    return torch.cat([session.tensor(p).detach().reshape(-1) for p in params])


def vector_to_parameters(session, vec: torch.Tensor, params: Sequence[int]) -> None:
    total = sum(session.tensor_numel(p) for p in params)
    if vec.numel() != total:
        raise ModuleError("vector_length_mismatch", f"vector has {vec.numel()} elements, parameters need {total}")
    off = 0
    for p in params:
        n = session.tensor_numel(p)
        session.tensor_update_param_values(p, vec[off: off + n])
        off += n
