"""Deterministic Autograd Contract (DAC): the tensor tape.

The tape is append-only; node ids are creation-order indices.  ``backward`` asks the
native scheduler (``libftcore``: reachability DFS, dependency counts, max-heap ready
queue that pops the highest node id first) for the execution plan, then runs each
node's VJP rule in exactly that order on one stream.  Contributions are accumulated
into the input slots in a fixed per-rule order (first contribution is stored
verbatim, later ones are added), so gradients and telemetry replay bit-identically.

Reference behaviour: ft-autograd/src/lib.rs :4268 (TensorTape), :11724-15706
(backward_with_options), :4520-4558 (hooks), :4389 (truncate_graph_to),
:21135-21173 (persistent leaf gradients), :1285-1333 (errors), and the scheduler
golden ft_autograd__tests__tensor_scheduler_telemetry_golden.snap.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field, replace
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..runtime import native
from ..runtime.ledger import ExecutionMode


# ------------------------------------------------------------------------------ errors
class AutogradError(RuntimeError):
    pass


class UnknownTensorNode(AutogradError):
    pass


class TensorRootDoesNotRequireGrad(AutogradError):
    pass


class TensorGraphConsumed(AutogradError):
    pass


class ReentrantDepthExceeded(AutogradError):
    def __init__(self, current: int, maximum: int):
        super().__init__(f"reentrant backward depth {current} exceeds maximum {maximum}")
        self.current, self.max = current, maximum


class TensorDependencyUnderflow(AutogradError):
    pass


class TensorGradientShapeMismatch(AutogradError):
    pass


class TensorRequiresGradNonLeaf(AutogradError):
    pass


class TensorRequiresGradNonFloating(AutogradError):
    pass


class BorrowedInputVersionMismatch(AutogradError):
    def __init__(self, node: int, recorded: int, observed: int):
        super().__init__(f"node {node}: borrowed input mutated in place (version {recorded} -> {observed})")
        self.node, self.recorded, self.observed = node, recorded, observed


class AnomalyDetected(AutogradError):
    pass


# ------------------------------------------------------------------------------ options / reports
class ReentrantPolicy:
    StrictFail = "strict_fail"
    HardenedBoundedFallback = "hardened_bounded_fallback"


@dataclass
class BackwardOptions:
    retain_graph: bool = False
    create_graph: bool = False
    max_reentrant_depth: int = 0
    current_reentrant_depth: int = 0
    policy: str = ReentrantPolicy.StrictFail
    detect_anomaly: bool = False

    # builder spelling of the reference (ft-autograd/src/lib.rs BackwardOptions::with_*): each returns a copy
    def with_retain_graph(self, flag: bool = True) -> "BackwardOptions":
        return replace(self, retain_graph=bool(flag))

    def with_create_graph(self, flag: bool = True) -> "BackwardOptions":
        """``create_graph`` implies that the graph is kept."""
        return replace(self, create_graph=bool(flag), retain_graph=self.retain_graph or bool(flag))

    def with_detect_anomaly(self, flag: bool = True) -> "BackwardOptions":
        return replace(self, detect_anomaly=bool(flag))

    @staticmethod
    def strict_default() -> "BackwardOptions":
        return BackwardOptions(policy=ReentrantPolicy.StrictFail, max_reentrant_depth=0)

    @staticmethod
    def hardened_default() -> "BackwardOptions":
        return BackwardOptions(policy=ReentrantPolicy.HardenedBoundedFallback, max_reentrant_depth=2)

    @staticmethod
    def for_mode(mode: ExecutionMode) -> "BackwardOptions":
        return BackwardOptions.hardened_default() if mode == ExecutionMode.Hardened else BackwardOptions.strict_default()


@dataclass
class TensorBackwardStep:
    node: int
    incoming_grad_len: int
    rule: str


@dataclass
class TensorSchedulerTelemetry:
    execution_order: List[int]
    queue_pushes: int
    queue_pops: int
    max_queue_len: int
    dependency_snapshot: List[int]
    reentrant_depth: int = 0
    reentrant_guard_triggered: bool = False
    hardened_fallback_used: bool = False

    def render(self, mode: str = "strict") -> str:
        """Stable text form (the layout of the reference's golden snapshot)."""
        return "\n".join([
            "dependency_snapshot=" + ",".join(map(str, self.dependency_snapshot)),
            "execution_order=" + ",".join(map(str, self.execution_order)),
            f"hardened_fallback_used={str(self.hardened_fallback_used).lower()}",
            f"max_queue_len={self.max_queue_len}",
            f"mode={mode}",
            f"queue_pops={self.queue_pops}",
            f"queue_pushes={self.queue_pushes}",
            f"reentrant_depth={self.reentrant_depth}",
            f"reentrant_guard_triggered={str(self.reentrant_guard_triggered).lower()}",
        ])


@dataclass
class TensorBackwardReport:
    gradients: Dict[int, torch.Tensor]
    steps: List[TensorBackwardStep]
    telemetry: TensorSchedulerTelemetry
    # create_graph=True only: tape id of the node that holds each gradient (differentiable further)
    gradient_nodes: Dict[int, int] = field(default_factory=dict)
    # leaves whose whole gradient of this backward arrived row-sparse (index_select_sparse)
    sparse_gradients: Dict[int, "RowSparseGradient"] = field(default_factory=dict)

    def gradient(self, node: int) -> Optional[torch.Tensor]:
        g = self.gradients.get(int(node))
        if g is None and int(node) in self.sparse_gradients:
            return self.sparse_gradients[int(node)].to_dense()
        return g

    def sparse_gradient(self, node: int):
        """The row-sparse gradient of ``node`` as a ``SparseCOOTensor`` (None if it was not sparse)."""
        g = self.sparse_gradients.get(int(node))
        return None if g is None else g.to_coo()

    def gradient_node(self, node: int) -> Optional[int]:
        return self.gradient_nodes.get(int(node))

    def is_sparse_gradient(self, node: int) -> bool:
        """Whether the whole gradient of ``node`` arrived row-sparse in this backward."""
        return int(node) in self.sparse_gradients

    def gradient_value(self, node: int) -> Optional["GradientValue"]:
        """The gradient of ``node`` in the form it was produced: dense, or row-sparse for a table read through
        ``index_select_sparse`` (ft-autograd/src/lib.rs:1113 ``GradientValue``)."""
        node = int(node)
        if node in self.sparse_gradients:
            return GradientValue(sparse=self.sparse_gradients[node])
        g = self.gradients.get(node)
        return None if g is None else GradientValue(dense=g)


class GradientValue:
    """A gradient that is either a dense tensor or a row-sparse one."""
    __slots__ = ("_dense", "_sparse")

    def __init__(self, dense: Optional[torch.Tensor] = None, sparse: Optional["RowSparseGradient"] = None):
        if (dense is None) == (sparse is None):
            raise ValueError("exactly one of dense / sparse")
        self._dense, self._sparse = dense, sparse

    def is_sparse(self) -> bool:
        return self._sparse is not None

    def as_dense(self) -> Optional[torch.Tensor]:
        return self._dense

    def as_sparse(self):
        """The COO form of a sparse gradient (``None`` for a dense one)."""
        return None if self._sparse is None else self._sparse.to_coo()

    def to_dense(self, numel: Optional[int] = None) -> torch.Tensor:
        """Dense tensor; with ``numel`` a flat tensor cut or zero-padded to that length."""
        d = self._dense if self._dense is not None else self._sparse.to_dense()
        if numel is None:
            return d
        flat = d.reshape(-1)
        if flat.numel() >= numel:
            return flat[:numel].clone()
        return torch.cat([flat, torch.zeros(numel - flat.numel(), dtype=flat.dtype, device=flat.device)])

    def scaled_clone(self, factor: float) -> "GradientValue":
        """A copy multiplied by ``factor``; a sparse gradient stays sparse."""
        if self._dense is not None:
            return GradientValue(dense=self._dense * factor)
        s = self._sparse
        return GradientValue(sparse=RowSparseGradient(s.rows.clone(), s.values * factor, s.shape))


class RowSparseGradient:
    """Gradient of a 2-D (or higher) table that is zero outside ``rows``: ``values[i]`` is the
    gradient of row ``rows[i]``; rows are unique and ascending, duplicates having been summed in
    source order (so the sum's bits do not depend on how the work was split).  What
    ``index_select_sparse`` hands to ``SparseAdam`` (ft-autograd/src/lib.rs:8204, :15680-15750)."""

    __slots__ = ("rows", "values", "shape")

    def __init__(self, rows: torch.Tensor, values: torch.Tensor, shape):
        self.rows, self.values, self.shape = rows, values, tuple(shape)

    @staticmethod
    def from_indexed(ids: torch.Tensor, g: torch.Tensor, shape) -> "RowSparseGradient":
        """Sum the rows of ``g`` (one per entry of ``ids``) that hit the same table row."""
        flat = ids.reshape(-1).to(torch.int64)
        g2 = g.reshape(flat.numel(), -1)
        rows, inverse = torch.unique(flat, sorted=True, return_inverse=True)
        values = torch.zeros((rows.numel(), g2.shape[1]), dtype=g2.dtype, device=g2.device)
        values.index_add_(0, inverse, g2)            # (CPU index_add_ adds in source order)
        return RowSparseGradient(rows, values.reshape((rows.numel(),) + tuple(shape[1:])), shape)

    def add(self, other: "RowSparseGradient") -> "RowSparseGradient":
        ids = torch.cat([self.rows, other.rows])
        vals = torch.cat([self.values, other.values])
        return RowSparseGradient.from_indexed(ids, vals, self.shape)

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self.shape, dtype=self.values.dtype, device=self.values.device)
        out.index_add_(0, self.rows, self.values)
        return out

    def to_coo(self):
        from ..core.tensor import SparseCOOTensor
        return SparseCOOTensor(self.rows.reshape(1, -1), self.values, self.shape)


# Marker a VJP rule returns for an input whose gradient it already accumulated in place into
# the target handed out by ``GradTargets.leaf_target`` (used by GEMM epilogues that write
# straight into the flat gradient buffer).
ACCUMULATED = object()


class GradTargets:
    """Lets a VJP rule write a leaf gradient in place instead of returning a temporary."""

    __slots__ = ("_tape", "_node", "_grads")

    def __init__(self, tape: "TensorTape", node: "TensorNode", grads: Optional[dict] = None):
        self._tape, self._node, self._grads = tape, node, grads

    def take_current(self, input_index: int) -> Optional[torch.Tensor]:
        """Remove and return the gradient accumulated so far for input ``input_index``.

        A rule that fuses the accumulation into its own kernel (``dx = f(...) + current``)
        takes the running value and returns the sum as that input's contribution; the sum
        is formed in the same position of the pop order, so replay stays bit-identical.
        """
        if self._grads is None:
            return None
        return self._grads.pop(self._node.inputs[input_index], None)

    def leaf_target(self, input_index: int) -> Optional[Tuple[torch.Tensor, bool]]:
        """``(buffer, has_value)`` for a leaf input with a preallocated gradient buffer."""
        nid = self._node.inputs[input_index]
        n = self._tape.nodes[nid]
        if not (n.is_leaf and n.requires_grad) or n.grad_buffer is None or n.hooks:
            return None
        return n.grad_buffer, n.grad_buffer_filled

    def mark_accumulated(self, input_index: int) -> None:
        nid = self._node.inputs[input_index]
        self._tape.nodes[nid].grad_buffer_filled = True
        fn = self._tape.leaf_grad_written_fn
        if fn is not None:
            fn(nid)


class TensorNode:
    __slots__ = ("id", "op", "inputs", "value", "requires_grad", "is_leaf", "vjp", "rule", "retain_grad",
                 "hooks", "grad", "grad_buffer", "grad_buffer_filled", "version", "saved", "name", "cg",
                 "sparse_grad")

    def __init__(self, nid, op, inputs, value, requires_grad, is_leaf, vjp, rule):
        self.id = nid
        self.op = op
        self.inputs = inputs
        self.value = value
        self.requires_grad = requires_grad
        self.is_leaf = is_leaf
        self.vjp = vjp
        self.rule = rule
        self.retain_grad = False
        self.hooks: List[Tuple[int, Callable]] = []
        self.grad: Optional[torch.Tensor] = None         # persistent accumulated gradient
        self.grad_buffer: Optional[torch.Tensor] = None   # preallocated view (flat buffers)
        self.grad_buffer_filled = False
        self.version = 0
        self.saved = None
        self.name = None
        self.cg = None      # graph-building backward: (grad node id) -> per-input contribution node ids
        self.sparse_grad = None   # accumulated row-sparse gradient (leaves fed through index_select_sparse)


@dataclass(frozen=True)
class TensorHookHandle:
    node: int
    hook_id: int


class TensorTape:
    """Append-only tape of tensor operations with a deterministic backward pass."""

    def __init__(self, grad_dtype: Optional[torch.dtype] = torch.float64):
        self._lib = native.load()
        self._h = self._lib.ftc_tape_new()
        self.nodes: List[TensorNode] = []
        self.grad_dtype = grad_dtype      # None: keep the dtype the VJP rule produces
        self._next_hook = 0
        self.grad_enabled = True
        # CPU/f64 sessions keep the reference behaviour (an unreached node sees a zero gradient and
        # its hooks still run); the GPU training path skips such nodes instead of launching fills.
        self.materialize_zero_grads = grad_dtype is not None
        self.accumulate_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor] = lambda a, b: a + b
        # optional profiler hook: a callable returning a context manager, entered around every
        # backward rule (NVTX ranges per tape node, see utils/profiling.py)
        self.range_fn: Optional[Callable[[str], object]] = None
        # optional observer, called with the leaf id each time a rule has written that leaf's
        # gradient in place (the kernel is already on the stream); the data-parallel engine uses it
        # to start a bucket's reduction as soon as its last gradient is in
        self.leaf_grad_written_fn: Optional[Callable[[int], None]] = None
        # optional observer of every recorded (non-leaf) node: called with (node id, operator, output value)
        # right after the node was appended, i.e. after its forward kernels were queued
        self.record_hook: Optional[Callable[[int, str, torch.Tensor], None]] = None
        # optional queue of deferred weight-gradient products (ops/fused.py WgradQueue): flushed when a
        # backward pass ends, so every gradient is on the stream when backward() returns
        self.wgrad_queue = None
        self.last_plan_cache: Dict[Tuple[int, int], Tuple] = {}
        # tape-level anomaly mode (ft-autograd/src/lib.rs:4424-4434): every backward pass checks the gradients it
        # produces for NaN / Inf, whatever the pass's own options say
        self.detect_anomaly = False

    def __del__(self):
        try:
            if self._h:
                self._lib.ftc_tape_free(self._h)
                self._h = None
        except Exception:
            pass

    # ------------------------------------------------------------------ construction
    def __len__(self) -> int:
        return len(self.nodes)

    def _append(self, op, inputs, value, requires_grad, is_leaf, vjp, rule) -> int:
        arr = (C.c_int64 * max(1, len(inputs)))(*inputs)
        nid = self._lib.ftc_tape_add_node(self._h, arr, len(inputs), int(requires_grad), int(is_leaf))
        if nid < 0:
            raise UnknownTensorNode(f"invalid input ids {inputs}")
        self.nodes.append(TensorNode(nid, op, tuple(inputs), value, requires_grad, is_leaf, vjp, rule))
        return int(nid)

    def leaf(self, value: torch.Tensor, requires_grad: bool = False, name: Optional[str] = None) -> int:
        if requires_grad and not value.is_floating_point() and not value.is_complex():
            raise TensorRequiresGradNonFloating(f"dtype {value.dtype} cannot require grad")
        nid = self._append("leaf", (), value, requires_grad, True, None, "leaf")
        self.nodes[nid].name = name
        return nid

    def record(self, op: str, inputs: Sequence[int], value: torch.Tensor,
               vjp: Optional[Callable], rule: str, saved: Any = None, cg: Optional[Callable] = None) -> int:
        """Append a computed node.  ``vjp(grad_out, targets) -> sequence of per-input grads``;
        ``cg(grad_node_id) -> sequence of per-input contribution node ids`` is the graph-building
        form of the same rule, used by ``backward(..., create_graph=True)``."""
        for i in inputs:
            if i < 0 or i >= len(self.nodes):
                raise UnknownTensorNode(f"node {i}")
        rg = self.grad_enabled and any(self.nodes[i].requires_grad for i in inputs) and vjp is not None
        nid = self._append(op, tuple(inputs), value, rg, False, vjp if rg else None, rule)
        self.nodes[nid].saved = saved if rg else None
        self.nodes[nid].cg = cg if rg else None
        if self.record_hook is not None:
            self.record_hook(nid, op, value)
        return nid

    def value(self, nid: int) -> torch.Tensor:
        return self._node(nid).value

    def _node(self, nid: int) -> TensorNode:
        if nid < 0 or nid >= len(self.nodes):
            raise UnknownTensorNode(f"node {nid}")
        return self.nodes[nid]

    def requires_grad_(self, nid: int, flag: bool = True) -> None:
        n = self._node(nid)
        if not n.is_leaf:
            raise TensorRequiresGradNonLeaf(f"node {nid} is not a leaf")
        if flag and not n.value.is_floating_point():
            raise TensorRequiresGradNonFloating(f"node {nid} has dtype {n.value.dtype}")
        n.requires_grad = flag
        self._lib.ftc_tape_set_requires_grad(self._h, nid, int(flag))

    def retain_grad(self, nid: int) -> None:
        n = self._node(nid)
        if not n.requires_grad:
            raise AutogradError("retain_grad() can only be called on tensors with requires_grad=True")
        if not n.is_leaf:          # a leaf keeps its gradient anyway
            n.retain_grad = True

    # ------------------------------------------------------------------ introspection (ft-autograd/src/lib.rs:4424-4520)
    def is_detect_anomaly(self) -> bool:
        return self.detect_anomaly

    def set_detect_anomaly(self, enabled: bool) -> None:
        self.detect_anomaly = bool(enabled)

    def set_grad_enabled(self, enabled: bool) -> bool:
        """Switch recording on or off; returns the previous setting."""
        prev, self.grad_enabled = self.grad_enabled, bool(enabled)
        return prev

    def node_count(self) -> int:
        return len(self.nodes)

    def tensor_is_leaf(self, nid: int) -> bool:
        return self._node(nid).is_leaf

    def tensor_retains_grad(self, nid: int) -> bool:
        n = self._node(nid)
        return bool(n.retain_grad) and not n.is_leaf

    def tensor_has_hooks(self, nid: int) -> bool:
        return bool(self._node(nid).hooks)

    def tensor_grad_fn(self, nid: int) -> Optional[str]:
        """Name of the backward function of a computed node that requires grad (``"MulBackward"``); ``None`` for
        leaves and for nodes outside the graph."""
        n = self._node(nid)
        if n.is_leaf or not n.requires_grad:
            return None
        return "".join(p.capitalize() for p in str(n.op).split("_")) + "Backward"

    def detach_in_place(self, nid: int) -> None:
        """Cut a node out of the graph: it becomes a leaf that does not require grad (its value is kept, its rule
        and inputs are dropped), so nothing upstream of it receives a gradient through it."""
        n = self._node(nid)
        n.is_leaf, n.requires_grad, n.vjp, n.inputs, n.retain_grad = True, False, None, [], False
        self._lib.ftc_tape_set_requires_grad(self._h, nid, 0)
        self.last_plan_cache.clear()

    def bump_version(self, nid: int) -> int:
        n = self._node(nid)
        n.version += 1
        return n.version

    def version(self, nid: int) -> int:
        return self._node(nid).version

    def truncate_graph_to(self, boundary: int) -> None:
        """Drop nodes with id >= boundary (parameters are low-index leaves and survive)."""
        boundary = max(0, min(boundary, len(self.nodes)))
        del self.nodes[boundary:]
        self._lib.ftc_tape_truncate(self._h, boundary)
        self.last_plan_cache.clear()

    def clear_graph(self) -> None:
        self.truncate_graph_to(0)

    def release_values(self, lo: int, hi: int) -> int:
        """Drop the values, rules and saved tensors of the computed (non-leaf, non-retained) nodes with
        ``lo <= id < hi`` whose backward has run, keeping the nodes themselves: ids stay valid for
        bookkeeping, but the nodes can no longer be read or differentiated through.  Frees the
        activations of one micro-batch while other graphs on the same tape are still needed.
        Returns the number of nodes released."""
        n = 0
        for node in self.nodes[max(0, lo): max(0, min(hi, len(self.nodes)))]:
            if node.is_leaf or node.retain_grad or node.value is None:
                continue
            node.value = None
            node.vjp = None
            node.saved = None
            n += 1
        return n

    # ------------------------------------------------------------------ hooks
    def register_tensor_hook(self, nid: int, fn: Callable[[torch.Tensor], Optional[torch.Tensor]]) -> TensorHookHandle:
        n = self._node(nid)
        hid = self._next_hook
        self._next_hook += 1
        n.hooks.append((hid, fn))
        return TensorHookHandle(nid, hid)

    def remove_tensor_hook(self, handle: TensorHookHandle) -> bool:
        n = self._node(handle.node)
        before = len(n.hooks)
        n.hooks = [(h, f) for (h, f) in n.hooks if h != handle.hook_id]
        return len(n.hooks) != before

    # ------------------------------------------------------------------ gradient accessors
    def accumulated_gradient(self, nid: int) -> Optional[torch.Tensor]:
        n = self._node(nid)
        if n.grad_buffer is not None:
            return n.grad_buffer if n.grad_buffer_filled else None
        if n.sparse_grad is not None:
            dense = n.sparse_grad.to_dense()
            return dense if n.grad is None else n.grad + dense
        return n.grad

    def accumulated_sparse_gradient(self, nid: int) -> Optional["RowSparseGradient"]:
        """The accumulated gradient in row-sparse form, when all of it arrived that way."""
        n = self._node(nid)
        return n.sparse_grad if n.grad is None else None

    def set_accumulated_gradient(self, nid: int, grad: Optional[torch.Tensor]) -> None:
        n = self._node(nid)
        if n.grad_buffer is not None and grad is not None:
            n.grad_buffer.copy_(grad)
            n.grad_buffer_filled = True
        else:
            n.grad = grad

    def zero_accumulated_gradient(self, nid: int) -> None:
        n = self._node(nid)
        n.grad = None
        n.sparse_grad = None
        n.grad_buffer_filled = False

    def bind_grad_buffer(self, nid: int, buf: torch.Tensor) -> None:
        """Make ``buf`` (e.g. a view of a flat fp32 gradient arena) the leaf's gradient storage."""
        n = self._node(nid)
        if not n.is_leaf:
            raise TensorRequiresGradNonLeaf(f"node {nid} is not a leaf")
        n.grad_buffer = buf
        n.grad_buffer_filled = False

    # ------------------------------------------------------------------ value-level entry points
    # The reference's tape is also usable without a session: leaves are made from dense tensors or value
    # lists, parameters are updated in place by an optimizer, and the persistent gradient is read, set and
    # cleared by node id (ft-autograd/src/lib.rs:4490 ``set_tensor_requires_grad``, :4512
    # ``detach_tensor_in_place``, :4570 ``leaf_tensor``, :4614-4651 the accumulated-gradient accessors, :4653
    # ``leaf_f32``, :4798-4811 ``to_f16 / to_bf16 / to_dtype``, :21239-21290 ``update_tensor_values*``).
    def leaf_tensor(self, tensor, requires_grad: bool = False) -> int:
        """Leaf over a :class:`DenseTensor` (its buffer is shared, not copied).  Under ``set_grad_enabled(False)``
        the leaf does not require grad, whatever was asked."""
        data = tensor.data if hasattr(tensor, "data") and not isinstance(tensor, torch.Tensor) else tensor
        return self.leaf(data, requires_grad and self.grad_enabled)

    def leaf_f32(self, values, shape, requires_grad: bool = False) -> int:
        t = torch.as_tensor(values, dtype=torch.float32)
        if t.numel() != int(torch.Size(shape).numel()):
            raise AutogradError(f"leaf_f32: {t.numel()} values do not fill shape {tuple(shape)}")
        return self.leaf(t.reshape(tuple(shape)).clone(), requires_grad and self.grad_enabled)

    def leaf_f64(self, values, shape, requires_grad: bool = False) -> int:
        t = torch.as_tensor(values, dtype=torch.float64)
        if t.numel() != int(torch.Size(shape).numel()):
            raise AutogradError(f"leaf_f64: {t.numel()} values do not fill shape {tuple(shape)}")
        return self.leaf(t.reshape(tuple(shape)).clone(), requires_grad and self.grad_enabled)

    def values(self, nid: int) -> list:
        return self._node(nid).value.detach().reshape(-1).to("cpu", torch.float64).tolist()

    def values_f32(self, nid: int) -> torch.Tensor:
        v = self._node(nid).value
        if v.dtype != torch.float32:
            raise AutogradError(f"node {nid} holds {v.dtype}, not float32")
        return v.detach().reshape(-1)

    def set_tensor_requires_grad(self, nid: int, requires_grad: bool) -> None:
        self.requires_grad_(nid, requires_grad)

    def detach_tensor_in_place(self, nid: int) -> None:
        self.detach_in_place(nid)
        self.zero_accumulated_gradient(nid)

    def tensor_accumulated_gradient(self, nid: int) -> Optional[torch.Tensor]:
        return self.accumulated_gradient(nid)

    def tensor_accumulated_gradient_values(self, nid: int) -> Optional[list]:
        g = self.accumulated_gradient(nid)
        return None if g is None else g.detach().reshape(-1).to("cpu", torch.float64).tolist()

    def tensor_accumulated_gradient_len(self, nid: int) -> Optional[int]:
        g = self.accumulated_gradient(nid)
        return None if g is None else g.numel()

    def set_tensor_accumulated_gradient(self, nid: int, gradient) -> None:
        """Replace the persistent gradient; the length must be the node's element count."""
        v = self._node(nid).value
        g = torch.as_tensor(gradient, dtype=self.grad_dtype or v.dtype, device=v.device)
        if g.numel() != v.numel():
            raise TensorGradientShapeMismatch(f"node {nid}: gradient has {g.numel()} elements, the tensor {v.numel()}")
        self.set_accumulated_gradient(nid, g.reshape(v.shape))

    def zero_tensor_accumulated_gradient(self, nid: int) -> None:
        """Fill the persistent gradient with zeros, keeping it allocated (a node without one stays without)."""
        n = self._node(nid)
        if n.grad_buffer is not None:
            n.grad_buffer.zero_()
        elif n.grad is not None or n.sparse_grad is not None:
            shape = n.value.shape
            n.grad = torch.zeros(shape, dtype=(n.grad.dtype if n.grad is not None else self.grad_dtype or n.value.dtype),
                                 device=n.value.device)
            n.sparse_grad = None

    def update_tensor_values(self, nid: int, new_values) -> None:
        """Overwrite a node's values in place; the version counter moves, so a backward that saved the old
        contents by reference refuses to run."""
        n = self._node(nid)
        src = torch.as_tensor(new_values, dtype=n.value.dtype, device=n.value.device)
        if src.numel() != n.value.numel():
            raise AutogradError(f"node {nid}: update has {src.numel()} values, the tensor {n.value.numel()}")
        with torch.no_grad():
            n.value.copy_(src.reshape(n.value.shape))
        n.version += 1

    def update_tensor_values_f32(self, nid: int, new_values) -> None:
        if self._node(nid).value.dtype != torch.float32:
            raise AutogradError(f"node {nid} holds {self._node(nid).value.dtype}, not float32")
        self.update_tensor_values(nid, new_values)

    def update_tensor_values_with(self, nid: int, update: Callable[[torch.Tensor], None]) -> None:
        """``update(values)`` mutates the node's buffer in place (one version bump)."""
        n = self._node(nid)
        with torch.no_grad():
            update(n.value)
        n.version += 1

    def update_tensor_values_with_accumulated_gradient(self, nid: int,
                                                       update: Callable[[torch.Tensor, torch.Tensor], None]) -> bool:
        """``update(gradient, values)`` for an optimizer step without copying either; False (and no call) when
        the node has no persistent gradient."""
        n = self._node(nid)
        g = self.accumulated_gradient(nid)
        if g is None:
            return False
        with torch.no_grad():
            update(g, n.value)
        n.version += 1
        return True

    def to_dtype(self, nid: int, dtype) -> int:
        """Differentiable cast between floating dtypes; the gradient is cast back to the input's dtype.  The
        input is returned as it is when it already has the dtype; integer, bool, complex and quantized targets
        are refused."""
        tdt = dtype if isinstance(dtype, torch.dtype) else dtype.to_torch()
        if tdt not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            raise AutogradError(f"to_dtype: unsupported target {tdt}")
        v = self._node(nid).value
        if not v.is_floating_point():
            raise AutogradError(f"to_dtype: node {nid} holds {v.dtype}, not a floating dtype")
        if v.dtype == tdt:
            return nid
        src = v.dtype
        return self.record("to_dtype", [nid], v.to(tdt), lambda g, targets: [g.to(src) if self.grad_dtype is None else g],
                           "cast: gradient passes through in the input dtype")

    def to_f16(self, nid: int) -> int:
        return self.to_dtype(nid, torch.float16)

    def to_bf16(self, nid: int) -> int:
        return self.to_dtype(nid, torch.bfloat16)

    # ------------------------------------------------------------------ backward
    def schedule(self, root: int, check_consumed: bool = True):
        n = len(self.nodes)
        order = (C.c_int64 * max(1, n))()
        deps = (C.c_int64 * max(1, n))()
        stats = (C.c_int64 * 3)()
        cnt = self._lib.ftc_tape_schedule(self._h, root, int(check_consumed), order, deps, stats)
        if cnt == -1:
            raise UnknownTensorNode(f"node {root}")
        if cnt == -2:
            raise TensorRootDoesNotRequireGrad(f"node {root} does not require grad")
        if cnt == -3:
            raise TensorGraphConsumed("the graph was consumed by an earlier backward; pass retain_graph=True")
        if cnt < 0:
            raise TensorDependencyUnderflow(f"scheduler error {cnt}")
        return list(order[:cnt]), list(deps[:n]), (int(stats[0]), int(stats[1]), int(stats[2]))

    def _cast_grad(self, g: torch.Tensor) -> torch.Tensor:
        if self.grad_dtype is not None and g.dtype != self.grad_dtype and g.is_floating_point():
            return g.to(self.grad_dtype)
        return g

    def backward(self, root: int, options: Optional[BackwardOptions] = None,
                 seed: Optional[torch.Tensor] = None) -> TensorBackwardReport:
        opts = options or BackwardOptions()
        guard = fallback = False
        if opts.current_reentrant_depth > opts.max_reentrant_depth:
            if opts.policy == ReentrantPolicy.StrictFail:
                raise ReentrantDepthExceeded(opts.current_reentrant_depth, opts.max_reentrant_depth)
            guard = fallback = True
        depth = min(opts.current_reentrant_depth, opts.max_reentrant_depth)
        order, deps, (pushes, pops, max_len) = self.schedule(root)
        if opts.create_graph:
            return self._backward_create_graph(root, opts, seed, order, deps, (pushes, pops, max_len), depth, guard,
                                               fallback)

        rootn = self.nodes[root]
        if seed is None:
            seed = torch.ones_like(rootn.value, dtype=self.grad_dtype or rootn.value.dtype)
            seed._ft_unit_seed = True   # lets fused loss rules skip a multiply by one
        grads: Dict[int, torch.Tensor] = {root: seed}
        sparse: Dict[int, RowSparseGradient] = {}
        steps: List[TensorBackwardStep] = []
        nodes = self.nodes
        for nid in order:
            node = nodes[nid]
            incoming = grads.get(nid)
            if incoming is None and nid in sparse:
                steps.append(TensorBackwardStep(nid, int(node.value.numel()), "leaf"))
                continue
            if incoming is None:
                # No gradient reached this node: either it does not require grad, or every rule
                # that feeds it accumulated in place (bound gradient buffers).  A zero gradient
                # contributes nothing downstream, so the node is skipped (it still counts in the
                # execution order, which is a property of the graph alone).
                if node.is_leaf and node.requires_grad and not node.hooks and node.grad_buffer is not None:
                    steps.append(TensorBackwardStep(nid, node.value.numel(), "leaf"))
                    continue
                if not node.requires_grad or not self.materialize_zero_grads:
                    continue
                incoming = torch.zeros_like(node.value, dtype=self.grad_dtype or node.value.dtype)
            for _, hook in node.hooks:
                res = hook(incoming)
                if res is not None:
                    if tuple(res.shape) != tuple(incoming.shape):
                        raise TensorGradientShapeMismatch(
                            f"hook on node {nid} changed the gradient shape {tuple(incoming.shape)} -> {tuple(res.shape)}")
                    incoming = res
            grads[nid] = incoming
            if node.is_leaf:
                if node.requires_grad:
                    steps.append(TensorBackwardStep(nid, incoming.numel(), "leaf"))
                continue
            if not node.requires_grad or node.vjp is None:
                continue
            steps.append(TensorBackwardStep(nid, incoming.numel(), node.rule))
            if self.range_fn is not None:
                with self.range_fn("bwd:%s#%d" % (node.rule, nid)):
                    contribs = node.vjp(incoming, GradTargets(self, node, grads))
            else:
                contribs = node.vjp(incoming, GradTargets(self, node, grads))
            if len(contribs) != len(node.inputs):
                raise TensorGradientShapeMismatch(
                    f"rule '{node.rule}' returned {len(contribs)} gradients for {len(node.inputs)} inputs")
            for inp, g in zip(node.inputs, contribs):
                if g is None or g is ACCUMULATED:
                    continue
                if not nodes[inp].requires_grad:
                    continue
                if isinstance(g, RowSparseGradient):
                    tgt = nodes[inp]
                    if tgt.is_leaf and not tgt.hooks and tgt.grad_buffer is None and inp not in grads:
                        prev_s = sparse.get(inp)
                        sparse[inp] = g if prev_s is None else prev_s.add(g)
                        continue
                    g = g.to_dense()          # a consumer that needs the dense form (hooks, non-leaf, mixed)
                if inp in sparse:             # a dense contribution joins an earlier sparse one: go dense
                    g = self.accumulate_fn(sparse.pop(inp).to_dense(), self._cast_grad(g))
                g = self._cast_grad(g)
                prev = grads.get(inp)
                if prev is None:
                    grads[inp] = g                      # first contribution: stored verbatim
                else:
                    grads[inp] = self.accumulate_fn(prev, g)   # later contributions: added in rule order
            if opts.detect_anomaly or self.detect_anomaly:
                for inp in node.inputs:
                    t = grads.get(inp)
                    if t is not None and not bool(torch.isfinite(t).all()):
                        raise AnomalyDetected(f"non-finite gradient produced by node {nid} ({node.rule})")

        if self.wgrad_queue is not None:
            self.wgrad_queue.flush()        # weight gradients that rules handed to the queue are launched now

        # persistent gradients: leaves that require grad and nodes marked retain_grad
        for nid in order:
            node = nodes[nid]
            if not node.requires_grad:
                continue
            if not (node.is_leaf or node.retain_grad):
                continue
            g = grads.get(nid)
            if g is None:
                continue
            if node.grad_buffer is not None:
                if node.grad_buffer_filled:
                    node.grad_buffer.add_(g)
                else:
                    node.grad_buffer.copy_(g)
                    node.grad_buffer_filled = True
            elif node.grad is None:
                node.grad = g.clone() if g is seed else g
                if node.sparse_grad is not None:          # earlier sparse history folds into the dense slot
                    node.grad = node.grad + node.sparse_grad.to_dense()
                    node.sparse_grad = None
            else:
                node.grad = node.grad + g

        for nid, sg in sparse.items():
            node = nodes[nid]
            sg = RowSparseGradient(sg.rows, self._cast_grad(sg.values), sg.shape)
            sparse[nid] = sg
            if node.grad is not None:                     # mixed history: keep accumulating densely
                node.grad = node.grad + sg.to_dense()
            else:
                node.sparse_grad = sg if node.sparse_grad is None else node.sparse_grad.add(sg)
        if not (opts.retain_graph or opts.create_graph):
            self._lib.ftc_tape_mark_consumed(self._h)
        telemetry = TensorSchedulerTelemetry(order, pushes, pops, max_len, deps, depth, guard, fallback)
        return TensorBackwardReport(grads, steps, telemetry, sparse_gradients=sparse)

    # ------------------------------------------------------------------ graph-building backward
    def _backward_create_graph(self, root, opts, seed, order, deps, stats, depth, guard, fallback):
        """The same scheduler order as ``backward``, but every gradient is a tape node: a rule's
        contributions are appended as nodes (``node.cg``), accumulation is an ``add`` node, and the
        report maps each reached node to the id of its gradient node.  The graph is never consumed
        (``create_graph`` implies ``retain_graph``, ft-autograd/src/lib.rs:15755)."""
        pushes, pops, max_len = stats
        nodes = self.nodes
        rootn = nodes[root]
        if seed is None:
            seed = torch.ones_like(rootn.value, dtype=self.grad_dtype or rootn.value.dtype)
        gnode: Dict[int, int] = {root: self.leaf(seed, requires_grad=False)}
        steps: List[TensorBackwardStep] = []
        for nid in list(order):
            node = nodes[nid]
            gi = gnode.get(nid)
            if gi is None:
                continue
            gval = nodes[gi].value
            for _, hook in node.hooks:
                res = hook(gval)
                if res is not None:
                    if tuple(res.shape) != tuple(gval.shape):
                        raise TensorGradientShapeMismatch(
                            f"hook on node {nid} changed the gradient shape {tuple(gval.shape)} -> {tuple(res.shape)}")
                    gi = self.leaf(res, requires_grad=False)      # a replaced gradient is a constant of the new graph
                    gval = res
                    gnode[nid] = gi
            if node.is_leaf:
                if node.requires_grad:
                    steps.append(TensorBackwardStep(nid, gval.numel(), "leaf"))
                continue
            if not node.requires_grad:
                continue
            if node.cg is None:
                raise AutogradError(f"rule '{node.rule}' (node {nid}) has no graph-building backward; "
                                    "create_graph needs apply_function_with_create_graph for custom functions")
            steps.append(TensorBackwardStep(nid, gval.numel(), node.rule))
            contribs = node.cg(gi)
            if len(contribs) != len(node.inputs):
                raise TensorGradientShapeMismatch(
                    f"rule '{node.rule}' returned {len(contribs)} gradient nodes for {len(node.inputs)} inputs")
            for inp, c in zip(node.inputs, contribs):
                if c is None or not nodes[inp].requires_grad:
                    continue
                prev = gnode.get(inp)
                gnode[inp] = c if prev is None else self._cg_add(prev, c)
        grads = {nid: nodes[g].value for nid, g in gnode.items()}
        for nid in order:
            node = nodes[nid]
            if not node.requires_grad or not (node.is_leaf or node.retain_grad) or nid not in grads:
                continue
            g = self._cast_grad(grads[nid])
            node.grad = g.clone() if node.grad is None else node.grad + g
        telemetry = TensorSchedulerTelemetry(order, pushes, pops, max_len, deps, depth, guard, fallback)
        return TensorBackwardReport(grads, steps, telemetry, dict(gnode))

    def _cg_add(self, a: int, b: int) -> int:
        """Accumulation of two gradient nodes as a node of its own (contributions are added in rule order)."""
        va, vb = self.nodes[a].value, self.nodes[b].value
        return self.record("add", [a, b], self.accumulate_fn(va, vb), lambda g, targets: [g, g],
                           "d(a+b)/da=1; d(a+b)/db=1", cg=lambda g_id: [g_id, g_id])
