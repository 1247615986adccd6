"""Operator surface of ``FrankenTorchSession`` (installed onto the class by ``install``).

The tensor operators are generated from the VJP rule table: ``tensor_<op>(ids..., **params)``
runs the forward, records a dispatch decision in the ledger and appends a tape node whose
backward is the table's rule.  On the CPU device forward and backward are PyTorch CPU operators
(f64).  On the CUDA device the entry point first asks the sm_100a kernel registry
(``dispatch/sm100.py``): a registered operator with qualifying operands runs the hand-written
kernels of ``ops/fused.py``; an operator without a kernel is an error in strict mode and a
ledger-recorded PyTorch fallback in hardened mode.
"""
from __future__ import annotations

import math
from typing import Any, Callable, List, Optional, Sequence, Tuple

import torch

from .autograd.functions import OPS, OpDef
from .autograd.tape import (AutogradError, BackwardOptions, BorrowedInputVersionMismatch, TensorBackwardReport,
                            TensorHookHandle)
from .core.dtype import DType
from .runtime.ledger import EvidenceKind

_INDEX_INPUT_OPS = {"index_select": (1,), "gather": (1,), "scatter": (1,), "scatter_add": (1,), "masked_fill": (1,),
                    "where": (0,), "embedding": (1,), "index_select_sparse": (1,), "cross_entropy": (1,), "nll_loss": (1,), "multi_margin_loss": (1,),
                    "multilabel_margin_loss": (1,), "max_unpool1d": (1,), "max_unpool2d": (1,), "max_unpool3d": (1,),
                    "embedding_bag": (1, 2), "index_put": (1,), "masked_select": (1,), "ctc_loss": (1, 2, 3)}
_MATMUL_CLASS = {"matmul", "bmm", "linear", "addmm", "mv", "baddbmm", "addbmm", "conv1d", "conv2d", "conv3d", "sdpa"}


def _apply(self, name: str, inputs: Sequence[int], **kw) -> int:
    """Run operator ``name`` on tape nodes ``inputs``; returns the id of the result node."""
    op: OpDef = OPS[name]
    tape = self.tensor_tape
    vals = [tape.value(i) for i in inputs]
    idx_pos = _INDEX_INPUT_OPS.get(name, ())
    for p in idx_pos:   # float-valued index tensors are accepted (reference convention)
        if p < len(vals) and vals[p].is_floating_point() and name not in ("where", "masked_fill", "masked_select"):
            vals[p] = vals[p].long()
    cast_back = None
    if self._autocast is not None and name in _MATMUL_CLASS:
        cast_back = vals[0].dtype
        vals = [v.to(self._autocast.to_torch()) if v.is_floating_point() else v for v in vals]
    rg = tape.grad_enabled and any(tape.nodes[i].requires_grad for i in inputs)
    if self.is_cuda:
        from .dispatch import sm100
        route = sm100.ROUTES.get(name)
        if route is not None and self._autocast is None:
            res = route(self, list(inputs), vals, kw)
            if res is not None:
                self._record_dispatch(name, rg, launched=res[1])
                return res[0]
        if name in sm100.LAYOUT_OPS:
            self._record_dispatch(name, rg, launched=f"layout::{name}")
        else:
            why = "no route" if route is None else "operands do not qualify (dtype / layout / extents)"
            if self.runtime.mode.value != "hardened" or not sm100.fallback_allowed("hardened"):
                raise sm100.NoKernelForBackend(name, why)
            self._record_dispatch(name, rg, launched=f"torch::{name}", deviation=sm100.DEVIATION_ID)
    else:
        self._record_dispatch(name, rg)
    out = op.fwd(*vals, **kw)
    if cast_back is not None:
        out = out.to(cast_back)
    vjp = None
    if rg and op.vjp is not None:
        gdt = tape.grad_dtype
        saved_vals = vals

        def vjp(g, targets, _op=op, _vals=saved_vals, _out=out, _kw=kw, _gdt=gdt):
            if _gdt is not None:
                ins = [v.to(_gdt) if v.is_floating_point() else v for v in _vals]
                o = _out.to(_gdt) if _out.is_floating_point() else _out
            else:
                ins, o = _vals, _out
            return list(_op.vjp(g, ins, o, _kw))
    cg = None
    if vjp is not None and not self.is_cuda:
        from .autograd.double_backward import op_cg
        cg = op_cg(tape, op, kw, inputs)
    return tape.record(name, list(inputs), out, vjp, op.rule, cg=cg)


_BUILTIN_BINARY = {"max", "min", "atan2", "fmod", "remainder", "pow_tensor", "matmul", "bmm", "dot", "outer", "kron",
                   "inner", "mv", "linalg_solve", "special_xlogy"}


def _params(name: str):
    """Parameters of the forward, or None for builtins that expose no signature."""
    import inspect
    try:
        return list(inspect.signature(OPS[name].fwd).parameters.values())
    except (ValueError, TypeError):
        return None


def _make_op_method(name: str, n_tensor_args: Optional[int]):
    allp = _params(name)
    ps = [] if allp is None else [p for p in allp if p.kind != p.VAR_POSITIONAL]
    extra_names = [p.name for p in (ps if n_tensor_args is None else ps[n_tensor_args:])]

    def method(self, *args, **kw):
        if n_tensor_args is None:      # variadic: the first positional is a list of ids
            ids, rest = list(args[0]), args[1:]
        else:
            ids, rest = [a for a in args[:n_tensor_args] if a is not None], args[n_tensor_args:]
        for pname, v in zip(extra_names, rest):   # positional parameters follow the forward's order
            kw.setdefault(pname, v)
        return _apply(self, name, ids, **kw)
    method.__name__ = "tensor_" + name
    method.__doc__ = f"``{name}`` on tape nodes; backward rule: {OPS[name].rule}"
    return method


def _tensor_arity(name: str) -> Optional[int]:
    import inspect
    ps = _params(name)
    if ps is None:
        return 2 if name in _BUILTIN_BINARY else 1
    if any(p.kind == p.VAR_POSITIONAL for p in ps):
        return None
    # tensor arguments = leading parameters without a default, plus optional tensor slots named w/b/bias/mask
    n = 0
    for p in ps:
        if p.default is inspect.Parameter.empty or p.name in ("w", "b", "bias", "mask"):
            n += 1
        else:
            break
    return n


# ------------------------------------------------------------------------------------ autograd API
def tensor_backward(self, root: int) -> TensorBackwardReport:
    return self.tensor_backward_with_options(root, BackwardOptions.for_mode(self.runtime.mode))


def tensor_backward_with_options(self, root: int, options: BackwardOptions) -> TensorBackwardReport:
    rep = self.tensor_tape.backward(root, options)
    t = rep.telemetry
    self.runtime.ledger.record(
        EvidenceKind.Backward,
        f"tensor backward root={root} steps={len(rep.steps)} queue_pushes={t.queue_pushes} queue_pops={t.queue_pops} "
        f"max_queue_len={t.max_queue_len} reentrant_depth={t.reentrant_depth} "
        f"reentrant_guard_triggered={str(t.reentrant_guard_triggered).lower()} "
        f"hardened_fallback_used={str(t.hardened_fallback_used).lower()}")
    return rep


def tensor_gradient(self, report: TensorBackwardReport, nid: int):
    g = report.gradient(nid)
    return None if g is None else g.detach().to("cpu", torch.float64).reshape(-1).tolist()


def tensor_grad(self, nid: int):
    return self.tensor_accumulated_gradient(nid)


def tensor_accumulated_gradient(self, nid: int):
    g = self.tensor_tape.accumulated_gradient(nid)
    return None if g is None else g.detach().to("cpu", torch.float64).reshape(-1).tolist()


def tensor_accumulated_gradient_tensor(self, nid: int) -> Optional[torch.Tensor]:
    return self.tensor_tape.accumulated_gradient(nid)


def tensor_accumulated_gradient_len(self, nid: int) -> Optional[int]:
    g = self.tensor_tape.accumulated_gradient(nid)
    return None if g is None else g.numel()


def tensor_set_accumulated_gradient(self, nid: int, values) -> None:
    ref = self.tensor(nid)
    gdt = self.tensor_tape.grad_dtype or ref.dtype
    g = values if isinstance(values, torch.Tensor) else torch.tensor(list(values), dtype=torch.float64)
    self.tensor_tape.set_accumulated_gradient(nid, g.reshape(ref.shape).to(device=ref.device, dtype=gdt))


def tensor_zero_grad(self, nid: int) -> None:
    self.tensor_tape.zero_accumulated_gradient(nid)


def tensor_zero_grads(self, ids: Sequence[int]) -> None:
    for i in ids:
        self.tensor_tape.zero_accumulated_gradient(i)


def tensor_retain_grad(self, nid: int) -> None:
    self.tensor_tape.retain_grad(nid)


def tensor_autograd_grad(self, outputs: int, inputs: Sequence[int], retain_graph: bool = True,
                         create_graph: bool = False):
    """Gradients of ``outputs`` w.r.t. ``inputs`` without touching the accumulated ``.grad`` slots.

    Returns tensors; with ``create_graph=True`` returns the tape ids of the gradient nodes instead
    (``None`` for an input the output does not depend on), which can be differentiated again."""
    tape = self.tensor_tape
    n_before = len(tape.nodes)
    saved = {i: (tape.nodes[i].grad, tape.nodes[i].grad_buffer_filled) for i in range(n_before)}
    opts = BackwardOptions.for_mode(self.runtime.mode)
    opts.retain_graph = retain_graph or create_graph
    opts.create_graph = create_graph
    rep = tape.backward(outputs, opts)
    for i, (g, f) in saved.items():
        tape.nodes[i].grad, tape.nodes[i].grad_buffer_filled = g, f
    if create_graph:
        return [rep.gradient_node(i) for i in inputs]
    return [rep.gradient(i) for i in inputs]


def tensor_functional_hessian(self, y, x: int) -> torch.Tensor:
    """Dense Hessian ``d2 y / dx dx`` of a scalar node ``y`` w.r.t. the tensor node ``x`` by double
    backward: one graph-building backward gives the gradient as a tape node, then one ordinary
    backward per gradient element (seeded with a unit vector) gives a row
    (ft-api tests/*_double_backward_parity.rs call it as ``tensor_functional_hessian(out, x)``).
    ``y`` may also be a callable ``fn(session, x_id) -> scalar node id``; it is evaluated once."""
    tape = self.tensor_tape
    if callable(y):
        y = y(self, x)
    if self.tensor(y).numel() != 1:
        raise ValueError("tensor_functional_hessian needs a scalar output")
    (g_id,) = self.tensor_autograd_grad(y, [x], create_graph=True)
    xv = self.tensor(x)
    n = xv.numel()
    H = torch.zeros(n, n, dtype=torch.float64)
    if g_id is None:
        return H
    gdt = tape.grad_dtype or self.tensor(g_id).dtype
    saved = {i: tape.nodes[i].grad for i in range(len(tape.nodes))}
    for j in range(n):
        if not tape.nodes[g_id].requires_grad:
            break                                   # the gradient is constant in x: the Hessian is zero
        seed = torch.zeros(n, dtype=gdt, device=xv.device)
        seed[j] = 1.0
        rep = tape.backward(g_id, BackwardOptions(retain_graph=True), seed=seed.reshape(self.tensor(g_id).shape))
        row = rep.gradient(x)
        if row is not None:
            H[j] = row.reshape(-1).to("cpu", torch.float64)
    for i, g in saved.items():
        tape.nodes[i].grad = g
    return H


def tensor_apply_function_with_create_graph(self, inputs: Sequence[int], forward_fn, backward_fn) -> int:
    """Custom autograd function whose backward is written in session operators, so it can be
    differentiated again (ft-autograd/src/lib.rs:8951, :1520-1533).

    ``forward_fn(ctx, tensors) -> tensor`` as in :func:`tensor_apply_function`;
    ``backward_fn(session, ctx, grad_id, input_ids) -> list of node ids (or None)`` builds the
    input gradients out of ``tensor_*`` calls.  An ordinary backward evaluates it without recording."""
    from .session import FunctionCtx
    tape = self.tensor_tape
    inputs = list(inputs)
    vals = [tape.value(i) for i in inputs]
    ctx = FunctionCtx([tape.nodes[i].requires_grad for i in inputs])
    out = forward_fn(ctx, vals)
    self._record_dispatch("custom_function", any(ctx.needs_input_grad), "custom_function")

    def vjp(g, targets):
        mark = len(tape)
        prev, tape.grad_enabled = tape.grad_enabled, False
        try:
            gid = tape.leaf(g, requires_grad=False)
            ids = backward_fn(self, ctx, gid, inputs)
            res = [None if i is None else tape.value(i) for i in ids]
        finally:
            tape.grad_enabled = prev
        tape.truncate_graph_to(mark)
        return res

    def cg(g_id):
        prev, tape.grad_enabled = tape.grad_enabled, True
        try:
            return list(backward_fn(self, ctx, g_id, inputs))
        finally:
            tape.grad_enabled = prev

    return tape.record("custom_function", inputs, out, vjp, "custom autograd function backward", cg=cg)


def truncate_autograd_graph(self, boundary: int) -> None:
    self.tensor_tape.truncate_graph_to(boundary)


def autograd_graph_len(self) -> int:
    return len(self.tensor_tape)


def register_tensor_hook(self, nid: int, fn) -> TensorHookHandle:
    return self.tensor_tape.register_tensor_hook(nid, fn)


def remove_tensor_hook(self, handle: TensorHookHandle) -> bool:
    return self.tensor_tape.remove_tensor_hook(handle)


def tensor_apply_function(self, inputs: Sequence[int], forward_fn, backward_fn, borrow_inputs: bool = False) -> int:
    """Custom autograd function (ft-autograd/src/lib.rs:8761).

    ``forward_fn(ctx, tensors) -> tensor``; ``backward_fn(ctx, grad_out) -> list of grads or None``.
    With ``borrow_inputs`` the live inputs are re-read in backward and their version counters
    are checked (``BorrowedInputVersionMismatch`` if one was mutated in place).
    """
    from .session import FunctionCtx
    tape = self.tensor_tape
    vals = [tape.value(i) for i in inputs]
    ctx = FunctionCtx([tape.nodes[i].requires_grad for i in inputs])
    out = forward_fn(ctx, vals)
    versions = [tape.version(i) for i in inputs]
    self._record_dispatch("custom_function", any(ctx.needs_input_grad), "custom_function")

    def vjp(g, targets):
        if borrow_inputs:
            for i, rec in zip(inputs, versions):
                if tape.version(i) != rec:
                    raise BorrowedInputVersionMismatch(i, rec, tape.version(i))
        res = backward_fn(ctx, g)
        return list(res)

    return tape.record("custom_function", list(inputs), out, vjp, "custom autograd function backward")


def tensor_apply_complex_bridge(self, inputs: Sequence[int], output: torch.Tensor, backward_fn) -> int:
    """A complex <-> real bridge node (ft-autograd/src/lib.rs:8884): the caller builds the forward output
    itself, so it may be a complex tensor, and ``backward_fn(ctx, grad_out) -> list of grads or None`` maps the
    output's gradient to one gradient per input.

    A complex node carries its gradient as a REAL tensor with a trailing dimension of 2 (real, imaginary:
    the ``view_as_real`` convention, interleaved in memory), a real node as a tensor of its own shape;
    ``backward_fn`` receives and returns gradients in that form.  With no input that needs a gradient (or with
    recording off) the output is a plain leaf.  The node is an ordinary custom-function node for the scheduler.
    """
    from .session import FunctionCtx
    tape = self.tensor_tape
    needs = [tape.nodes[i].requires_grad and tape.grad_enabled for i in inputs]
    if not any(needs):
        return tape.leaf(output, requires_grad=False)
    ctx = FunctionCtx(needs)
    want = [tuple(tape.value(i).shape) + ((2,) if tape.value(i).is_complex() else ()) for i in inputs]
    out_shape = tuple(output.shape) + ((2,) if output.is_complex() else ())
    self._record_dispatch("complex_bridge", True, "custom_function")

    def vjp(g, targets):
        if tuple(g.shape) != out_shape:
            raise AutogradError(f"complex bridge: output gradient has shape {tuple(g.shape)}, expected {out_shape} "
                                "(complex nodes carry [..., 2] real gradients)")
        res = list(backward_fn(ctx, g))
        if len(res) != len(inputs):
            raise AutogradError(f"complex bridge backward returned {len(res)} gradients for {len(inputs)} inputs")
        for k, (r, w) in enumerate(zip(res, want)):
            if r is not None and (r.is_complex() or tuple(r.shape) != w):
                raise AutogradError(f"complex bridge backward: gradient {k} must be real with shape {w}, "
                                    f"got {r.dtype} {tuple(r.shape)}")
        return res

    return tape.record("complex_bridge", list(inputs), output, vjp,
                       "complex bridge: interleaved (re, im) gradient of the output -> per-input gradients")


def checkpoint(self, fn: Callable, inputs: Sequence[int]) -> int:
    """Recompute-on-backward: run ``fn(session, *ids)`` without recording, replay it in backward."""
    tape = self.tensor_tape
    self.no_grad_enter()
    try:
        out_id = fn(self, *inputs)
        out = tape.value(out_id).detach()
    finally:
        self.no_grad_exit()
    tape.truncate_graph_to(out_id) if out_id == len(tape) - 1 and False else None
    vals = [tape.value(i) for i in inputs]

    def vjp(g, targets):
        # rebuild the sub-graph on fresh leaves, run a nested deterministic backward
        mark = len(tape)
        leaves = [tape.leaf(v.detach(), tape.nodes[i].requires_grad) for v, i in zip(vals, inputs)]
        prev, tape.grad_enabled = tape.grad_enabled, True
        try:
            o = fn(self, *leaves)
            opts = BackwardOptions(retain_graph=True)
            rep = tape.backward(o, opts, seed=g.to(tape.grad_dtype or g.dtype))
        finally:
            tape.grad_enabled = prev
        grads = [rep.gradient(l) for l in leaves]
        for l in leaves:
            tape.nodes[l].grad = None
        return grads

    return tape.record("checkpoint", list(inputs), out, vjp, "checkpoint: recompute forward, then backward")


# ------------------------------------------------------------------------------------ in-place / param update
def _inplace(self, nid: int, fn) -> int:
    t = self.tensor(nid)
    node = self.tensor_tape.nodes[nid]
    if node.requires_grad and self.tensor_tape.grad_enabled and node.is_leaf:
        raise RuntimeError("a leaf that requires grad cannot be modified in place while grad mode is on")
    fn(t)
    self.tensor_tape.bump_version(nid)
    return nid


def tensor_add_(self, a: int, b: int) -> int:
    return _inplace(self, a, lambda t: t.add_(self.tensor(b)))


def tensor_sub_(self, a: int, b: int) -> int:
    return _inplace(self, a, lambda t: t.sub_(self.tensor(b)))


def tensor_mul_(self, a: int, b: int) -> int:
    return _inplace(self, a, lambda t: t.mul_(self.tensor(b)))


def tensor_div_(self, a: int, b: int) -> int:
    return _inplace(self, a, lambda t: t.div_(self.tensor(b)))


def tensor_neg_(self, a: int) -> int:
    return _inplace(self, a, lambda t: t.neg_())


def tensor_zero_(self, a: int) -> int:
    return _inplace(self, a, lambda t: t.zero_())


def tensor_fill_(self, a: int, value: float) -> int:
    return _inplace(self, a, lambda t: t.fill_(value))


def tensor_clamp_(self, a: int, lo=None, hi=None) -> int:
    return _inplace(self, a, lambda t: t.clamp_(lo, hi))


def tensor_update_param_values(self, nid: int, values) -> None:
    t = self.tensor(nid)
    new = values if isinstance(values, torch.Tensor) else torch.tensor(list(values), dtype=torch.float64)
    t.copy_(new.reshape(t.shape).to(t.dtype))
    self.tensor_tape.bump_version(nid)


def tensor_update_param_values_f64_with(self, nid: int, fn: Callable[[torch.Tensor], None]) -> None:
    fn(self.tensor(nid))
    self.tensor_tape.bump_version(nid)


def tensor_update_param_values_f64_with_accumulated_gradient(self, nid: int, fn) -> bool:
    g = self.tensor_tape.accumulated_gradient(nid)
    if g is None:
        return False
    fn(g, self.tensor(nid))
    self.tensor_tape.bump_version(nid)
    return True


def install(cls) -> None:
    for name in list(OPS):
        setattr(cls, "tensor_" + name, _make_op_method(name, _tensor_arity(name)))
    for fn in (tensor_backward, tensor_backward_with_options, tensor_gradient, tensor_grad, tensor_accumulated_gradient,
               tensor_accumulated_gradient_tensor, tensor_accumulated_gradient_len, tensor_set_accumulated_gradient,
               tensor_zero_grad, tensor_zero_grads, tensor_retain_grad, tensor_autograd_grad, tensor_functional_hessian,
               truncate_autograd_graph, autograd_graph_len, register_tensor_hook, remove_tensor_hook,
               tensor_apply_function, tensor_apply_function_with_create_graph, tensor_apply_complex_bridge, checkpoint, tensor_add_, tensor_sub_, tensor_mul_, tensor_div_, tensor_neg_,
               tensor_zero_, tensor_fill_, tensor_clamp_, tensor_update_param_values, tensor_update_param_values_f64_with,
               tensor_update_param_values_f64_with_accumulated_gradient):
        setattr(cls, fn.__name__, fn)
    cls._apply = _apply
    cls.zero_grads_tensor = tensor_zero_grads
