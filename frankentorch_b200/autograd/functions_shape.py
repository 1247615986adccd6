"""VJP rules, part 2: reductions, normalisation, scans, shape, join and index operators.

Registers into the same table as :mod:`frankentorch_b200.autograd.functions`; rule strings
follow the reference (ft-autograd/src/lib.rs:11807-15602).
"""
from __future__ import annotations

import math
from typing import List

import torch

from .functions import OPS, OpDef, _reg, local_vjp, unbroadcast


def _expand_to(g, x, dim, keepdim):
    if dim is None:
        return g.expand(x.shape) if g.dim() else g.reshape(()).expand(x.shape)
    if not keepdim:
        g = g.unsqueeze(dim)
    return g.expand(x.shape)


# ---------------------------------------------------------------------------------- reductions
_reg("sum", lambda x: x.sum(), lambda g, i, o, kw: [g.expand(i[0].shape)], "d(sum(x))/dx_i=1")
_reg("mean", lambda x: x.mean(), lambda g, i, o, kw: [(g / i[0].numel()).expand(i[0].shape)], "d(mean(x))/dx_i=1/n")
_reg("sum_dim", lambda x, dim=0, keepdim=False: x.sum(dim, keepdim=keepdim),
     lambda g, i, o, kw: [_expand_to(g, i[0], kw.get("dim", 0), kw.get("keepdim", False))],
     "d(sum_dim(x))/dx=broadcast_grad_along_dim")
_reg("mean_dim", lambda x, dim=0, keepdim=False: x.mean(dim, keepdim=keepdim),
     lambda g, i, o, kw: [_expand_to(g, i[0], kw.get("dim", 0), kw.get("keepdim", False)) / i[0].shape[kw.get("dim", 0)]],
     "d(mean_dim(x))/dx=broadcast_grad_along_dim/reduce_size")


def _prod_dim_vjp(g, i, o, kw):
    x, dim, keep = i[0], kw.get("dim", 0), kw.get("keepdim", False)
    gg = _expand_to(g, x, dim, keep)
    oo = _expand_to(o, x, dim, keep)
    return [gg * oo / x]


_reg("prod_dim", lambda x, dim=0, keepdim=False: x.prod(dim, keepdim=keepdim), _prod_dim_vjp,
     "d(prod_dim(x))/dx_i=prod/x_i")


def _var_dim_vjp(g, i, o, kw):
    x, dim, keep, corr = i[0], kw.get("dim", 0), kw.get("keepdim", False), kw.get("correction", 1)
    n = x.shape[dim]
    mu = x.mean(dim, keepdim=True)
    return [_expand_to(g, x, dim, keep) * 2 * (x - mu) / (n - corr)]


def _std_dim_vjp(g, i, o, kw):
    x, dim, keep, corr = i[0], kw.get("dim", 0), kw.get("keepdim", False), kw.get("correction", 1)
    n = x.shape[dim]
    mu = x.mean(dim, keepdim=True)
    return [_expand_to(g, x, dim, keep) * (x - mu) / ((n - corr) * _expand_to(o, x, dim, keep))]


_reg("var_dim", lambda x, dim=0, keepdim=False, correction=1: x.var(dim, keepdim=keepdim, correction=correction),
     _var_dim_vjp, "d(var_dim(x))/dx_i=2*(x_i-mean)/(n-1)")
_reg("std_dim", lambda x, dim=0, keepdim=False, correction=1: x.std(dim, keepdim=keepdim, correction=correction),
     _std_dim_vjp, "d(std_dim(x))/dx_i=(x_i-mean)/((n-1)*std)")
_reg("trace", torch.trace,
     lambda g, i, o, kw: [g * torch.eye(i[0].shape[0], i[0].shape[1], dtype=g.dtype)], "d(trace(X))/dX=grad_out*I")


def _norm_vjp(g, i, o, kw):
    x, p = i[0], kw.get("p", 2.0)
    if p == 2.0:
        return [g * x / o] if float(o) != 0.0 else [torch.zeros_like(x)]
    if p == 1.0:
        return [g * torch.sign(x)]
    if math.isinf(p):
        m = (x.abs() == o).to(x.dtype)
        return [g * torch.sign(x) * m / m.sum()]
    return [g * x * x.abs().pow(p - 2) / o.pow(p - 1)]


def _norm_dim_vjp(g, i, o, kw):
    x, p, dim, keep = i[0], kw.get("p", 2.0), kw.get("dim", 0), kw.get("keepdim", False)
    gg, oo = _expand_to(g, x, dim, keep), _expand_to(o, x, dim, keep)
    if p == 2.0:
        return [torch.where(oo != 0, gg * x / oo, torch.zeros_like(x))]
    if p == 1.0:
        return [gg * torch.sign(x)]
    return [gg * x * x.abs().pow(p - 2) / oo.pow(p - 1)]


_reg("norm", lambda x, p=2.0: torch.linalg.vector_norm(x, p), _norm_vjp, "d(norm_p(x))/dx=x*|x|^(p-2)/norm^(p-1)")
_reg("norm_dim", lambda x, p=2.0, dim=0, keepdim=False: torch.linalg.vector_norm(x, p, dim=dim, keepdim=keepdim),
     _norm_dim_vjp, "d(norm_dim_p(x))/dx=x*|x|^(p-2)/norm^(p-1) along dim")


def _minmax_dim(which):
    def fwd(x, dim=0, keepdim=False):
        return getattr(x, which)(dim, keepdim=keepdim).values

    def vjp(g, i, o, kw):
        x, dim, keep = i[0], kw.get("dim", 0), kw.get("keepdim", False)
        idx = getattr(x, "arg" + which)(dim, keepdim=True)
        gg = g if keep else g.unsqueeze(dim)
        return [torch.zeros_like(x).scatter_(dim, idx, gg.to(x.dtype))]
    return fwd, vjp


for _w in ("max", "min"):
    _f, _v = _minmax_dim(_w)
    _reg(_w + "_dim", _f, _v, f"d({_w}_dim(x))/dx=scatter_grad_to_arg{_w}")

_reg("logsumexp", lambda x, dim=-1, keepdim=False: torch.logsumexp(x, dim, keepdim=keepdim),
     lambda g, i, o, kw: [_expand_to(g, i[0], kw.get("dim", -1) % i[0].dim(), kw.get("keepdim", False))
                          * torch.exp(i[0] - _expand_to(o, i[0], kw.get("dim", -1) % i[0].dim(), kw.get("keepdim", False)))],
     "d(logsumexp(x))/dx=softmax(x)*grad")

# ---------------------------------------------------------------------------------- normalise / scans
_reg("softmax", lambda x, dim=-1: torch.softmax(x, dim),
     lambda g, i, o, kw: [o * (g - (g * o).sum(kw.get("dim", -1), keepdim=True))],
     "d(softmax(x))/dx_i=s_i*(grad_i-sum(grad*s))")
_reg("log_softmax", lambda x, dim=-1: torch.log_softmax(x, dim),
     lambda g, i, o, kw: [g - torch.exp(o) * g.sum(kw.get("dim", -1), keepdim=True)],
     "d(log_softmax(x))/dx_i=grad_i-softmax_i*sum(grad)")
_reg("cumsum", lambda x, dim=0: torch.cumsum(x, dim),
     lambda g, i, o, kw: [torch.flip(torch.cumsum(torch.flip(g, [kw.get("dim", 0)]), kw.get("dim", 0)), [kw.get("dim", 0)])],
     "d(cumsum(x))/dx=reverse_cumsum(grad)")
OPS["cumprod"] = OpDef("cumprod", lambda x, dim=0: torch.cumprod(x, dim),
                       local_vjp(lambda x, dim=0: torch.cumprod(x, dim)), "d(cumprod(x))/dx=reverse_cumsum(grad*out)/x")

# ---------------------------------------------------------------------------------- shape
_reg("reshape", lambda x, shape=(): x.reshape(tuple(shape)), lambda g, i, o, kw: [g.reshape(i[0].shape)],
     "d(shape_op(x))/dx=identity")
_reg("contiguous", lambda x: x.contiguous(), lambda g, i, o, kw: [g], "d(shape_op(x))/dx=identity")
_reg("view", lambda x, shape=(): x.reshape(tuple(shape)), lambda g, i, o, kw: [g.reshape(i[0].shape)],
     "d(shape_op(x))/dx=identity")
_reg("squeeze", lambda x, dim=None: x.squeeze() if dim is None else x.squeeze(dim),
     lambda g, i, o, kw: [g.reshape(i[0].shape)], "d(shape_op(x))/dx=identity")
_reg("unsqueeze", lambda x, dim=0: x.unsqueeze(dim), lambda g, i, o, kw: [g.reshape(i[0].shape)],
     "d(shape_op(x))/dx=identity")
_reg("flatten", lambda x, start=0, end=-1: x.flatten(start, end), lambda g, i, o, kw: [g.reshape(i[0].shape)],
     "d(shape_op(x))/dx=identity")
_reg("transpose", lambda x, dim0=0, dim1=1: x.transpose(dim0, dim1).contiguous(),
     lambda g, i, o, kw: [g.transpose(kw.get("dim0", 0), kw.get("dim1", 1)).contiguous()],
     "d(transpose(x))/dx=transpose_inverse(grad)")


def _inv_perm(dims):
    inv = [0] * len(dims)
    for k, d in enumerate(dims):
        inv[d] = k
    return inv


_reg("permute", lambda x, dims=(): x.permute(*dims).contiguous(),
     lambda g, i, o, kw: [g.permute(*_inv_perm([d % i[0].dim() for d in kw["dims"]])).contiguous()],
     "d(permute(x))/dx=inverse_permute(grad)")
_reg("expand", lambda x, shape=(): x.expand(*shape).contiguous(),
     lambda g, i, o, kw: [unbroadcast(g, i[0].shape) if g.dim() == i[0].dim()
                          else unbroadcast(g, (1,) * (g.dim() - i[0].dim()) + tuple(i[0].shape)).reshape(i[0].shape)],
     "d(expand(x))/dx=sum_broadcast_dims(grad)")
_reg("sum_to_shape", lambda x, shape=(): unbroadcast(x, shape).reshape(tuple(shape)),
     lambda g, i, o, kw: [g.expand(i[0].shape)], "d(sum_to_shape(x))/dx=broadcast(grad)")


def _narrow_vjp(g, i, o, kw):
    z = torch.zeros_like(i[0], dtype=g.dtype)
    z.narrow(kw.get("dim", 0), kw.get("start", 0), kw.get("length", 1)).copy_(g)
    return [z]


_reg("narrow", lambda x, dim=0, start=0, length=1: x.narrow(dim, start, length).contiguous(), _narrow_vjp,
     "d(narrow(x))/dx=zero_pad_grad")
_reg("flip", lambda x, dims=(0,): torch.flip(x, list(dims)), lambda g, i, o, kw: [torch.flip(g, list(kw.get("dims", (0,))))],
     "d(flip(x))/dx=flip(grad)")
_reg("roll", lambda x, shifts=1, dims=0: torch.roll(x, shifts, dims),
     lambda g, i, o, kw: [torch.roll(g, tuple(-s for s in kw["shifts"]) if isinstance(kw.get("shifts", 1), (tuple, list))
                                     else -kw.get("shifts", 1), kw.get("dims", 0))], "d(roll(x))/dx=roll_back(grad)")


def _repeat_vjp(g, i, o, kw):
    x, reps = i[0], list(kw["repeats"])
    shape = [1] * (len(reps) - x.dim()) + list(x.shape)
    view = []
    for r, s in zip(reps, shape):
        view += [r, s]
    return [g.reshape(view).sum(list(range(0, 2 * len(reps), 2))).reshape(x.shape)]


_reg("repeat", lambda x, repeats=(): x.repeat(*repeats), _repeat_vjp, "d(repeat(x))/dx=sum_repeats(grad)")


def _pad_vjp(g, i, o, kw):
    pad = list(kw["padding"])
    sl = [slice(None)] * g.dim()
    for k in range(len(pad) // 2):
        d = g.dim() - 1 - k
        lo, hi = pad[2 * k], pad[2 * k + 1]
        sl[d] = slice(lo, g.shape[d] - hi)
    return [g[tuple(sl)].contiguous()]


_reg("pad", lambda x, padding=(), value=0.0: torch.nn.functional.pad(x, list(padding), value=value), _pad_vjp,
     "d(pad(x))/dx=unpad(grad)")
_reg("tril", lambda x, k=0: torch.tril(x, k), lambda g, i, o, kw: [torch.tril(g, kw.get("k", 0))], "d(tril(x))/dx=tril(grad)")
_reg("triu", lambda x, k=0: torch.triu(x, k), lambda g, i, o, kw: [torch.triu(g, kw.get("k", 0))], "d(triu(x))/dx=triu(grad)")
for _c, _dt in (("cast_f32", torch.float32), ("cast_f64", torch.float64), ("cast_f16", torch.float16),
                ("cast_bf16", torch.bfloat16)):
    _reg(_c, (lambda dt: (lambda x: x.to(dt)))(_dt), lambda g, i, o, kw: [g], "d(cast)/d_input=grad (identity)")

# ---------------------------------------------------------------------------------- join (variadic)
_reg("cat", lambda *xs, dim=0: torch.cat(xs, dim),
     lambda g, i, o, kw: list(torch.split(g, [x.shape[kw.get("dim", 0)] for x in i], kw.get("dim", 0))),
     "d(cat(x...))/dx_i=split_grad_along_dim")
_reg("stack", lambda *xs, dim=0: torch.stack(xs, dim),
     lambda g, i, o, kw: list(torch.unbind(g, kw.get("dim", 0))), "d(stack(x...))/dx_i=slice_grad_along_dim")

# ---------------------------------------------------------------------------------- index ops
# index tensors are passed as non-differentiable inputs (int64), value tensors as inputs


def _index_select_vjp(g, i, o, kw):
    x, idx = i
    return [torch.zeros_like(x, dtype=g.dtype).index_add_(kw.get("dim", 0), idx, g), None]


_reg("index_select", lambda x, idx, dim=0: torch.index_select(x, dim, idx), _index_select_vjp,
     "d(index_select(x))/dx=scatter_add_grad")
_reg("gather", lambda x, idx, dim=0: torch.gather(x, dim, idx),
     lambda g, i, o, kw: [torch.zeros_like(i[0], dtype=g.dtype).scatter_add_(kw.get("dim", 0), i[1], g), None],
     "d(gather(x))/dx=scatter_add_grad")
_reg("scatter", lambda x, idx, src, dim=0: torch.scatter(x, dim, idx, src),
     lambda g, i, o, kw: [g.scatter(kw.get("dim", 0), i[1], 0.0), None, torch.gather(g, kw.get("dim", 0), i[1])],
     "d(scatter(x,idx,src))/dx=mask_grad; d/dsrc=gather(grad)")
_reg("scatter_add", lambda x, idx, src, dim=0: torch.scatter_add(x, dim, idx, src),
     lambda g, i, o, kw: [g, None, torch.gather(g, kw.get("dim", 0), i[1])],
     "d(scatter_add(x,idx,src))/dx=grad; d/dsrc=gather(grad)")
_reg("masked_fill", lambda x, mask, value=0.0: x.masked_fill(mask.bool(), value),
     lambda g, i, o, kw: [g.masked_fill(i[1].bool(), 0.0), None], "d(masked_fill(x))/dx=grad where not mask")
_reg("where", lambda cond, a, b: torch.where(cond.bool(), a, b),
     lambda g, i, o, kw: [None, unbroadcast(torch.where(i[0].bool(), g, torch.zeros_like(g)), i[1].shape),
                          unbroadcast(torch.where(i[0].bool(), torch.zeros_like(g), g), i[2].shape)],
     "d(where(c,a,b))/da=grad*c; d/db=grad*(1-c)")


def _sort_vjp(g, i, o, kw):
    x, dim = i[0], kw.get("dim", -1)
    idx = torch.sort(x, dim=dim, descending=kw.get("descending", False), stable=True).indices
    return [torch.zeros_like(x, dtype=g.dtype).scatter_(dim, idx, g)]


_reg("sort", lambda x, dim=-1, descending=False: torch.sort(x, dim=dim, descending=descending, stable=True).values,
     _sort_vjp, "d(sort(x))/dx=scatter_grad_to_sorted_positions")


def _topk_vjp(g, i, o, kw):
    x, dim = i[0], kw.get("dim", -1)
    idx = torch.topk(x, kw["k"], dim=dim, largest=kw.get("largest", True), sorted=True).indices
    return [torch.zeros_like(x, dtype=g.dtype).scatter_(dim, idx, g)]


_reg("topk", lambda x, k=1, dim=-1, largest=True: torch.topk(x, k, dim=dim, largest=largest, sorted=True).values,
     _topk_vjp, "d(topk(x))/dx=scatter_grad_to_topk_positions")
def _index_select_sparse_vjp(g, i, o, kw):
    from .tape import RowSparseGradient
    return [RowSparseGradient.from_indexed(i[1], g, i[0].shape), None]


# the same gather as `embedding`; its table gradient is row-sparse (ft-autograd/src/lib.rs:582-587, :8204)
_reg("index_select_sparse", lambda w, ids: w[ids], _index_select_sparse_vjp,
     "d(index_select(x))/dx=scatter_add_grad [row-sparse]")
_reg("embedding", lambda w, ids: w[ids],
     lambda g, i, o, kw: [torch.zeros_like(i[0], dtype=g.dtype).index_add_(0, i[1].reshape(-1), g.reshape(-1, i[0].shape[1])), None],
     "d(index_select(x))/dx=scatter_add_grad")
