"""Session methods whose argument order, return shape or side effect differs from the plain
``tensor_<op>(tensor ids..., **params)`` form that the rule table generates (installed onto
``FrankenTorchSession`` by ``install``).

The reference's per-operator benches and probes call these names with positional arguments
(ft-api/benches/ops_bench.rs, special_bench.rs, distributions in ft-api/examples/*_probe.rs), so each
wrapper takes them in that order: ``tensor_index_add(x, dim, index, src)``, ``tensor_renorm(x, p, dim,
maxnorm)``, ``tensor_lu_solve(lu, pivots, b)`` and so on.  Groups:

* positional wrappers over rules of ``autograd/functions_parity.py``;
* second names of operators that already exist (``tensor_cholesky`` for ``tensor_linalg_cholesky``);
* multi-output forms (``tensor_aminmax``, ``tensor_var_mean``, ``tensor_qr``, ``tensor_histogram``);
* in-place variants (``tensor_hypot_`` ...), which follow the version-counter rules of ``tensor_add_``;
* samplers of the session's xoshiro256++ stream (``tensor_exponential``, ``tensor_gamma`` ...);
* the raw recurrent forwards ``tensor_rnn / tensor_lstm / tensor_gru`` (outputs are leaves without history).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

from ._session_factories import _new, _numel
from .core.dtype import DType
from ._session_ops import _inplace
from .autograd.tape import AutogradError


def _opt(ids):
    return [i for i in ids if i is not None]


# ------------------------------------------------------------------------------------ positional wrappers
def tensor_logit(self, x, eps=None):
    return self._apply("logit", [x], eps=eps)


def tensor_nan_to_num(self, x, nan=0.0, posinf=None, neginf=None):
    return self._apply("nan_to_num", [x], nan=nan, posinf=posinf, neginf=neginf)


def tensor_polygamma(self, n, x):
    return self._apply("polygamma", [x], n=int(n))


def tensor_amax(self, x, dim=None, keepdim=False):
    return self._apply("amax", [x], dim=dim, keepdim=keepdim)


def tensor_amin(self, x, dim=None, keepdim=False):
    return self._apply("amin", [x], dim=dim, keepdim=keepdim)


def tensor_aminmax(self, x, dim=None) -> Tuple[int, int]:
    return tensor_amin(self, x, dim), tensor_amax(self, x, dim)


def tensor_kthvalue(self, x, k, dim=-1, keepdim=False) -> Tuple[int, int]:
    """``(values, indices)`` of the k-th smallest element along ``dim`` (k counts from 1)."""
    v = self._apply("kthvalue", [x], k=int(k), dim=dim, keepdim=keepdim)
    idx = torch.kthvalue(self.tensor(x), int(k), dim, keepdim).indices
    return v, _new(self, idx.to(torch.float64), False)


def tensor_dist(self, a, b, p=2.0):
    return self._apply("dist", [a, b], p=float(p))


def tensor_diff(self, x, dim=-1):
    return self._apply("diff", [x], dim=dim)


def tensor_diff_full(self, x, n=1, dim=-1, prepend=None, append=None):
    if prepend is not None and append is not None:
        return self._apply("diff_full_both", [x, prepend, append], n=n, dim=dim)
    if prepend is not None:
        return self._apply("diff_full_prepend", [x, prepend], n=n, dim=dim)
    if append is not None:
        return self._apply("diff_full_append", [x, append], n=n, dim=dim)
    return self._apply("diff_full", [x], n=n, dim=dim)


def tensor_trapezoid(self, y, x=None, dim=-1, dx=1.0):
    return self._apply("trapezoid", [y], dx=dx, dim=dim) if x is None else self._apply("trapezoid_x", [y, x], dim=dim)


def tensor_cumulative_trapezoid(self, y, x=None, dim=-1, dx=1.0):
    if x is None:
        return self._apply("cumulative_trapezoid", [y], dx=dx, dim=dim)
    return self._apply("cumulative_trapezoid_x", [y, x], dim=dim)


def tensor_gradient_dim(self, x, dim=0, spacing=1.0, edge_order=1):
    return self._apply("gradient_dim", [x], dim=dim, spacing=spacing, edge_order=edge_order)


def tensor_select(self, x, dim, index):
    return self._apply("select", [x], dim=dim, index=index)


def tensor_select_scatter(self, x, src, dim, index):
    return self._apply("select_scatter", [x, src], dim=dim, index=index)


def tensor_slice_scatter(self, x, src, dim=0, start=None, end=None, step=1):
    return self._apply("slice_scatter", [x, src], dim=dim, start=start, end=end, step=step)


def tensor_rot90(self, x, k=1, dims=(0, 1)):
    return self._apply("rot90", [x], k=k, dims=tuple(dims))


def tensor_renorm(self, x, p, dim, maxnorm):
    return self._apply("renorm", [x], p=float(p), dim=dim, maxnorm=float(maxnorm))


def tensor_normalize(self, x, p=2.0, dim=1, eps=1e-12):
    return self._apply("normalize", [x], p=float(p), dim=dim, eps=eps)


def tensor_index_add(self, x, dim, index, src, alpha=1.0):
    return self._apply("index_add", [x, index, src], dim=dim, alpha=alpha)


def tensor_index_copy(self, x, dim, index, src):
    return self._apply("index_copy", [x, index, src], dim=dim)


def tensor_index_fill(self, x, dim, index, value):
    return self._apply("index_fill", [x, index], dim=dim, value=value)


def tensor_index_reduce(self, x, dim, index, src, reduce, include_self=True):
    return self._apply("index_reduce", [x, index, src], dim=dim, reduce=reduce, include_self=include_self)


def tensor_scatter_reduce(self, x, dim, index, src, reduce, include_self=True):
    return self._apply("scatter_reduce", [x, index, src], dim=dim, reduce=reduce, include_self=include_self)


def tensor_take_along_dim(self, x, index, dim):
    return self._apply("take_along_dim", [x, index], dim=dim)


def tensor_put(self, x, index, values, accumulate=False):
    return self._apply("put", [x, index, values], accumulate=accumulate)


def tensor_repeat_interleave(self, x, repeats, dim=None):
    return self._apply("repeat_interleave", [x], repeats=int(repeats), dim=dim)


def tensor_repeat_interleave_tensor(self, x, repeats, dim=None):
    return self._apply("repeat_interleave_tensor", [x], repeats=tuple(int(r) for r in repeats), dim=dim)


def tensor_repeat_interleave_repeats(self, x, repeats, dim=None):
    """``repeats`` is a tensor node: one count per element (or per slice of ``dim``), or a single count for all."""
    reps = [float(v) for v in self.tensor(repeats).detach().reshape(-1).tolist()]
    if any(r < 0 or r != int(r) for r in reps):
        raise ValueError("repeat_interleave: repeats must be non-negative integers")
    n = self.tensor_numel(x) if dim is None else self.tensor_shape(x)[dim]
    if len(reps) == 1:
        reps = reps * n
    if len(reps) != n:
        raise ValueError(f"repeat_interleave: {len(reps)} repeat counts for {n} positions")
    return tensor_repeat_interleave_tensor(self, x, reps, dim)


def tensor_addcmul(self, x, t1, t2, value=1.0):
    return self._apply("addcmul", [x, t1, t2], value=value)


def tensor_addcdiv(self, x, t1, t2, value=1.0):
    return self._apply("addcdiv", [x, t1, t2], value=value)


def tensor_addr(self, x, v1, v2, beta=1.0, alpha=1.0):
    return self._apply("addr", [x, v1, v2], beta=beta, alpha=alpha)


def tensor_where_scalar(self, cond, x, y):
    return self._apply("where_scalar", [cond], x=float(x), y=float(y))


def tensor_isclose(self, a, b, rtol=1e-5, atol=1e-8, equal_nan=False):
    return self._apply("isclose", [a, b], rtol=rtol, atol=atol, equal_nan=equal_nan)


def tensor_float_power(self, x, exponent):
    return self._apply("float_power", [x], exponent=float(exponent))


def tensor_clamp_min(self, x, min):
    return self._apply("clamp_min", [x], min=float(min))


def tensor_clamp_max(self, x, max):
    return self._apply("clamp_max", [x], max=float(max))


def tensor_round_decimals(self, x, decimals):
    return self._apply("round_decimals", [x], decimals=int(decimals))


def tensor_mvlgamma(self, x, p):
    return self._apply("mvlgamma", [x], p=int(p))


def tensor_one_hot(self, index, num_classes=-1):
    return self._apply("one_hot", [index], num_classes=num_classes)


def tensor_vander(self, x, n=None, increasing=False):
    return self._apply("vander", [x], n=n, increasing=increasing)


def tensor_combinations(self, x, r=2, with_replacement=False):
    return self._apply("combinations", [x], r=r, with_replacement=with_replacement)


def tensor_nanvar(self, x, correction=1, dim=None, keepdim=False):
    return self._apply("nanvar", [x], correction=correction, dim=dim, keepdim=keepdim)


def tensor_nanstd(self, x, correction=1, dim=None, keepdim=False):
    return self._apply("nanstd", [x], correction=correction, dim=dim, keepdim=keepdim)


def tensor_var_mean(self, x, dim, correction=1, keepdim=False) -> Tuple[int, int]:
    return (self.tensor_var_dim(x, dim=dim, keepdim=keepdim, correction=correction),
            self.tensor_mean_dim(x, dim=dim, keepdim=keepdim))


def tensor_std_mean(self, x, dim, correction=1, keepdim=False) -> Tuple[int, int]:
    return (self.tensor_std_dim(x, dim=dim, keepdim=keepdim, correction=correction),
            self.tensor_mean_dim(x, dim=dim, keepdim=keepdim))


def _quantile(self, x, q, dim, keepdim, interpolation, ignore_nan=False):
    q = [float(v) for v in q] if isinstance(q, (list, tuple)) else float(q)
    return self._apply("quantile_full", [x], q=q, dim=dim, keepdim=keepdim, interpolation=interpolation, ignore_nan=ignore_nan)


def tensor_quantile_dim(self, x, q, dim, keepdim=False, interpolation="linear"):
    return _quantile(self, x, q, dim, keepdim, interpolation)


def tensor_quantile_multi(self, x, qs, interpolation="linear"):
    return _quantile(self, x, list(qs), None, False, interpolation)


def tensor_quantile_dim_multi(self, x, qs, dim, keepdim=False, interpolation="linear"):
    return _quantile(self, x, list(qs), dim, keepdim, interpolation)


def tensor_nanquantile(self, x, q, dim=None, keepdim=False, interpolation="linear"):
    return _quantile(self, x, q, dim, keepdim, interpolation, ignore_nan=True)


def tensor_cross_entropy_full(self, logits, target, weight=None, ignore_index=None, reduction="mean", label_smoothing=0.0):
    return self._apply("cross_entropy_full", _opt([logits, target, weight]),
                       ignore_index=-100 if ignore_index is None else int(ignore_index), reduction=reduction,
                       label_smoothing=label_smoothing)


def tensor_nll_loss_full(self, lp, target, weight=None, ignore_index=None, reduction="mean"):
    return self._apply("nll_loss_full", _opt([lp, target, weight]),
                       ignore_index=-100 if ignore_index is None else int(ignore_index), reduction=reduction)


def tensor_bce_with_logits_pos_weight(self, x, t, pos_weight, reduction="mean"):
    return self._apply("bce_with_logits_pos_weight", [x, t], pos_weight=float(pos_weight), reduction=reduction)


def tensor_binary_cross_entropy(self, p, t, reduction="mean"):
    return self.tensor_bce_loss(p, t, reduction=reduction)


def tensor_block_diag(self, ids):
    return self._apply("block_diag", list(ids))


def tensor_cartesian_prod(self, ids):
    return self._apply("cartesian_prod", list(ids))


def tensor_column_stack(self, ids):
    return self._apply("column_stack", list(ids))


def tensor_meshgrid(self, ids, indexing="ij") -> List[int]:
    """One expanded view per input (``indexing`` 'ij' or 'xy'); each output's gradient sums back onto its vector."""
    ids = list(ids)
    sizes = [self.tensor_shape(i)[0] for i in ids]
    order = list(range(len(ids)))
    if indexing == "xy" and len(ids) >= 2:
        order[0], order[1] = 1, 0
    out_shape = [sizes[k] for k in order]
    outs = []
    for k, i in enumerate(ids):
        shape = [1] * len(ids)
        shape[order.index(k)] = sizes[k]
        outs.append(self.tensor_expand(self.tensor_reshape(i, shape=shape), shape=tuple(out_shape)))
    return outs


def tensor_rfft2(self, x, s=None, norm=None):
    return self._apply("rfft2", [x], s=s, norm=norm)


def tensor_rfftn(self, x, s=None, dim=None, norm=None):
    return self._apply("rfftn", [x], s=s, dim=None if dim is None else tuple(dim), norm=norm)


def tensor_irfft2(self, z, s=None, norm=None):
    return self._apply("irfft2", [z], s=s, norm=norm)


def tensor_fft_norm(self, x, n=None, norm="backward"):
    return self.tensor_fft(x, n=n, norm=norm)


def tensor_split_with_sizes(self, x, sizes, dim=0) -> List[int]:
    outs, off = [], 0
    for s in sizes:
        outs.append(self.tensor_narrow(x, dim=dim, start=off, length=int(s)))
        off += int(s)
    return outs


def tensor_roll_dims(self, x, shifts, dims):
    return self.tensor_roll(x, shifts=tuple(shifts), dims=tuple(dims))


def tensor_swapaxes(self, x, a, b):
    return self.tensor_transpose(x, dim0=a, dim1=b)


def tensor_broadcast_to(self, x, shape):
    return self.tensor_expand(x, shape=tuple(shape))


def tensor_cummax_dim(self, x, dim):
    return self.tensor_cummax(x, dim=dim)


def tensor_cummin_dim(self, x, dim):
    return self.tensor_cummin(x, dim=dim)


def tensor_scaled_dot_product_attention_gqa(self, q, k, v, mask=None, is_causal=False, scale=None, enable_gqa=True):
    """Attention with fewer key / value heads than query heads: each key / value head serves a group of
    ``Hq / Hkv`` consecutive query heads (the heads are repeated with ``repeat_interleave``, whose rule sums the
    group's gradients back)."""
    hq, hkv = self.tensor_shape(q)[-3], self.tensor_shape(k)[-3]
    if hq != hkv:
        if not enable_gqa or hq % hkv:
            raise ValueError(f"query heads ({hq}) must be a multiple of key/value heads ({hkv}) with enable_gqa")
        hd = len(self.tensor_shape(k)) - 3
        k = tensor_repeat_interleave(self, k, hq // hkv, dim=hd)
        v = tensor_repeat_interleave(self, v, hq // hkv, dim=hd)
    return self.tensor_sdpa(q, k, v, mask, is_causal=is_causal, scale=scale)


# ------------------------------------------------------------------------------------ matrices: second names, factor pairs
def tensor_cholesky(self, a, upper=False):
    l = self.tensor_linalg_cholesky(a)
    return self._apply("matrix_transpose", [l]) if upper else l


def tensor_cholesky_solve(self, b, l, upper=False):
    return self.tensor_linalg_cholesky_solve(b, l, upper=upper)


def tensor_cholesky_inverse(self, l, upper=False):
    return self._apply("cholesky_inverse", [l], upper=upper)


def tensor_triangular_solve(self, a, b, upper=True):
    return self.tensor_linalg_triangular_solve(a, b, upper=upper)


def tensor_matrix_power(self, a, n):
    return self.tensor_linalg_matrix_power(a, n=int(n))


def tensor_matrix_norm(self, a, ord="fro"):
    return self.tensor_linalg_matrix_norm(a, ord=ord)


def tensor_qr(self, a, reduced=True) -> Tuple[int, int]:
    if reduced:
        return self.tensor_linalg_qr(a)
    q, r = torch.linalg.qr(self.tensor(a), mode="complete")
    return _new(self, q, False, self.tensor_dtype(a)), _new(self, r, False, self.tensor_dtype(a))


def tensor_lu_factor(self, a) -> Tuple[int, List[int]]:
    """Packed ``LU`` (unit lower below the diagonal, upper on and above) and the 1-based row pivots."""
    lu, piv = torch.linalg.lu_factor(self.tensor(a))
    return _new(self, lu, False, self.tensor_dtype(a)), [int(p) for p in piv.reshape(-1).tolist()]


def tensor_lu_solve(self, lu, pivots, b):
    """Solve ``A x = b`` from ``tensor_lu_factor``'s outputs.  The solve is linear in ``b``: its rule is the
    transposed solve ``db = A^-T grad``."""
    LU = self.tensor(lu)
    piv = torch.as_tensor(list(pivots), dtype=torch.int32, device=LU.device).reshape(LU.shape[:-1])

    def fwd(ctx, ts):
        return torch.linalg.lu_solve(LU, piv, ts[0])

    def bwd(ctx, g):
        return [torch.linalg.lu_solve(LU.to(g.dtype), piv, g, adjoint=True)]

    return self.tensor_apply_function([b], fwd, bwd)


def tensor_ormqr(self, a, tau, c, left=True, transpose=False):
    out = torch.ormqr(self.tensor(a), self.tensor(tau), self.tensor(c), left, transpose)
    return _new(self, out, False, self.tensor_dtype(c))


def tensor_linalg_pinv_hermitian(self, a):
    """Pseudo-inverse of a symmetric matrix from its eigendecomposition (eigenvalues below ``eps * max|w| * n`` dropped)."""
    A = self.tensor(a)
    return _new(self, torch.linalg.pinv(A, hermitian=True), False, self.tensor_dtype(a))


def tensor_eigh(self, a) -> Tuple[int, int]:
    return self.tensor_linalg_eigh(a)


# ------------------------------------------------------------------------------------ non-differentiable multi-output forms
def tensor_histogram(self, x, bins, min=0.0, max=0.0, weight=None, density=False) -> Tuple[int, int]:
    """``(hist, bin_edges)``; ``min == max`` means the data range."""
    t = self.tensor(x).detach().to("cpu", torch.float64).reshape(-1)
    w = None if weight is None else self.tensor(weight).detach().to("cpu", torch.float64).reshape(-1)
    rng = None if min == max else (float(min), float(max))
    h = torch.histogram(t, int(bins), range=rng, weight=w, density=bool(density))
    return _new(self, h.hist, False), _new(self, h.bin_edges, False)


def tensor_histogramdd(self, x, bins, ranges=None, density=False) -> Tuple[int, List[int]]:
    t = self.tensor(x).detach().to("cpu", torch.float64)
    rng = None if ranges is None else [float(v) for v in ranges]
    h = torch.histogramdd(t, [int(b) for b in bins], range=rng, density=bool(density))
    return _new(self, h.hist, False), [_new(self, e, False) for e in h.bin_edges]


def tensor_unique_consecutive(self, x, return_inverse=False, return_counts=False):
    """``(values, inverse or None, counts or None)`` of runs of equal elements (flattened input)."""
    v, inv, cnt = torch.unique_consecutive(self.tensor(x).reshape(-1), return_inverse=True, return_counts=True)
    dt = self.tensor_dtype(x)
    return (_new(self, v, False, dt), _new(self, inv.to(torch.float64), False) if return_inverse else None,
            _new(self, cnt.to(torch.float64), False) if return_counts else None)


def tensor_gradients_iter(self, report):
    """Iterate ``(node id, gradient values)`` over every gradient a backward report holds, in node order."""
    for nid in sorted(report.gradients):
        yield nid, report.gradients[nid].detach().to("cpu", torch.float64).reshape(-1).tolist()


def tensor_is_leaf(self, nid) -> bool:
    return self.tensor_tape.tensor_is_leaf(nid)


def tensor_grad_fn(self, nid):
    return self.tensor_tape.tensor_grad_fn(nid)


def tensor_has_hooks(self, nid) -> bool:
    return self.tensor_tape.tensor_has_hooks(nid)


def tensor_retains_grad(self, nid) -> bool:
    return self.tensor_tape.tensor_retains_grad(nid)


def tensor_node_count(self) -> int:
    return self.tensor_tape.node_count()


def tensor_detach_(self, nid) -> int:
    """Detach a node in place: it becomes a leaf without history that does not require grad."""
    self.tensor_tape.detach_in_place(nid)
    return nid


def set_detect_anomaly(self, enabled: bool) -> None:
    """Tape-level anomaly mode: every backward pass of this session checks its gradients for NaN / Inf."""
    self.tensor_tape.set_detect_anomaly(enabled)


def is_detect_anomaly(self) -> bool:
    return self.tensor_tape.is_detect_anomaly()


def set_grad_enabled(self, enabled: bool) -> bool:
    """Switch gradient recording; returns the previous setting (nesting is the caller's business, unlike
    ``no_grad_enter`` / ``no_grad_exit`` which count)."""
    prev = self.is_grad_enabled()
    self._no_grad_depth = 0 if enabled else max(self._no_grad_depth, 1)
    self.tensor_tape.grad_enabled = bool(enabled)
    return prev


def tensor_register_hook(self, nid, fn):
    return self.register_tensor_hook(nid, fn)


# ------------------------------------------------------------------------------------ in-place variants
def _inplace_binary(name, fn):
    def method(self, a, b, *extra):
        return _inplace(self, a, lambda t: fn(t, self.tensor(b), *extra))
    method.__name__ = name
    method.__doc__ = f"In-place ``{name[7:-1]}``: overwrites the first tensor, bumps its version, returns its id."
    return method


def tensor_where_(self, a, cond, other):
    """``a = where(cond, a, other)`` in place."""
    return _inplace(self, a, lambda t: t.copy_(torch.where(self.tensor(cond).bool(), t, self.tensor(other))))


def tensor_masked_fill_(self, a, mask, value):
    return _inplace(self, a, lambda t: t.masked_fill_(self.tensor(mask).bool(), value))


def tensor_addcmul_(self, a, t1, t2, value=1.0):
    return _inplace(self, a, lambda t: t.addcmul_(self.tensor(t1), self.tensor(t2), value=value))


def tensor_lerp_(self, a, end, weight):
    """``a += weight * (end - a)`` in place; ``weight`` is a number."""
    return _inplace(self, a, lambda t: t.lerp_(self.tensor(end), float(weight)))


def tensor_sigmoid_(self, a):
    return _inplace(self, a, lambda t: t.sigmoid_())


def tensor_acosh_(self, a):
    return _inplace(self, a, lambda t: t.acosh_())


def tensor_ones_(self, a):
    return _inplace(self, a, lambda t: t.fill_(1.0))


# ------------------------------------------------------------------------------------ samplers (session stream)
def _u(self, n):
    return self.rng.uniform(n)


def _shape_out(self, t, shape, requires_grad):
    return _new(self, t.reshape(tuple(shape)), requires_grad)


def tensor_1d(self, values, requires_grad=False):
    return self.tensor_variable(list(values), [len(values)], requires_grad)


def tensor_normal(self, mean, std, shape, requires_grad=False):
    return _shape_out(self, mean + std * self.rng.normal(_numel(shape)), shape, requires_grad)


def tensor_log_normal(self, mean, std, shape, requires_grad=False):
    return _shape_out(self, torch.exp(mean + std * self.rng.normal(_numel(shape))), shape, requires_grad)


def tensor_half_normal(self, scale, shape, requires_grad=False):
    return _shape_out(self, scale * self.rng.normal(_numel(shape)).abs(), shape, requires_grad)


def tensor_cauchy(self, median, sigma, shape, requires_grad=False):
    u = _u(self, _numel(shape))
    return _shape_out(self, median + sigma * torch.tan(math.pi * (u - 0.5)), shape, requires_grad)


def tensor_exponential(self, rate, shape, requires_grad=False):
    u = _u(self, _numel(shape))
    return _shape_out(self, -torch.log1p(-u) / rate, shape, requires_grad)


def tensor_weibull(self, scale, concentration, shape, requires_grad=False):
    u = _u(self, _numel(shape))
    return _shape_out(self, scale * (-torch.log1p(-u)).pow(1.0 / concentration), shape, requires_grad)


def _gamma_draws(self, alpha: float, n: int) -> torch.Tensor:
    """Marsaglia-Tsang squeeze for shape ``alpha`` (boosted by ``u^(1/alpha)`` below 1), vectorised: each round
    draws candidates for the positions still open."""
    boost = alpha < 1.0
    a = alpha + 1.0 if boost else alpha
    d = a - 1.0 / 3.0
    c = 1.0 / math.sqrt(9.0 * d)
    out = torch.empty(n, dtype=torch.float64)
    open_idx = torch.arange(n)
    while open_idx.numel():
        m = open_idx.numel()
        z = self.rng.normal(m)
        u = _u(self, m)
        v = (1.0 + c * z) ** 3
        ok = (v > 0) & (torch.log(u) < 0.5 * z * z + d - d * v + d * torch.log(torch.where(v > 0, v, torch.ones_like(v))))
        out[open_idx[ok]] = d * v[ok]
        open_idx = open_idx[~ok]
    if boost:
        out = out * _u(self, n).pow(1.0 / alpha)
    return out


def tensor_gamma(self, concentration, rate, shape, requires_grad=False):
    return _shape_out(self, _gamma_draws(self, float(concentration), _numel(shape)) / rate, shape, requires_grad)


def tensor_chi2(self, df, shape, requires_grad=False):
    return _shape_out(self, 2.0 * _gamma_draws(self, 0.5 * float(df), _numel(shape)), shape, requires_grad)


def tensor_beta(self, a, b, shape, requires_grad=False):
    n = _numel(shape)
    x, y = _gamma_draws(self, float(a), n), _gamma_draws(self, float(b), n)
    return _shape_out(self, x / (x + y), shape, requires_grad)


def tensor_studentt(self, df, shape, requires_grad=False):
    n = _numel(shape)
    z = self.rng.normal(n)
    chi2 = 2.0 * _gamma_draws(self, 0.5 * float(df), n)
    return _shape_out(self, z / torch.sqrt(chi2 / df), shape, requires_grad)


def tensor_dirichlet(self, alphas, shape, requires_grad=False):
    """Samples of shape ``shape + [len(alphas)]``: independent gammas normalised over the last dimension."""
    n = _numel(shape)
    g = torch.stack([_gamma_draws(self, float(a), n) for a in alphas], -1)
    return _new(self, (g / g.sum(-1, keepdim=True)).reshape(tuple(shape) + (len(alphas),)), requires_grad)


def tensor_binomial(self, total_count, p, shape, requires_grad=False):
    n = _numel(shape)
    u = _u(self, n * int(total_count)).reshape(n, int(total_count))
    return _shape_out(self, (u < p).sum(-1).to(torch.float64), shape, requires_grad)


def _fill_from(self, nid, values):
    t = self.tensor(nid)
    t.copy_(values.reshape(t.shape).to(device=t.device, dtype=t.dtype))
    self.tensor_tape.bump_version(nid)
    return nid


def tensor_log_normal_(self, nid, mean=1.0, std=2.0):
    return _fill_from(self, nid, torch.exp(mean + std * self.rng.normal(self.tensor_numel(nid))))


def tensor_cauchy_(self, nid, median=0.0, sigma=1.0):
    return _fill_from(self, nid, median + sigma * torch.tan(math.pi * (_u(self, self.tensor_numel(nid)) - 0.5)))


def tensor_exponential_(self, nid, rate=1.0):
    return _fill_from(self, nid, -torch.log1p(-_u(self, self.tensor_numel(nid))) / rate)


def tensor_geometric_(self, nid, p):
    """Number of Bernoulli(p) trials up to and including the first success (support 1, 2, ...)."""
    u = _u(self, self.tensor_numel(nid))
    return _fill_from(self, nid, torch.ceil(torch.log1p(-u) / math.log1p(-p)).clamp_min(1.0))


# ------------------------------------------------------------------------------------ raw recurrent forwards
def _cell_step(kind, x_t, h, c, w, nonlinearity):
    w_ih, w_hh, b_ih, b_hh = w
    gi = x_t @ w_ih.t() + (b_ih if b_ih is not None else 0)
    gh = h @ w_hh.t() + (b_hh if b_hh is not None else 0)
    if kind == "rnn":
        return (torch.tanh if nonlinearity == "tanh" else torch.relu)(gi + gh), None
    if kind == "lstm":
        i, f, g, o = (gi + gh).chunk(4, -1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        return torch.sigmoid(o) * torch.tanh(c), c
    ir, iz, inn = gi.chunk(3, -1)
    hr, hz, hn = gh.chunk(3, -1)
    r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
    n = torch.tanh(inn + r * hn)
    return (1 - z) * n + z * h, None


def _recurrent(self, kind, input, hx, weights, bidirectional, batch_first, nonlinearity="tanh"):
    """Stacked (optionally bidirectional) recurrence over ``input`` [T, B, I] (or [B, T, I] with ``batch_first``).
    ``weights`` holds one ``(w_ih, w_hh, b_ih or None, b_hh or None)`` tuple of node ids per layer and direction
    (forward then reverse).  Gate order: LSTM i, f, g, o; GRU r, z, n.  Outputs are history-free leaves."""
    x = self.tensor(input).detach()
    unbatched = x.dim() == 2
    if unbatched:
        x = x.unsqueeze(1)
    elif batch_first:
        x = x.transpose(0, 1)
    ndir = 2 if bidirectional else 1
    layers = len(weights) // ndir
    W = [tuple(None if i is None else self.tensor(i).detach() for i in w) for w in weights]
    hid = W[0][1].shape[1]
    B = x.shape[1]

    def state(idx):
        if hx is None:
            return torch.zeros(layers * ndir, B, hid, dtype=x.dtype, device=x.device)
        t = self.tensor(hx[idx] if kind == "lstm" else hx).detach()
        return t.unsqueeze(1) if unbatched else t

    h0 = state(0)
    c0 = state(1) if kind == "lstm" else None
    hs, cs = [], []
    for l in range(layers):
        outs = []
        for d in range(ndir):
            k = l * ndir + d
            h, c = h0[k], (c0[k] if c0 is not None else None)
            steps = range(x.shape[0] - 1, -1, -1) if d == 1 else range(x.shape[0])
            seq = [None] * x.shape[0]
            for t in steps:
                h, c = _cell_step(kind, x[t], h, c, W[k], nonlinearity)
                seq[t] = h
            outs.append(torch.stack(seq))
            hs.append(h)
            cs.append(c)
        x = torch.cat(outs, -1)
    out = x.squeeze(1) if unbatched else (x.transpose(0, 1) if batch_first else x)
    hn = torch.stack(hs)
    dt = self.tensor_dtype(input)
    mk = lambda t: _new(self, (t.squeeze(1) if unbatched else t).contiguous(), False, dt)   # noqa: E731
    if kind == "lstm":
        return _new(self, out.contiguous(), False, dt), (mk(hn), mk(torch.stack(cs)))
    return _new(self, out.contiguous(), False, dt), mk(hn)


def tensor_rnn(self, input, hx, weights, bidirectional=False, batch_first=False, nonlinearity="tanh"):
    return _recurrent(self, "rnn", input, hx, weights, bidirectional, batch_first, nonlinearity)


def tensor_lstm(self, input, hx, weights, bidirectional=False, batch_first=False):
    return _recurrent(self, "lstm", input, hx, weights, bidirectional, batch_first)


def tensor_gru(self, input, hx, weights, bidirectional=False, batch_first=False):
    return _recurrent(self, "gru", input, hx, weights, bidirectional, batch_first)


# ------------------------------------------------------------------------------------ second batch (parity matrix names)
def tensor_cross_entropy_label_smoothing(self, logits, target, label_smoothing, reduction="mean"):
    return tensor_cross_entropy_full(self, logits, target, None, None, reduction, float(label_smoothing))


def tensor_cross_entropy_soft(self, logits, probs, reduction="mean"):
    """Cross-entropy against class probabilities (soft targets)."""
    return self._apply("cross_entropy_soft", [logits, probs], reduction=reduction)


def tensor_triplet_margin_loss_swap(self, anchor, positive, negative, margin=1.0, p=2.0, swap=True, reduction="mean"):
    """Triplet loss with the distance swap: the negative distance is the smaller of d(a, n) and d(p, n)."""
    eps = 1e-6

    def dist(a, b):
        d = self.tensor_add_scalar(self.tensor_sub(a, b), c=eps)
        return self.tensor_norm_dim(d, p=float(p), dim=-1 % len(self.tensor_shape(a)))
    dap, dan = dist(anchor, positive), dist(anchor, negative)
    if swap:
        dpn = dist(positive, negative)
        dan = self.tensor_sub(dan, self.tensor_relu(self.tensor_sub(dan, dpn)))          # min(dan, dpn)
    loss = self.tensor_relu(self.tensor_add_scalar(self.tensor_sub(dap, dan), c=float(margin)))
    if reduction == "mean":
        return self.tensor_mean(loss)
    return self.tensor_sum(loss) if reduction == "sum" else loss


def tensor_linalg_solve_triangular(self, a, b, upper=True):
    return self.tensor_linalg_triangular_solve(a, b, upper=upper)


def tensor_unflatten_dim(self, x, dim, sizes):
    shape = self.tensor_shape(x)
    dim = dim % len(shape)
    return self.tensor_reshape(x, shape=tuple(shape[:dim]) + tuple(int(v) for v in sizes) + tuple(shape[dim + 1:]))


def tensor_flatten_dims(self, x, start_dim=0, end_dim=-1):
    return self.tensor_flatten(x, start=start_dim, end=end_dim)


def tensor_movedim_multi(self, x, sources, destinations):
    return self.tensor_movedim(x, source=tuple(sources), destination=tuple(destinations))


def tensor_unsqueeze_dim(self, x, dim):
    return self.tensor_unsqueeze(x, dim=dim)


def tensor_squeeze_neg_dim(self, x, dim):
    return self.tensor_squeeze(x, dim=dim % len(self.tensor_shape(x)))


def tensor_var_dims(self, x, dims, correction=1, keepdim=False):
    return self._apply("var_dims", [x], dims=tuple(dims), correction=correction, keepdim=keepdim)


def tensor_std_dims(self, x, dims, correction=1, keepdim=False):
    return self._apply("std_dims", [x], dims=tuple(dims), correction=correction, keepdim=keepdim)


def tensor_quantile_interpolation(self, x, q, interpolation="linear"):
    return _quantile(self, x, q, None, False, interpolation)


def tensor_nanquantile_interpolation(self, x, q, interpolation="linear"):
    return _quantile(self, x, q, None, False, interpolation, ignore_nan=True)


def tensor_searchsorted_side(self, sorted_seq, values, side="left"):
    if side not in ("left", "right"):
        raise ValueError("side must be 'left' or 'right'")
    return self.tensor_searchsorted(sorted_seq, values, right=(side == "right"))


def tensor_searchsorted_sorter(self, seq, values, sorter, right=False):
    """``seq`` need not be sorted: ``sorter`` holds the indices that sort it."""
    idx = torch.searchsorted(self.tensor(seq), self.tensor(values), right=right, sorter=self.tensor(sorter).long())
    return _new(self, idx.to(torch.float64), False)


def tensor_linalg_inv_ex(self, a):
    A = self.tensor(a)
    inv, info = torch.linalg.inv_ex(A)
    if int(info.max()) != 0:
        return None, int(info.max())
    return self.tensor_inverse(a), 0


def tensor_linalg_cholesky_ex(self, a, upper=False):
    _, info = torch.linalg.cholesky_ex(self.tensor(a), upper=upper)
    if int(info.max()) != 0:
        return None, int(info.max())
    return tensor_cholesky(self, a, upper), 0


def tensor_linalg_solve_ex(self, a, b):
    _, info = torch.linalg.solve_ex(self.tensor(a), self.tensor(b))
    if int(info.max()) != 0:
        return None, int(info.max())
    return self.tensor_linalg_solve(a, b), 0


def tensor_linalg_lu_factor_ex(self, a):
    lu, piv, info = torch.linalg.lu_factor_ex(self.tensor(a))
    return _new(self, lu, False, self.tensor_dtype(a)), [int(p) for p in piv.reshape(-1).tolist()], int(info.max())


def tensor_linalg_ldl_factor(self, a, hermitian=False):
    """``(LD, pivots)`` of a symmetric matrix (compact Bunch-Kaufman form)."""
    ld, piv = torch.linalg.ldl_factor(self.tensor(a), hermitian=hermitian)
    return _new(self, ld, False, self.tensor_dtype(a)), [int(p) for p in piv.reshape(-1).tolist()]


def tensor_linalg_ldl_solve(self, ld, pivots, b, hermitian=False):
    LD = self.tensor(ld)
    piv = torch.as_tensor(list(pivots), dtype=torch.int32, device=LD.device).reshape(LD.shape[:-1])
    return _new(self, torch.linalg.ldl_solve(LD, piv, self.tensor(b), hermitian=hermitian), False, self.tensor_dtype(b))


def tensor_geqrf(self, a):
    """``(packed Householder reflectors and R, tau)``; ``tensor_householder_product`` rebuilds Q."""
    qr, tau = torch.geqrf(self.tensor(a))
    dt = self.tensor_dtype(a)
    return _new(self, qr, False, dt), _new(self, tau, False, dt)


def tensor_cfloat(self, x):
    """Complex tensor with zero imaginary part (the ``[..., 2]`` layout), components in f32."""
    re = self.tensor_to_dtype(x, DType.F32)
    return self.tensor_complex(re, self.zeros_like(re))


def tensor_cdouble(self, x):
    re = self.tensor_to_dtype(x, DType.F64)
    return self.tensor_complex(re, self.zeros_like(re))


def tensor_conj(self, z):
    return self.tensor_complex_conj(z)


def tensor_ihfft(self, x, n=None, dim=-1):
    return self._apply("ihfft", [x], n=n, dim=dim)


def tensor_ihfft_norm(self, x, n=None, norm="backward", dim=-1):
    return self._apply("ihfft", [x], n=n, dim=dim, norm=norm)


def tensor_irfftn(self, z, s=None, dim=None):
    return self._apply("irfftn", [z], s=s, dim=None if dim is None else tuple(dim))


def tensor_irfftn_norm(self, z, s=None, dim=None, norm="backward"):
    return self._apply("irfftn", [z], s=s, dim=None if dim is None else tuple(dim), norm=norm)


def tensor_rfftn_norm(self, x, s=None, dim=None, norm="backward"):
    return tensor_rfftn(self, x, s, dim, norm)


def tensor_irfft_norm(self, z, n=None, norm="backward"):
    s = None if n is None else (int(n),)
    return self._apply("irfftn", [z], s=s, dim=(-1,), norm=norm)


def tensor_hfft_norm(self, z, n=None, norm="backward"):
    """``hfft`` of a half spectrum under ``norm``: the default-norm transform rescaled (the transform is linear)."""
    out = self.tensor_hfft(z, n=n)
    length = self.tensor_shape(out)[-1]
    scale = {"backward": 1.0, None: 1.0, "ortho": 1.0 / math.sqrt(length), "forward": 1.0 / length}[norm]
    return out if scale == 1.0 else self.tensor_mul_scalar(out, c=scale)


def tensor_fftn_norm(self, x, norm="backward"):
    return self.tensor_fftn(x, norm=norm)


def tensor_ifftn_norm(self, z, norm="backward"):
    return self.tensor_ifftn(z, norm=norm)


def tensor_ifft2_norm(self, z, norm="backward"):
    return self.tensor_ifft2(z, norm=norm)


def tensor_fft_along_dim(self, x, dim, n=None, norm=None):
    return self.tensor_fft(x, n=n, dim=dim, norm=norm)


def tensor_any(self, x, dim=None, keepdim=False):
    return self._apply("any", [x], dim=dim, keepdim=keepdim)


def tensor_all(self, x, dim=None, keepdim=False):
    return self._apply("all", [x], dim=dim, keepdim=keepdim)


def tensor_trapezoid_dx(self, y, dx=1.0, dim=-1):
    return tensor_trapezoid(self, y, None, dim, dx)


def tensor_trapz(self, y, x=None, dim=-1):
    return tensor_trapezoid(self, y, x, dim)


def tensor_cumulative_trapezoid_dx(self, y, dx=1.0, dim=-1):
    return tensor_cumulative_trapezoid(self, y, None, dim, dx)


def tensor_vecdot(self, a, b, dim=-1):
    return self._apply("vecdot", [a, b], dim=dim)


def tensor_roll_flat(self, x, shift):
    return self._apply("roll_flat", [x], shift=int(shift))


def tensor_linalg_tensorinv(self, x, ind=2):
    return self._apply("linalg_tensorinv", [x], ind=int(ind))


def tensor_slogdet(self, a):
    return self.tensor_linalg_slogdet(a)


def tensor_unique_dim(self, x, dim):
    """Unique slices along ``dim`` in sorted order: ``(values, inverse, counts)``."""
    v, inv, cnt = torch.unique(self.tensor(x), dim=dim, return_inverse=True, return_counts=True)
    return (_new(self, v, False, self.tensor_dtype(x)), _new(self, inv.to(torch.float64), False), _new(self, cnt.to(torch.float64), False))


def tensor_addmm_scaled(self, x, m1, m2, beta, alpha):
    return self.tensor_addmm(x, m1, m2, beta=float(beta), alpha=float(alpha))


# ------------------------------------------------------------------------------------ metadata, splits, misc (third batch)
def tensor_stride(self, x) -> List[int]:
    return list(self.tensor(x).stride())


def tensor_dim(self, x) -> int:
    return self.tensor(x).dim()


def tensor_nelement(self, x) -> int:
    return self.tensor(x).numel()


def tensor_clone(self, x):
    """A copy that stays in the graph: its gradient flows to ``x`` unchanged."""
    return self.tensor_contiguous(self.tensor_mul_scalar(x, c=1.0))


def tensor_bool(self, x):
    """0 / 1 mask of the non-zero elements (a node without history)."""
    return _new(self, (self.tensor(x) != 0).to(torch.float64), False, self.tensor_dtype(x))


def tensor_int_long(self, x):
    """Values truncated toward zero, as an int64 node (indices, labels)."""
    return self.tensor_tape.leaf(self.tensor(x).detach().to(torch.int64), False)


def tensor_broadcast_shapes(self, *shapes) -> List[int]:
    return list(torch.broadcast_shapes(*[tuple(s) for s in shapes]))


def tensor_array_split(self, x, sections, dim=0) -> List[int]:
    """``sections`` pieces along ``dim``: the first ``n % sections`` get one element more (numpy's rule)."""
    n = self.tensor_shape(x)[dim]
    base, extra = divmod(n, int(sections))
    return tensor_split_with_sizes(self, x, [base + (1 if k < extra else 0) for k in range(int(sections))], dim)


def tensor_nonzero_as_tuple(self, x) -> List[int]:
    return [_new(self, t.to(torch.float64), False) for t in torch.nonzero(self.tensor(x), as_tuple=True)]


def tensor_matrix_rank(self, a):
    return self.tensor_linalg_matrix_rank(a)


def tensor_kthvalue_dim(self, x, k, dim, keepdim=False):
    return tensor_kthvalue(self, x, k, dim, keepdim)


def tensor_ger(self, a, b):
    return self.tensor_outer(a, b)


def tensor_tensordot_dims(self, a, b, dims_a, dims_b):
    return self.tensor_tensordot(a, b, dims=(list(dims_a), list(dims_b)))


def tensor_fft_fftshift(self, x, dim=None):
    return self.tensor_fftshift(x, dim=dim) if dim is not None else self.tensor_fftshift(x)


def tensor_fft_ifftshift(self, x, dim=None):
    return self.tensor_ifftshift(x, dim=dim) if dim is not None else self.tensor_ifftshift(x)


def tensor_scalbn(self, x, n):
    """``x * 2^n`` for an integer ``n``."""
    return self.tensor_mul_scalar(x, c=float(2.0 ** int(n)))


def tensor_frexp(self, x) -> Tuple[int, int]:
    """``(mantissa in [0.5, 1), integer exponent)`` with ``x = mantissa * 2^exponent``.  The mantissa is ``x``
    scaled by a constant power of two per element, so its gradient is ``grad * 2^-exponent``."""
    m, e = torch.frexp(self.tensor(x).detach())
    scale = self.tensor_tape.leaf(torch.exp2(-e.to(self.tensor(x).dtype)), False)
    return self.tensor_mul(x, scale), _new(self, e.to(torch.float64), False)


def tensor_modf(self, x) -> Tuple[int, int]:
    """``(fractional part, integral part)``, both with the sign of ``x``."""
    return self.tensor_frac(x), self.tensor_trunc(x)


def tensor_lobpcg(self, a, k=1, niter=200, tol=1e-10, seed=0x4654) -> Tuple[int, int]:
    """The ``k`` largest eigenpairs of a symmetric matrix by locally optimal block preconditioned conjugate
    gradients (no preconditioner): Rayleigh-Ritz over ``[X, R, P]`` each iteration.  Outputs are leaves."""
    A = self.tensor(a).detach().to(torch.float64)
    n = A.shape[-1]
    k = int(k)
    if A.dim() != 2 or A.shape[0] != n or not 0 < k <= n:
        raise ValueError("lobpcg needs a square matrix and 0 < k <= n")
    g = torch.Generator().manual_seed(int(seed))
    X = torch.linalg.qr(torch.randn(n, k, generator=g, dtype=torch.float64)).Q
    P = None
    for _ in range(int(niter)):
        AX = A @ X
        lam = (X * AX).sum(0)
        R = AX - X * lam
        if float(R.norm()) <= tol * max(1.0, float(lam.abs().max())):
            break
        S_ = torch.cat([X, R] + ([P] if P is not None else []), 1)
        Q = torch.linalg.qr(S_).Q
        keep = torch.linalg.matrix_rank(S_)
        Q = Q[:, : int(keep)] if int(keep) >= k else Q
        w, V = torch.linalg.eigh(Q.t() @ A @ Q)
        C = V[:, -k:].flip(1)                                # the k largest, descending
        Xn = Q @ C
        P = Xn - X @ (X.t() @ Xn)
        P = None if float(P.norm()) < 1e-14 else P
        X = Xn
    lam = (X * (A @ X)).sum(0)
    order = torch.argsort(lam, descending=True)
    dt = self.tensor_dtype(a)
    return _new(self, lam[order], False, dt), _new(self, X[:, order], False, dt)


def tensor_von_mises(self, loc, concentration, shape, requires_grad=False):
    """Best-Fisher rejection sampler of the von Mises distribution on ``(-pi, pi]``."""
    n = _numel(shape)
    kappa = float(concentration)
    if kappa < 1e-8:
        return _shape_out(self, (2 * math.pi * _u(self, n) - math.pi), shape, requires_grad)
    tau = 1.0 + math.sqrt(1.0 + 4.0 * kappa * kappa)
    rho = (tau - math.sqrt(2.0 * tau)) / (2.0 * kappa)
    r = (1.0 + rho * rho) / (2.0 * rho)
    out = torch.empty(n, dtype=torch.float64)
    open_idx = torch.arange(n)
    while open_idx.numel():
        m = open_idx.numel()
        u1, u2, u3 = _u(self, m), _u(self, m), _u(self, m)
        z = torch.cos(math.pi * u1)
        f = (1.0 + r * z) / (r + z)
        c = kappa * (r - f)
        ok = (c * (2.0 - c) - u2 > 0) | (torch.log(c / u2) + 1.0 - c >= 0)
        theta = torch.sign(u3 - 0.5) * torch.acos(f.clamp(-1.0, 1.0))
        out[open_idx[ok]] = theta[ok]
        open_idx = open_idx[~ok]
    out = torch.remainder(out + float(loc) + math.pi, 2 * math.pi) - math.pi
    return _shape_out(self, out, shape, requires_grad)


def tensor_fishersnedecor(self, df1, df2, shape, requires_grad=False):
    """F distribution: the ratio of two chi-square variates, each divided by its degrees of freedom."""
    n = _numel(shape)
    a = 2.0 * _gamma_draws(self, 0.5 * float(df1), n) / float(df1)
    b = 2.0 * _gamma_draws(self, 0.5 * float(df2), n) / float(df2)
    return _shape_out(self, a / b, shape, requires_grad)


def tensor_negative_binomial(self, total_count, p, shape, requires_grad=False):
    """Failures before ``total_count`` successes of probability ``1 - p`` each (torch's convention: ``p`` is the
    probability of a failure... of the counted kind), drawn as a gamma-Poisson mixture."""
    n = _numel(shape)
    lam = _gamma_draws(self, float(total_count), n) * (float(p) / (1.0 - float(p)))
    out = torch.zeros(n, dtype=torch.float64)
    for i, l in enumerate(lam.tolist()):                 # Poisson by inversion, as ``poisson`` does
        u = float(_u(self, 1)[0])
        pr = math.exp(-l)
        s_, x = pr, 0
        while u > s_ and x < 100000:
            x += 1
            pr *= l / x
            s_ += pr
        out[i] = x
    return _shape_out(self, out, shape, requires_grad)


def _inplace_from_op(name, op, n_tensors=1):
    """In-place form of a rule-table operator: ``a <- op(a, ...)``; follows the version rules of ``tensor_add_``."""
    def method(self, a, *rest, **kw):
        others = [self.tensor(r) for r in rest[: n_tensors - 1]]
        extra = rest[n_tensors - 1:]
        from .autograd.functions import OPS
        fwd = OPS[op].fwd
        return _inplace(self, a, lambda t: t.copy_(fwd(t, *others, *extra, **kw).to(t.dtype)))
    method.__name__ = name
    method.__doc__ = f"In-place ``{op}``: overwrites the first tensor, bumps its version, returns its id."
    return method


_INPLACE_UNARY_OPS = ["erf", "erfc", "logit", "nan_to_num", "asin", "acos", "atan", "sinh", "cosh", "tanh", "asinh", "atanh", "sin", "cos",
                      "tan", "exp", "exp2", "expm1", "log", "log2", "log10", "log1p", "sqrt", "rsqrt", "reciprocal", "abs", "sign",
                      "floor", "ceil", "round", "trunc", "frac", "relu", "relu6", "gelu", "silu", "mish", "elu", "selu", "celu",
                      "leaky_relu", "hardswish", "hardsigmoid", "hardtanh", "hardshrink", "softshrink", "threshold", "softplus",
                      "deg2rad", "rad2deg", "square", "tril", "triu", "pow", "float_power", "clamp_min", "clamp_max"]
_INPLACE_BINARY_OPS = ["logaddexp", "logaddexp2", "gcd", "lcm", "fmax", "fmin", "minimum", "nextafter", "ldexp", "pow_tensor", "atan2"]
_INPLACE_TERNARY_OPS = ["addcdiv"]


def tensor_bernoulli_(self, nid, p=0.5):
    """Fill with Bernoulli(p) draws of the session stream (1.0 where ``u < p``)."""
    return _fill_from(self, nid, (_u(self, self.tensor_numel(nid)) < float(p)).to(torch.float64))


# ------------------------------------------------------------------------------------ custom functions over live inputs
# The reference has one entry point per ownership pattern of a custom autograd function
# (ft-autograd/src/lib.rs:9065 ``apply_function_f64_borrowed_inputs``, :9161 ``..._borrowed_forward``, :9250
# ``..._saved_forward``, :9435 ``apply_function_f32_output_borrowed_inputs``, plus the create-graph forms).  Tensors
# here are device buffers that the tape already holds by reference, so the patterns differ only in what the
# backward closure receives and in which dtype is enforced.
def _custom_inputs(self, inputs, dtype):
    from .session import FunctionCtx
    tape = self.tensor_tape
    inputs = list(inputs)
    vals = [tape.value(i) for i in inputs]
    if dtype is not None:
        for i, v in zip(inputs, vals):
            if v.dtype != dtype:
                raise AutogradError(f"custom function input {i} holds {v.dtype}; this entry point takes {dtype}")
    ctx = FunctionCtx([tape.nodes[i].requires_grad and tape.grad_enabled for i in inputs])
    return tape, inputs, vals, ctx


def _check_versions(tape, inputs, versions):
    from .autograd.tape import BorrowedInputVersionMismatch
    for i, rec in zip(inputs, versions):
        if tape.version(i) != rec:
            raise BorrowedInputVersionMismatch(i, rec, tape.version(i))


def _custom_record(self, tape, inputs, ctx, out, out_dtype, vjp, cg=None):
    if out_dtype is not None and out.dtype != out_dtype:
        raise AutogradError(f"custom function returned {out.dtype}; this entry point produces {out_dtype}")
    self._record_dispatch("custom_function", any(ctx.needs_input_grad), "custom_function")
    if not any(ctx.needs_input_grad):
        return tape.leaf(out, requires_grad=False)
    return tape.record("custom_function", inputs, out, vjp, "custom autograd function backward", cg=cg)


def tensor_apply_function_borrowed_inputs(self, inputs, forward_fn, backward_fn, dtype=None, out_dtype=None) -> int:
    """``forward_fn(ctx, tensors) -> tensor``; ``backward_fn(ctx, grad_out, tensors) -> grads`` re-reads the LIVE
    inputs, so nothing is saved.  An input mutated in place between forward and backward is an error."""
    tape, inputs, vals, ctx = _custom_inputs(self, inputs, dtype)
    out = forward_fn(ctx, vals)
    versions = [tape.version(i) for i in inputs]

    def vjp(g, targets):
        _check_versions(tape, inputs, versions)
        return list(backward_fn(ctx, g, [tape.value(i) for i in inputs]))
    return _custom_record(self, tape, inputs, ctx, out, out_dtype, vjp)


def tensor_apply_function_f64_borrowed_inputs(self, inputs, forward_fn, backward_fn) -> int:
    return tensor_apply_function_borrowed_inputs(self, inputs, forward_fn, backward_fn, torch.float64, torch.float64)


def tensor_apply_function_f32_output_borrowed_inputs(self, inputs, forward_fn, backward_fn) -> int:
    """f32 inputs and output; the incoming gradient and the returned input gradients stay in the tape's gradient
    dtype (f64 by default), as in the reference's f32 conv / linear fast paths."""
    return tensor_apply_function_borrowed_inputs(self, inputs, forward_fn, backward_fn, torch.float32, torch.float32)


def tensor_apply_function_f64_borrowed_forward(self, inputs, forward_fn, backward_fn) -> int:
    """The forward reads the inputs in place; ``backward_fn(ctx, grad_out)`` uses only what ``ctx`` saved."""
    tape, inputs, vals, ctx = _custom_inputs(self, inputs, torch.float64)
    out = forward_fn(ctx, vals)
    return _custom_record(self, tape, inputs, ctx, out, torch.float64, lambda g, targets: list(backward_fn(ctx, g)))


def tensor_apply_function_f64_saved_forward(self, inputs, forward_fn, backward_fn) -> int:
    """``forward_fn(ctx) -> tensor``: the result was computed elsewhere (a fused loss cached by its producer) and
    only has to be attached to ``inputs``; the inputs are not handed to the forward at all."""
    tape, inputs, _, ctx = _custom_inputs(self, inputs, torch.float64)
    out = forward_fn(ctx)
    return _custom_record(self, tape, inputs, ctx, out, torch.float64, lambda g, targets: list(backward_fn(ctx, g)))


def tensor_apply_function_with_create_graph_borrowed_inputs(self, inputs, forward_fn, backward_fn, dtype=None,
                                                            out_dtype=None) -> int:
    """Twice-differentiable form: ``backward_fn(session, ctx, grad_id, input_ids) -> node ids`` builds the input
    gradients from session operators over the live input nodes (version-checked)."""
    tape, inputs, vals, ctx = _custom_inputs(self, inputs, dtype)
    out = forward_fn(ctx, vals)
    versions = [tape.version(i) for i in inputs]

    def vjp(g, targets):
        _check_versions(tape, inputs, versions)
        mark = len(tape)
        prev, tape.grad_enabled = tape.grad_enabled, False
        try:
            ids = backward_fn(self, ctx, tape.leaf(g, requires_grad=False), inputs)
            res = [None if i is None else tape.value(i) for i in ids]
        finally:
            tape.grad_enabled = prev
        tape.truncate_graph_to(mark)
        return res

    def cg(g_id):
        _check_versions(tape, inputs, versions)
        prev, tape.grad_enabled = tape.grad_enabled, True
        try:
            return list(backward_fn(self, ctx, g_id, inputs))
        finally:
            tape.grad_enabled = prev
    return _custom_record(self, tape, inputs, ctx, out, out_dtype, vjp, cg)


def tensor_apply_function_f32_output_with_create_graph_borrowed_inputs(self, inputs, forward_fn, backward_fn) -> int:
    return tensor_apply_function_with_create_graph_borrowed_inputs(self, inputs, forward_fn, backward_fn,
                                                                   torch.float32, torch.float32)


# value-level tape entry points under the session (the optimizer-facing forms of the reference)
def _tape_forward(name):
    def f(self, *args, **kwargs):
        return getattr(self.tensor_tape, name)(*args, **kwargs)
    f.__name__ = "tensor_" + name if not name.startswith("tensor_") else name
    f.__doc__ = f"``TensorTape.{name}`` of this session's tape."
    return f


tensor_leaf_tensor = _tape_forward("leaf_tensor")
tensor_leaf_f32 = _tape_forward("leaf_f32")
tensor_set_requires_grad = _tape_forward("set_tensor_requires_grad")
tensor_accumulated_gradient_values = _tape_forward("tensor_accumulated_gradient_values")
tensor_set_accumulated_gradient = _tape_forward("set_tensor_accumulated_gradient")
tensor_zero_accumulated_gradient = _tape_forward("zero_tensor_accumulated_gradient")
tensor_update_values = _tape_forward("update_tensor_values")
tensor_update_values_f32 = _tape_forward("update_tensor_values_f32")
tensor_update_values_with = _tape_forward("update_tensor_values_with")
tensor_update_values_with_accumulated_gradient = _tape_forward("update_tensor_values_with_accumulated_gradient")


def tensor_to_f16(self, a):
    return self.tensor_to_dtype(a, DType.F16)


def tensor_to_bf16(self, a):
    return self.tensor_to_dtype(a, DType.BF16)


# ------------------------------------------------------------------------------------ installation
_SECOND_NAMES = {
    # matrices
    "tensor_inverse": "tensor_inverse", "tensor_pinv": "tensor_linalg_pinv", "tensor_matrix_exp": "tensor_linalg_matrix_exp",
    "tensor_lstsq": "tensor_linalg_lstsq", "tensor_solve": "tensor_linalg_solve", "tensor_eigvalsh": "tensor_linalg_eigvalsh",
    "tensor_householder_product": "tensor_linalg_householder_product", "tensor_multi_dot": "tensor_linalg_multi_dot",
    # shape
    "tensor_swapdims": "tensor_swapaxes", "tensor_unsafe_chunk": "tensor_chunk",
    # factories and samplers under the tensor_ prefix
    "tensor_randn": "randn", "tensor_rand": "rand", "tensor_zeros": "zeros", "tensor_poisson": "poisson",
    "tensor_fft_fftfreq": "tensor_fftfreq", "tensor_fft_rfftfreq": "tensor_rfftfreq",
    "tensor_special_gammaln": "tensor_gammaln", "tensor_svdvals": "tensor_linalg_svdvals", "tensor_linalg_cross": "tensor_cross",
}

_INPLACE_BINARY = {
    "tensor_maximum_": lambda t, o: t.copy_(torch.maximum(t, o)), "tensor_xlogy_": lambda t, o: t.xlogy_(o),
    "tensor_remainder_": lambda t, o: t.remainder_(o), "tensor_hypot_": lambda t, o: t.hypot_(o),
    "tensor_heaviside_": lambda t, o: t.heaviside_(o), "tensor_fmod_": lambda t, o: t.fmod_(o),
    "tensor_copysign_": lambda t, o: t.copysign_(o), "tensor_atan2_": lambda t, o: t.atan2_(o),
}


def install(cls) -> None:
    from ._session_extras import _alias
    g = globals()
    for name, fn in list(g.items()):
        if (name.startswith("tensor_") or name in ("set_detect_anomaly", "is_detect_anomaly", "set_grad_enabled")) and callable(fn):
            setattr(cls, name, fn)
    for name, fn in _INPLACE_BINARY.items():
        setattr(cls, name, _inplace_binary(name, fn))
    for name, target in _SECOND_NAMES.items():
        if name != target and hasattr(cls, target):
            setattr(cls, name, _alias(target, name))
    from .autograd.functions import OPS
    for ops, n in ((_INPLACE_UNARY_OPS, 1), (_INPLACE_BINARY_OPS, 2), (_INPLACE_TERNARY_OPS, 3)):
        for op in ops:
            name = "tensor_" + ("pow" if op == "pow_tensor" else op) + "_"
            if op in OPS and not hasattr(cls, name):
                setattr(cls, name, _inplace_from_op(name, op, n))
