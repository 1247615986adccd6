"""Factories, random sampling, comparisons, initialisers and non-differentiable utilities of
``FrankenTorchSession`` (installed onto the class by ``install``).

Random draws come from the session's xoshiro256++ stream (seed 42 by default) and follow the
reference's conventions, recovered from its seeded fixtures
(ft-conformance/fixtures/tensor_random_cases.json, tensor_init_cases.json):
``rand`` = top-53-bit uniforms; ``randn`` = Box-Muller using both branches of each pair;
initialisers' normals use only the cosine branch (one normal per two uniforms);
``randint`` = ``low + floor(u * (high-low))``; ``randperm`` = Fisher-Yates from the top index
with ``j = floor(u * (i+1))``; ``bernoulli`` = ``u < p``; ``multinomial`` = inverse CDF on the
un-renormalised remaining weights, falling back to the last positive weight.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .core.dtype import DType


def _new(self, t: torch.Tensor, requires_grad: bool = False, dtype: Optional[DType] = None) -> int:
    dt = (dtype or (DType.F64 if not self.is_cuda else self.default_dtype)).to_torch()
    if not t.is_floating_point() and dtype is None:
        dt = t.dtype
    return self.tensor_tape.leaf(t.to(device=self.device, dtype=dt), requires_grad)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


# ------------------------------------------------------------------------------------ factories
def zeros(self, shape, requires_grad=False, dtype=None):
    return _new(self, torch.zeros(tuple(shape), dtype=torch.float64), requires_grad, dtype)


def ones(self, shape, requires_grad=False, dtype=None):
    return _new(self, torch.ones(tuple(shape), dtype=torch.float64), requires_grad, dtype)


def full(self, shape, fill_value, requires_grad=False, dtype=None):
    return _new(self, torch.full(tuple(shape), float(fill_value), dtype=torch.float64), requires_grad, dtype)


def zeros_like(self, nid, requires_grad=False):
    return _new(self, torch.zeros_like(self.tensor(nid), dtype=torch.float64), requires_grad, self.tensor_dtype(nid))


def ones_like(self, nid, requires_grad=False):
    return _new(self, torch.ones_like(self.tensor(nid), dtype=torch.float64), requires_grad, self.tensor_dtype(nid))


def full_like(self, nid, fill_value, requires_grad=False):
    return _new(self, torch.full_like(self.tensor(nid), float(fill_value), dtype=torch.float64), requires_grad,
                self.tensor_dtype(nid))


def eye(self, n, m=None, requires_grad=False, dtype=None):
    return _new(self, torch.eye(n, m if m is not None else n, dtype=torch.float64), requires_grad, dtype)


def arange(self, start, end=None, step=1.0, requires_grad=False, dtype=None):
    if end is None:
        start, end = 0.0, start
    if step == 0:
        raise ValueError("arange step must be non-zero")
    return _new(self, torch.arange(float(start), float(end), float(step), dtype=torch.float64), requires_grad, dtype)


def linspace(self, start, end, steps, requires_grad=False, dtype=None):
    return _new(self, torch.linspace(float(start), float(end), int(steps), dtype=torch.float64), requires_grad, dtype)


def logspace(self, start, end, steps, base=10.0, requires_grad=False, dtype=None):
    return _new(self, torch.logspace(float(start), float(end), int(steps), base=float(base), dtype=torch.float64),
                requires_grad, dtype)


def _window(fn):
    def w(self, n, periodic=True, **kw):
        return _new(self, fn(int(n), periodic=periodic, dtype=torch.float64, **kw))
    return w


hann_window = _window(torch.hann_window)
hamming_window = _window(torch.hamming_window)
blackman_window = _window(torch.blackman_window)
bartlett_window = _window(torch.bartlett_window)


def kaiser_window(self, n, periodic=True, beta=12.0):
    return _new(self, torch.kaiser_window(int(n), periodic=periodic, beta=beta, dtype=torch.float64))


# ------------------------------------------------------------------------------------ random
def manual_seed(self, seed: int) -> None:
    self.rng.seed(seed)


def rng_state(self) -> List[int]:
    return self.rng.get_state()


def set_rng_state(self, st: Sequence[int]) -> None:
    self.rng.set_state(st)


def rand(self, shape, requires_grad=False, dtype=None):
    return _new(self, self.rng.uniform(_numel(shape)).reshape(tuple(shape)), requires_grad, dtype)


def randn(self, shape, requires_grad=False, dtype=None):
    return _new(self, self.rng.normal(_numel(shape)).reshape(tuple(shape)), requires_grad, dtype)


def rand_like(self, nid, requires_grad=False):
    return rand(self, self.tensor_shape(nid), requires_grad, self.tensor_dtype(nid))


def randn_like(self, nid, requires_grad=False):
    return randn(self, self.tensor_shape(nid), requires_grad, self.tensor_dtype(nid))


def randint(self, low, high, shape, dtype=None):
    if high <= low:
        raise ValueError("randint needs high > low")
    u = self.rng.uniform(_numel(shape))
    return _new(self, (low + torch.floor(u * (high - low))).reshape(tuple(shape)), False, dtype)


def randperm(self, n, dtype=None):
    perm = list(range(n))
    u = self.rng.uniform(max(n - 1, 0)).tolist()
    for k, i in enumerate(range(n - 1, 0, -1)):
        j = int(u[k] * (i + 1))
        perm[i], perm[j] = perm[j], perm[i]
    return _new(self, torch.tensor(perm, dtype=torch.float64), False, dtype)


def _normal_cos(self, n: int) -> torch.Tensor:
    """Initialiser normals: cosine branch of Box-Muller, two uniforms per value."""
    u = self.rng.uniform(2 * n).reshape(n, 2) if n else torch.empty(0, 2, dtype=torch.float64)
    u1 = u[:, 0].clamp_min(1e-300)
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u[:, 1])


def bernoulli(self, probs_id):
    p = self.tensor(probs_id).detach().to("cpu", torch.float64)
    u = self.rng.uniform(p.numel()).reshape(p.shape)
    return _new(self, (u < p).to(torch.float64), False, self.tensor_dtype(probs_id))


def bernoulli_p(self, shape, p: float, dtype=None):
    u = self.rng.uniform(_numel(shape)).reshape(tuple(shape))
    return _new(self, (u < p).to(torch.float64), False, dtype)


def multinomial(self, weights_id, num_samples: int, replacement: bool = False):
    w = self.tensor(weights_id).detach().to("cpu", torch.float64)
    rows = w.reshape(-1, w.shape[-1]).clone()
    if (rows < 0).any() or not torch.isfinite(rows).all():
        raise ValueError("multinomial weights must be finite and non-negative")
    if not replacement and num_samples > int((rows > 0).sum(-1).min()):
        raise ValueError("multinomial without replacement needs enough non-zero weights")
    out = torch.zeros(rows.shape[0], num_samples, dtype=torch.float64)
    for r in range(rows.shape[0]):
        wr = rows[r]
        total = float(wr.sum())
        for k in range(num_samples):
            x = float(self.rng.uniform(1)[0]) * total
            acc, pick = 0.0, -1
            for idx in range(wr.numel()):
                acc += float(wr[idx])
                if float(wr[idx]) > 0 and x < acc:
                    pick = idx
                    break
            if pick < 0:   # ran off the end: last index that still has weight
                pick = int(torch.nonzero(wr > 0)[-1])
            out[r, k] = pick
            if not replacement:
                wr[pick] = 0.0
    return _new(self, out.reshape(*w.shape[:-1], num_samples), False)


def poisson(self, rates_id):
    lam = self.tensor(rates_id).detach().to("cpu", torch.float64).reshape(-1)
    out = torch.zeros_like(lam)
    for i, l in enumerate(lam.tolist()):
        u = float(self.rng.uniform(1)[0])
        p = math.exp(-l)
        s, x = p, 0
        while u > s and x < 10000:   # inversion by sequential search
            x += 1
            p *= l / x
            s += p
        out[i] = x
    return _new(self, out.reshape(self.tensor_shape(rates_id)), False)


def tensor_normal_(self, nid, mean=0.0, std=1.0):
    t = self.tensor(nid)
    t.copy_((mean + std * _normal_cos(self, t.numel())).reshape(t.shape).to(t.dtype))
    self.tensor_tape.bump_version(nid)
    return nid


def tensor_uniform_(self, nid, a=0.0, b=1.0):
    t = self.tensor(nid)
    t.copy_((a + (b - a) * self.rng.uniform(t.numel())).reshape(t.shape).to(t.dtype))
    self.tensor_tape.bump_version(nid)
    return nid


def functional_dropout(self, nid, p=0.5, training=True):
    """mask = rand > p, scaled by 1/(1-p) (ft-nn/src/lib.rs:2357-2373)."""
    if not training or p == 0.0:
        return nid
    if not (0.0 <= p < 1.0):
        raise ValueError("dropout p must be in [0, 1)")
    x = self.tensor(nid)
    if self.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
        # GPU backend: counter-based Philox mask (seed = the session seed, offset = elements drawn so far),
        # regenerated by the backward pass instead of being stored
        from .ops import fused as F
        off = self._dropout_calls
        self._dropout_calls += x.numel()
        rg = self.tensor_tape.grad_enabled and self.tensor_tape.nodes[nid].requires_grad
        self._record_dispatch("dropout", rg, launched="ftk::dropout_kernel<philox>")
        return F.dropout(self.tensor_tape, nid, float(p), int(self._seed), off)
    mask = (self.rng.uniform(self.tensor_numel(nid)).reshape(self.tensor_shape(nid)) > p).to(torch.float64) / (1.0 - p)
    m = _new(self, mask, False, self.tensor_dtype(nid))
    return self.tensor_mul(nid, m)


# ------------------------------------------------------------------------------------ comparisons / predicates
def _cmp(fn):
    def c(self, a, b):
        x, y = self.tensor(a), self.tensor(b)
        return _new(self, fn(x, y).to(torch.float64), False, self.tensor_dtype(a))
    return c


tensor_eq, tensor_ne = _cmp(torch.eq), _cmp(torch.ne)
tensor_lt, tensor_gt = _cmp(torch.lt), _cmp(torch.gt)
tensor_le, tensor_ge = _cmp(torch.le), _cmp(torch.ge)


def tensor_allclose(self, a, b, rtol=1e-5, atol=1e-8, equal_nan=False) -> bool:
    x, y = self.tensor(a), self.tensor(b)
    if x.shape != y.shape:
        return False
    return bool(torch.allclose(x, y, rtol=rtol, atol=atol, equal_nan=equal_nan))


def tensor_equal(self, a, b) -> bool:
    return bool(torch.equal(self.tensor(a), self.tensor(b)))


def tensor_isnan(self, a):
    return _new(self, torch.isnan(self.tensor(a)).to(torch.float64), False)


def tensor_isfinite(self, a):
    return _new(self, torch.isfinite(self.tensor(a)).to(torch.float64), False)


def tensor_argmax(self, a, dim=None):
    return _new(self, torch.argmax(self.tensor(a), dim).to(torch.float64), False)


def tensor_argmin(self, a, dim=None):
    return _new(self, torch.argmin(self.tensor(a), dim).to(torch.float64), False)


def tensor_argsort(self, a, dim=-1, descending=False):
    return _new(self, torch.argsort(self.tensor(a), dim=dim, descending=descending, stable=True).to(torch.float64), False)


def tensor_sort_with_indices(self, a, dim=-1, descending=False):
    vals = self.tensor_sort(a, dim=dim, descending=descending)
    return vals, tensor_argsort(self, a, dim, descending)


def tensor_topk_with_indices(self, a, k, dim=-1, largest=True):
    vals = self.tensor_topk(a, k=k, dim=dim, largest=largest)
    idx = torch.topk(self.tensor(a), k, dim=dim, largest=largest, sorted=True).indices
    return vals, _new(self, idx.to(torch.float64), False)


def tensor_searchsorted(self, sorted_seq, values, right=False):
    return _new(self, torch.searchsorted(self.tensor(sorted_seq), self.tensor(values), right=right).to(torch.float64), False)


def tensor_nonzero(self, a):
    return _new(self, torch.nonzero(self.tensor(a)).to(torch.float64), False)


def tensor_max(self, a, b=None):
    """``tensor_max(a, b)``: elementwise maximum; ``tensor_max(a)``: maximum over all elements."""
    if b is not None:
        return self._apply("max", [a, b])
    return self.tensor_max_dim(self.tensor_reshape(a, shape=(-1,)), dim=0)


def tensor_min(self, a, b=None):
    if b is not None:
        return self._apply("min", [a, b])
    return self.tensor_min_dim(self.tensor_reshape(a, shape=(-1,)), dim=0)


def tensor_prod(self, a):
    return self.tensor_prod_dim(self.tensor_reshape(a, shape=(-1,)), dim=0)


def tensor_var(self, a, correction=1):
    return self.tensor_var_dim(self.tensor_reshape(a, shape=(-1,)), dim=0, correction=correction)


def tensor_std(self, a, correction=1):
    return self.tensor_std_dim(self.tensor_reshape(a, shape=(-1,)), dim=0, correction=correction)


def tensor_mode(self, a, dim=-1):
    v = torch.mode(self.tensor(a), dim)
    return _new(self, v.values.to(torch.float64), False), _new(self, v.indices.to(torch.float64), False)


# ------------------------------------------------------------------------------------ dtype / layout / multi-output shape ops
def tensor_to_dtype(self, a, dtype: DType):
    name = {DType.F32: "cast_f32", DType.F64: "cast_f64", DType.F16: "cast_f16", DType.BF16: "cast_bf16"}.get(dtype)
    if name is None:
        return self.tensor_tape.leaf(self.tensor(a).to(dtype.to_torch()), False)
    return self._apply(name, [a])


def tensor_to_f32(self, a):
    return tensor_to_dtype(self, a, DType.F32)


def tensor_to_f64(self, a):
    return tensor_to_dtype(self, a, DType.F64)


def tensor_contiguous(self, a):
    """A dense row-major copy when ``a`` is a strided view, ``a`` itself otherwise."""
    if self.tensor(a).is_contiguous():
        return a
    return self._apply("contiguous", [a])


def tensor_split(self, a, split_size, dim=0):
    n = self.tensor_shape(a)[dim]
    return [self.tensor_narrow(a, dim=dim, start=s, length=min(split_size, n - s)) for s in range(0, n, split_size)]


def tensor_chunk(self, a, chunks, dim=0):
    n = self.tensor_shape(a)[dim]
    return tensor_split(self, a, (n + chunks - 1) // chunks, dim)


def tensor_unbind(self, a, dim=0):
    return [self.tensor_squeeze(self.tensor_narrow(a, dim=dim, start=i, length=1), dim=dim)
            for i in range(self.tensor_shape(a)[dim])]


def tensor_hstack(self, ids):
    return self.tensor_cat(ids, dim=0 if len(self.tensor_shape(ids[0])) == 1 else 1)


def tensor_vstack(self, ids):
    ids = [self.tensor_unsqueeze(i, dim=0) if len(self.tensor_shape(i)) == 1 else i for i in ids]
    return self.tensor_cat(ids, dim=0)


def tensor_dstack(self, ids):
    out = []
    for i in ids:
        while len(self.tensor_shape(i)) < 3:
            i = self.tensor_unsqueeze(i, dim=len(self.tensor_shape(i)) if len(self.tensor_shape(i)) == 2 else 0)
        out.append(i)
    return self.tensor_cat(out, dim=2)


def tensor_tile(self, a, reps):
    return self.tensor_repeat(a, repeats=tuple(reps))


def tensor_unflatten(self, a, dim, sizes):
    shp = self.tensor_shape(a)
    return self.tensor_reshape(a, shape=tuple(shp[:dim]) + tuple(sizes) + tuple(shp[dim + 1:]))


def tensor_fftfreq(self, n, d=1.0):
    return _new(self, torch.fft.fftfreq(n, d, dtype=torch.float64))


def tensor_rfftfreq(self, n, d=1.0):
    return _new(self, torch.fft.rfftfreq(n, d, dtype=torch.float64))


def tensor_fftshift(self, a):
    return _new(self, torch.fft.fftshift(self.tensor(a)))


def tensor_ifftshift(self, a):
    return _new(self, torch.fft.ifftshift(self.tensor(a)))


# ------------------------------------------------------------------------------------ initialisers (ft-nn/src/lib.rs:19629-19984)
def calculate_gain(self, nonlinearity: str, param: Optional[float] = None) -> float:
    return torch.nn.init.calculate_gain(nonlinearity, param)


def _fans(shape):
    if len(shape) < 2:
        raise ValueError("fan in/out need at least 2 dimensions")
    rf = 1
    for s in shape[2:]:
        rf *= s
    return shape[1] * rf, shape[0] * rf


def _fill(self, nid, values: torch.Tensor):
    t = self.tensor(nid)
    t.copy_(values.reshape(t.shape).to(t.dtype))
    self.tensor_tape.bump_version(nid)
    return nid


def init_constant_(self, nid, val):
    return _fill(self, nid, torch.full((self.tensor_numel(nid),), float(val), dtype=torch.float64))


def init_zeros_(self, nid):
    return init_constant_(self, nid, 0.0)


def init_ones_(self, nid):
    return init_constant_(self, nid, 1.0)


def init_uniform_(self, nid, a=0.0, b=1.0):
    return tensor_uniform_(self, nid, a, b)


def init_normal_(self, nid, mean=0.0, std=1.0):
    return tensor_normal_(self, nid, mean, std)


def init_trunc_normal_(self, nid, mean=0.0, std=1.0, a=-2.0, b=2.0):
    n = self.tensor_numel(nid)
    out, filled = torch.empty(n, dtype=torch.float64), 0
    while filled < n:   # rejection sampling on the session stream
        z = mean + std * _normal_cos(self, n - filled)
        z = z[(z >= a) & (z <= b)]
        out[filled: filled + z.numel()] = z
        filled += z.numel()
    return _fill(self, nid, out)


def init_eye_(self, nid):
    shp = self.tensor_shape(nid)
    return _fill(self, nid, torch.eye(shp[0], shp[1], dtype=torch.float64))


def init_dirac_(self, nid, groups=1):
    t = torch.zeros(self.tensor_shape(nid), dtype=torch.float64)
    torch.nn.init.dirac_(t, groups)
    return _fill(self, nid, t)


def init_xavier_uniform_(self, nid, gain=1.0):
    fi, fo = _fans(self.tensor_shape(nid))
    bound = gain * math.sqrt(6.0 / (fi + fo))
    return tensor_uniform_(self, nid, -bound, bound)


def init_xavier_normal_(self, nid, gain=1.0):
    fi, fo = _fans(self.tensor_shape(nid))
    return tensor_normal_(self, nid, 0.0, gain * math.sqrt(2.0 / (fi + fo)))


def init_kaiming_uniform_(self, nid, a=0.0, mode="fan_in", nonlinearity="leaky_relu"):
    fi, fo = _fans(self.tensor_shape(nid))
    fan = fi if mode == "fan_in" else fo
    bound = torch.nn.init.calculate_gain(nonlinearity, a) * math.sqrt(3.0 / fan)
    return tensor_uniform_(self, nid, -bound, bound)


def init_kaiming_normal_(self, nid, a=0.0, mode="fan_in", nonlinearity="leaky_relu"):
    fi, fo = _fans(self.tensor_shape(nid))
    fan = fi if mode == "fan_in" else fo
    return tensor_normal_(self, nid, 0.0, torch.nn.init.calculate_gain(nonlinearity, a) / math.sqrt(fan))


def init_orthogonal_(self, nid, gain=1.0):
    shp = self.tensor_shape(nid)
    rows, cols = shp[0], self.tensor_numel(nid) // shp[0]
    flat = _normal_cos(self, rows * cols).reshape(rows, cols)
    if rows < cols:
        flat = flat.t()
    q, r = torch.linalg.qr(flat)
    q = q * torch.sign(torch.diagonal(r))
    if rows < cols:
        q = q.t()
    return _fill(self, nid, gain * q)


def init_sparse_(self, nid, sparsity, std=0.01):
    shp = self.tensor_shape(nid)
    if len(shp) != 2:
        raise ValueError("sparse_ needs a 2-D tensor")
    rows, cols = shp
    t = (std * _normal_cos(self, rows * cols)).reshape(rows, cols)
    nz = int(math.ceil(sparsity * rows))
    for c in range(cols):
        perm = self.tensor_values(randperm(self, rows))
        for r in perm[:nz]:
            t[int(r), c] = 0.0
    return _fill(self, nid, t)


def install(cls) -> None:
    g = globals()
    skip = {"install", "math", "torch", "DType", "List", "Optional", "Sequence"}
    for name, fn in list(g.items()):
        if callable(fn) and not name.startswith("_") and name not in skip:
            setattr(cls, name, fn)
