"""VJP rules of the tensor tape (CPU / reference path and the long tail of operators).

Every operator is an :class:`OpDef`: a forward function on ``torch.Tensor`` values, the
backward rule and the rule string that appears in ``TensorBackwardStep.rule`` (kept verbatim
from the reference, ft-autograd/src/lib.rs:11807-15602, so step logs diff cleanly).

Hot-path operators of the sm_100a backend live in :mod:`frankentorch_b200.ops.fused`; the
rules here are formula-level restatements executed with PyTorch tensor arithmetic in the
gradient dtype of the tape (f64 on the CPU path).  Operators whose local derivative has no
closed form worth spelling out (linalg, FFT, interpolation ...) use ``local_vjp``: the forward
is re-run on detached inputs and PyTorch differentiates that ONE node; ordering and
accumulation across nodes still belong to the deterministic tape.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch


@dataclass
class OpDef:
    name: str
    fwd: Callable[..., torch.Tensor]
    vjp: Optional[Callable[..., Sequence[Optional[torch.Tensor]]]]   # (g, inputs, out, kw) -> grads
    rule: str


OPS: Dict[str, OpDef] = {}


def _reg(name: str, fwd, vjp, rule: str) -> None:
    OPS[name] = OpDef(name, fwd, vjp, rule)


def unbroadcast(g: torch.Tensor, shape) -> torch.Tensor:
    """Sum ``g`` over the dimensions that broadcasting expanded (``sum_broadcast_dims``)."""
    shape = tuple(shape)
    if tuple(g.shape) == shape:
        return g
    while g.dim() > len(shape):
        g = g.sum(0)
    for i, s in enumerate(shape):
        if s == 1 and g.shape[i] != 1:
            g = g.sum(i, keepdim=True)
    return g


def local_vjp(fwd):
    """VJP of one node by differentiating a re-run of its forward on detached inputs."""
    def vjp(g, inputs, out, kw):
        # Inside a graph-building backward the rule is itself being differentiated: its arguments carry
        # torch's grad tracking and the result must stay connected to them (see double_backward.py).
        higher = torch.is_grad_enabled() and (g.requires_grad or any(
            isinstance(x, torch.Tensor) and x.requires_grad for x in inputs))
        if higher:
            xs = [x if (x.requires_grad or not (x.is_floating_point() or x.is_complex()))
                  else x.detach().requires_grad_(True) for x in inputs]
        else:
            xs = [x.detach().clone().requires_grad_(x.is_floating_point() or x.is_complex()) for x in inputs]
        with torch.enable_grad():
            y = fwd(*xs, **kw)
            need = [x for x in xs if x.requires_grad]
            grads = torch.autograd.grad(y, need, g.to(y.dtype), allow_unused=True, create_graph=higher) if need else ()
        it = iter(grads)
        return [next(it) if x.requires_grad else None for x in xs]
    return vjp


# ---------------------------------------------------------------------------------- binary
def _bin(name, fwd, da, db, rule):
    def vjp(g, inputs, out, kw):
        a, b = inputs
        return [unbroadcast(da(g, a, b, out), a.shape), unbroadcast(db(g, a, b, out), b.shape)]
    _reg(name, fwd, vjp, rule)


_bin("add", lambda a, b: a + b, lambda g, a, b, o: g, lambda g, a, b, o: g, "d(a+b)/da=1; d(a+b)/db=1")
_bin("sub", lambda a, b: a - b, lambda g, a, b, o: g, lambda g, a, b, o: -g, "d(a-b)/da=1; d(a-b)/db=-1")
_bin("mul", lambda a, b: a * b, lambda g, a, b, o: g * b, lambda g, a, b, o: g * a, "d(a*b)/da=b; d(a*b)/db=a")
_bin("div", lambda a, b: a / b, lambda g, a, b, o: g / b, lambda g, a, b, o: -g * a / (b * b),
     "d(a/b)/da=1/b; d(a/b)/db=-(a/b^2)")


def _tie(a, b, cmp):
    # ties split the gradient 0.5 / 0.5 (reference semantics for min/max)
    return torch.where(cmp(a, b), torch.ones_like(a), torch.where(a == b, torch.full_like(a, 0.5), torch.zeros_like(a)))


_bin("max", torch.maximum, lambda g, a, b, o: g * _tie(*torch.broadcast_tensors(a, b), torch.gt),
     lambda g, a, b, o: g * _tie(*torch.broadcast_tensors(b, a), torch.gt),
     "d(max(a,b))/da=1(a>b) or 0.5(a=b); db=1(b>a) or 0.5(a=b)")
_bin("min", torch.minimum, lambda g, a, b, o: g * _tie(*torch.broadcast_tensors(a, b), torch.lt),
     lambda g, a, b, o: g * _tie(*torch.broadcast_tensors(b, a), torch.lt),
     "d(min(a,b))/da=1(a<b) or 0.5(a=b); db=1(b<a) or 0.5(a=b)")
_bin("atan2", torch.atan2, lambda g, a, b, o: g * b / (a * a + b * b), lambda g, a, b, o: -g * a / (a * a + b * b),
     "d(atan2(a,b))/da=b/(a^2+b^2); db=-a/(a^2+b^2)")
_bin("fmod", torch.fmod, lambda g, a, b, o: g, lambda g, a, b, o: -g * torch.trunc(a / b),
     "d(fmod(a,b))/da=1; db=-trunc(a/b)")
_bin("remainder", torch.remainder, lambda g, a, b, o: g, lambda g, a, b, o: -g * torch.floor(a / b),
     "d(remainder(a,b))/da=1; db=-floor(a/b)")
_bin("pow_tensor", torch.pow, lambda g, a, b, o: g * b * torch.pow(a, b - 1),
     lambda g, a, b, o: g * o * torch.log(a), "d(a^b)/da=b*a^(b-1); d(a^b)/db=a^b*ln(a)")

_reg("matmul", torch.matmul,
     lambda g, i, o, kw: _matmul_vjp(g, i[0], i[1]), "d(A@B)/dA=dOut@B^T; d(A@B)/dB=A^T@dOut")
_reg("bmm", torch.bmm, lambda g, i, o, kw: [g @ i[1].transpose(-1, -2), i[0].transpose(-1, -2) @ g],
     "d(bmm(A,B))/dA=dOut@B^T; d(bmm(A,B))/dB=A^T@dOut (batched)")
_reg("dot", torch.dot, lambda g, i, o, kw: [g * i[1], g * i[0]],
     "d(dot(a,b))/da=grad_out*b; d(dot(a,b))/db=grad_out*a")
_reg("outer", torch.outer, lambda g, i, o, kw: [g @ i[1], g.t() @ i[0]],
     "d(outer(a,b))/da=dOut@b; d(outer(a,b))/db=dOut^T@a")


def _matmul_vjp(g, a, b):
    if a.dim() == 1 and b.dim() == 1:
        return [g * b, g * a]
    if a.dim() == 1:
        return [(g.unsqueeze(-2) @ b.transpose(-1, -2)).squeeze(-2).reshape(a.shape) if b.dim() == 2
                else unbroadcast((g.unsqueeze(-2) @ b.transpose(-1, -2)).squeeze(-2), a.shape),
                unbroadcast(a.unsqueeze(-1) * g.unsqueeze(-2), b.shape)]
    if b.dim() == 1:
        return [g.unsqueeze(-1) * b, unbroadcast((a.transpose(-1, -2) @ g.unsqueeze(-1)).squeeze(-1), b.shape)]
    return [unbroadcast(g @ b.transpose(-1, -2), a.shape), unbroadcast(a.transpose(-1, -2) @ g, b.shape)]


_reg("addmm", lambda inp, m1, m2, beta=1.0, alpha=1.0: torch.addmm(inp, m1, m2, beta=beta, alpha=alpha),
     lambda g, i, o, kw: [unbroadcast(g * kw.get("beta", 1.0), i[0].shape), kw.get("alpha", 1.0) * g @ i[2].t(),
                          kw.get("alpha", 1.0) * i[1].t() @ g],
     "d(addmm)/d_input=beta*grad, d/d_mat1=alpha*grad@mat2^T, d/d_mat2=alpha*mat1^T@grad")
_reg("addmv", lambda inp, m, v, beta=1.0, alpha=1.0: torch.addmv(inp, m, v, beta=beta, alpha=alpha),
     lambda g, i, o, kw: [unbroadcast(g * kw.get("beta", 1.0), i[0].shape), kw.get("alpha", 1.0) * torch.outer(g, i[2]),
                          kw.get("alpha", 1.0) * i[1].t() @ g],
     "d(addmv)/d_input=beta*grad, d/d_mat=alpha*outer(grad,vec), d/d_vec=alpha*mat^T@grad")
_reg("lerp", lambda s, e, w=0.5: torch.lerp(s, e, w),
     lambda g, i, o, kw: [(1 - kw.get("w", 0.5)) * g, kw.get("w", 0.5) * g],
     "d(lerp(s,e,w))/ds=(1-w)*grad, d/de=w*grad")


# ---------------------------------------------------------------------------------- unary
def _un(name, fwd, d, rule):
    _reg(name, fwd, lambda g, i, o, kw: [d(g, i[0], o)], rule)


_SQ2PI = math.sqrt(2.0 / math.pi)
_un("neg", torch.neg, lambda g, x, y: -g, "d(-x)/dx=-1")
_un("abs", torch.abs, lambda g, x, y: g * torch.sign(x), "d|x|/dx=sign(x)")
_un("exp", torch.exp, lambda g, x, y: g * y, "d(exp(x))/dx=exp(x)")
_un("log", torch.log, lambda g, x, y: g / x, "d(ln(x))/dx=1/x")
_un("log2", torch.log2, lambda g, x, y: g / (x * math.log(2.0)), "d(log2(x))/dx=1/(x*ln2)")
_un("log10", torch.log10, lambda g, x, y: g / (x * math.log(10.0)), "d(log10(x))/dx=1/(x*ln10)")
_un("log1p", torch.log1p, lambda g, x, y: g / (1 + x), "d(log1p(x))/dx=1/(1+x)")
_un("expm1", torch.expm1, lambda g, x, y: g * (y + 1), "d(expm1(x))/dx=exp(x)")
_un("relu", torch.relu, lambda g, x, y: g * (x > 0), "d(relu(x))/dx=1 if x>0 else 0")
_un("sigmoid", torch.sigmoid, lambda g, x, y: g * y * (1 - y), "d(sigmoid(x))/dx=sigmoid(x)*(1-sigmoid(x))")
_un("tanh", torch.tanh, lambda g, x, y: g * (1 - y * y), "d(tanh(x))/dx=1-tanh(x)^2")
_un("sin", torch.sin, lambda g, x, y: g * torch.cos(x), "d(sin(x))/dx=cos(x)")
_un("cos", torch.cos, lambda g, x, y: -g * torch.sin(x), "d(cos(x))/dx=-sin(x)")
_un("tan", torch.tan, lambda g, x, y: g * (1 + y * y), "d(tan(x))/dx=1+tan(x)^2")
_un("asin", torch.asin, lambda g, x, y: g / torch.sqrt(1 - x * x), "d(asin(x))/dx=1/sqrt(1-x^2)")
_un("acos", torch.acos, lambda g, x, y: -g / torch.sqrt(1 - x * x), "d(acos(x))/dx=-1/sqrt(1-x^2)")
_un("atan", torch.atan, lambda g, x, y: g / (1 + x * x), "d(atan(x))/dx=1/(1+x^2)")
_un("sinh", torch.sinh, lambda g, x, y: g * torch.cosh(x), "d(sinh(x))/dx=cosh(x)")
_un("cosh", torch.cosh, lambda g, x, y: g * torch.sinh(x), "d(cosh(x))/dx=sinh(x)")
_un("sqrt", torch.sqrt, lambda g, x, y: g * 0.5 / y, "d(sqrt(x))/dx=0.5/sqrt(x)")
_un("rsqrt", torch.rsqrt, lambda g, x, y: -0.5 * g * y * y * y, "d(rsqrt(x))/dx=-0.5*rsqrt(x)^3")
_un("square", torch.square, lambda g, x, y: 2 * g * x, "d(x^2)/dx=2x")
_un("reciprocal", torch.reciprocal, lambda g, x, y: -g * y * y, "d(1/x)/dx=-1/x^2")
for _n, _f in (("floor", torch.floor), ("ceil", torch.ceil), ("round", torch.round), ("trunc", torch.trunc),
               ("sign", torch.sign)):
    _un(_n, _f, lambda g, x, y: torch.zeros_like(g), "d(floor|ceil|round)/dx=0")
_un("frac", torch.frac, lambda g, x, y: g, "d(frac(x))/dx=1")
_un("gelu", lambda x: torch.nn.functional.gelu(x),
    lambda g, x, y: g * (0.5 * (1 + torch.erf(x / math.sqrt(2.0))) + x * torch.exp(-0.5 * x * x) / math.sqrt(2 * math.pi)),
    "d(gelu(x))/dx")
_un("gelu_tanh", lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
    lambda g, x, y: g * _gelu_tanh_grad(x), "d(gelu_tanh(x))/dx")
_un("silu", torch.nn.functional.silu,
    lambda g, x, y: g * (torch.sigmoid(x) * (1 + x * (1 - torch.sigmoid(x)))),
    "d(silu(x))/dx=sigmoid(x)*(1+x*(1-sigmoid(x)))")
_un("softplus", torch.nn.functional.softplus, lambda g, x, y: g * torch.sigmoid(x), "d(softplus(x))/dx=sigmoid(x)")
_un("mish", torch.nn.functional.mish, None, "d(mish(x))/dx")
_un("erf", torch.erf, lambda g, x, y: g * 2 / math.sqrt(math.pi) * torch.exp(-x * x), "d(erf(x))/dx=2/sqrt(pi)*exp(-x^2)")


def _gelu_tanh_grad(x):
    u = _SQ2PI * (x + 0.044715 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * _SQ2PI * (1 + 3 * 0.044715 * x * x)


OPS["mish"] = OpDef("mish", torch.nn.functional.mish, local_vjp(torch.nn.functional.mish), "d(mish(x))/dx")

_reg("leaky_relu", lambda x, slope=0.01: torch.nn.functional.leaky_relu(x, slope),
     lambda g, i, o, kw: [g * torch.where(i[0] > 0, torch.ones_like(g), torch.full_like(g, kw.get("slope", 0.01)))],
     "d(leaky_relu(x))/dx=1 if x>0 else slope")
_reg("elu", lambda x, alpha=1.0: torch.nn.functional.elu(x, alpha),
     lambda g, i, o, kw: [g * torch.where(i[0] > 0, torch.ones_like(g), o + kw.get("alpha", 1.0))],
     "d(elu(x))/dx=1 if x>0 else alpha*exp(x)")
_reg("mul_scalar", lambda x, c=1.0: x * c, lambda g, i, o, kw: [g * kw.get("c", 1.0)], "d(a*c)/da=c")
_reg("add_scalar", lambda x, c=0.0: x + c, lambda g, i, o, kw: [g], "d(a+c)/da=1")
_reg("pow", lambda x, n=2.0: torch.pow(x, n),
     lambda g, i, o, kw: [g * kw.get("n", 2.0) * torch.pow(i[0], kw.get("n", 2.0) - 1)], "d(x^n)/dx=n*x^(n-1)")
_reg("clamp", lambda x, min=None, max=None: torch.clamp(x, min, max),
     lambda g, i, o, kw: [g * ((i[0] >= (kw.get("min") if kw.get("min") is not None else -math.inf))
                               & (i[0] <= (kw.get("max") if kw.get("max") is not None else math.inf)))],
     "d(clamp(x,min,max))/dx=1 if min<=x<=max else 0")
