"""Closed-form VJP rules of the pointwise, special-function, reduction and indexing operators that the
reference's session exposes beyond the core table (its per-operator benches and examples call them:
ft-api/benches/ops_bench.rs, special_bench.rs, ft-api/examples/*_h2h.rs, *_probe.rs).

Every rule here is written out as tensor arithmetic; none re-runs the forward under another autograd
engine.  Tie and boundary conventions follow PyTorch's derivative formulas: ``amax`` / ``amin`` split
the gradient evenly among equal extrema, ``fmax`` / ``fmin`` send it to the non-NaN operand,
``xlogy`` masks the first operand's gradient where it is zero, integer-valued and predicate operators
have no rule (their nodes never require a gradient).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from .functions import OPS, _bin as _bin_raw, _reg, _tie, _un, unbroadcast

_SQRT_PI = math.sqrt(math.pi)
_SQRT_2PI = math.sqrt(2.0 * math.pi)
_LN2 = math.log(2.0)
_LN10 = math.log(10.0)


def _bin(name, fwd, da, db, rule):
    # a Python-level signature lets the session count the tensor arguments (builtins expose none)
    _bin_raw(name, lambda a, b: fwd(a, b), da, db, rule)


def _alias(new: str, old: str) -> None:
    """Second name for an operator that already has a rule (``maximum`` is ``max`` of two tensors)."""
    o = OPS[old]
    _reg(new, o.fwd, o.vjp, o.rule)


def _nograd(name: str, fwd, rule: str = "no gradient (integer- or boolean-valued)") -> None:
    _reg(name, fwd, None, rule)


def _as_float(x: torch.Tensor) -> torch.Tensor:
    return x if x.is_floating_point() else x.to(torch.float64)


# ---------------------------------------------------------------------------------- unary, elementary
_un("acosh", torch.acosh, lambda g, x, y: g / torch.sqrt(x * x - 1), "d(acosh(x))/dx=1/sqrt(x^2-1)")
_un("asinh", torch.asinh, lambda g, x, y: g / torch.sqrt(x * x + 1), "d(asinh(x))/dx=1/sqrt(x^2+1)")
_un("atanh", torch.atanh, lambda g, x, y: g / (1 - x * x), "d(atanh(x))/dx=1/(1-x^2)")
_un("exp2", torch.exp2, lambda g, x, y: g * y * _LN2, "d(2^x)/dx=2^x*ln2")
_un("exp10", lambda x: torch.pow(10.0, x), lambda g, x, y: g * y * _LN10, "d(10^x)/dx=10^x*ln10")
_un("cbrt", lambda x: torch.sign(x) * torch.abs(x).pow(1.0 / 3.0), lambda g, x, y: g / (3 * y * y),
    "d(cbrt(x))/dx=1/(3*cbrt(x)^2)")
_un("deg2rad", torch.deg2rad, lambda g, x, y: g * (math.pi / 180.0), "d(deg2rad(x))/dx=pi/180")
_un("rad2deg", torch.rad2deg, lambda g, x, y: g * (180.0 / math.pi), "d(rad2deg(x))/dx=180/pi")
_un("absolute", torch.abs, lambda g, x, y: g * torch.sign(x), "d|x|/dx=sign(x)")
_un("fix", torch.trunc, lambda g, x, y: torch.zeros_like(g), "d(fix(x))/dx=0")
_un("sgn", torch.sgn, lambda g, x, y: torch.zeros_like(g), "d(sgn(x))/dx=0")
_un("angle", lambda x: torch.angle(x), lambda g, x, y: torch.zeros_like(g), "d(angle(x))/dx=0 for real x")
_un("entr", torch.special.entr, lambda g, x, y: -g * (torch.log(x) + 1), "d(-x*ln(x))/dx=-(ln(x)+1)")


def _sinc_d(x):
    px = math.pi * x
    safe = torch.where(x == 0, torch.ones_like(x), x)
    d = (torch.cos(px) * px - torch.sin(px)) / (math.pi * safe * safe)
    return torch.where(x == 0, torch.zeros_like(x), d)


_un("sinc", torch.sinc, lambda g, x, y: g * _sinc_d(x), "d(sinc(x))/dx=(cos(pi x)*pi x-sin(pi x))/(pi x^2); 0 at x=0")


def _logit_fwd(x, eps=None):
    return torch.logit(x, eps)


def _logit_vjp(g, i, o, kw):
    x, eps = i[0], kw.get("eps")
    d = 1.0 / (x * (1 - x))
    if eps is not None:   # the clamped region is flat
        d = torch.where((x < eps) | (x > 1 - eps), torch.zeros_like(x), d)
    return [g * d]


_reg("logit", _logit_fwd, _logit_vjp, "d(logit(x))/dx=1/(x*(1-x)); 0 outside [eps,1-eps]")


def _nan_to_num_fwd(x, nan=0.0, posinf=None, neginf=None):
    return torch.nan_to_num(x, nan=nan, posinf=posinf, neginf=neginf)


_reg("nan_to_num", _nan_to_num_fwd, lambda g, i, o, kw: [g * torch.isfinite(i[0])],
     "d(nan_to_num(x))/dx=1 where x is finite, else 0")
_reg("round_decimals", lambda x, decimals=0: torch.round(x, decimals=int(decimals)),
     lambda g, i, o, kw: [torch.zeros_like(g)], "d(round(x,decimals))/dx=0")
_reg("clamp_min", lambda x, min=0.0: torch.clamp_min(x, min), lambda g, i, o, kw: [g * (i[0] >= kw.get("min", 0.0))],
     "d(clamp_min(x,m))/dx=1(x>=m)")
_reg("clamp_max", lambda x, max=0.0: torch.clamp_max(x, max), lambda g, i, o, kw: [g * (i[0] <= kw.get("max", 0.0))],
     "d(clamp_max(x,m))/dx=1(x<=m)")
_reg("float_power", lambda x, exponent=2.0: torch.pow(_as_float(x), exponent),
     lambda g, i, o, kw: [g * kw.get("exponent", 2.0) * torch.pow(i[0], kw.get("exponent", 2.0) - 1)],
     "d(x^p)/dx=p*x^(p-1)")

# ---------------------------------------------------------------------------------- unary, error / gamma family
_un("erfc", torch.erfc, lambda g, x, y: -g * (2.0 / _SQRT_PI) * torch.exp(-x * x), "d(erfc(x))/dx=-2/sqrt(pi)*exp(-x^2)")
_un("erfinv", torch.erfinv, lambda g, x, y: g * (_SQRT_PI / 2.0) * torch.exp(y * y),
    "d(erfinv(x))/dx=sqrt(pi)/2*exp(erfinv(x)^2)")
_un("erfcx", torch.special.erfcx, lambda g, x, y: g * (2 * x * y - 2.0 / _SQRT_PI), "d(erfcx(x))/dx=2x*erfcx(x)-2/sqrt(pi)")
_un("digamma", torch.digamma, lambda g, x, y: g * torch.polygamma(1, x), "d(digamma(x))/dx=trigamma(x)")
_un("lgamma", torch.lgamma, lambda g, x, y: g * torch.digamma(x), "d(lgamma(x))/dx=digamma(x)")
_alias("gammaln", "lgamma")
_reg("polygamma", lambda x, n=1: torch.polygamma(int(n), x),
     lambda g, i, o, kw: [g * torch.polygamma(int(kw.get("n", 1)) + 1, i[0])], "d(polygamma(n,x))/dx=polygamma(n+1,x)")


def _mvlgamma_vjp(g, i, o, kw):
    x, p = i[0], int(kw.get("p", 1))
    return [g * sum(torch.digamma(x - 0.5 * j) for j in range(p))]


_reg("mvlgamma", lambda x, p=1: torch.mvlgamma(x, int(p)), _mvlgamma_vjp, "d(mvlgamma(x,p))/dx=sum_{j<p} digamma(x-j/2)")
_alias("multigammaln", "mvlgamma")
_un("ndtr", torch.special.ndtr, lambda g, x, y: g * torch.exp(-0.5 * x * x) / _SQRT_2PI, "d(ndtr(x))/dx=exp(-x^2/2)/sqrt(2pi)")
_un("log_ndtr", torch.special.log_ndtr, lambda g, x, y: g * torch.exp(-0.5 * x * x - y) / _SQRT_2PI,
    "d(log_ndtr(x))/dx=exp(-x^2/2)/(sqrt(2pi)*ndtr(x))")
_un("ndtri", torch.special.ndtri, lambda g, x, y: g * _SQRT_2PI * torch.exp(0.5 * y * y), "d(ndtri(p))/dp=sqrt(2pi)*exp(ndtri(p)^2/2)")
for _n in ("ndtr", "log_ndtr", "ndtri", "erfcx", "entr"):
    _alias("special_" + _n, _n)


# ---------------------------------------------------------------------------------- unary, Bessel family
def _over_x(num, x, at_zero):
    """``num / x`` with the limit value at ``x == 0``."""
    safe = torch.where(x == 0, torch.ones_like(x), x)
    return torch.where(x == 0, torch.full_like(x, at_zero), num / safe)


_S = torch.special
_un("i0", torch.i0, lambda g, x, y: g * _S.i1(x), "d(I0(x))/dx=I1(x)")
_un("i0e", _S.i0e, lambda g, x, y: g * (_S.i1e(x) - torch.sign(x) * y), "d(I0e(x))/dx=I1e(x)-sign(x)*I0e(x)")
_un("i1", _S.i1, lambda g, x, y: g * (torch.i0(x) - _over_x(y, x, 0.5)), "d(I1(x))/dx=I0(x)-I1(x)/x")
_un("i1e", _S.i1e, lambda g, x, y: g * (_S.i0e(x) - y * torch.sign(x) - _over_x(y, x, 0.5)),
    "d(I1e(x))/dx=I0e(x)-I1e(x)*(sign(x)+1/x)")
_un("special_bessel_j0", _S.bessel_j0, lambda g, x, y: -g * _S.bessel_j1(x), "d(J0(x))/dx=-J1(x)")
_un("special_bessel_j1", _S.bessel_j1, lambda g, x, y: g * (_S.bessel_j0(x) - _over_x(y, x, 0.5)), "d(J1(x))/dx=J0(x)-J1(x)/x")
_un("special_bessel_y0", _S.bessel_y0, lambda g, x, y: -g * _S.bessel_y1(x), "d(Y0(x))/dx=-Y1(x)")
_un("special_bessel_y1", _S.bessel_y1, lambda g, x, y: g * (_S.bessel_y0(x) - y / x), "d(Y1(x))/dx=Y0(x)-Y1(x)/x")
_un("special_modified_bessel_i0", _S.modified_bessel_i0, lambda g, x, y: g * _S.modified_bessel_i1(x), "d(I0(x))/dx=I1(x)")
_un("special_modified_bessel_i1", _S.modified_bessel_i1,
    lambda g, x, y: g * (_S.modified_bessel_i0(x) - _over_x(y, x, 0.5)), "d(I1(x))/dx=I0(x)-I1(x)/x")
_un("special_modified_bessel_k0", _S.modified_bessel_k0, lambda g, x, y: -g * _S.modified_bessel_k1(x), "d(K0(x))/dx=-K1(x)")
_un("special_modified_bessel_k1", _S.modified_bessel_k1,
    lambda g, x, y: -g * (_S.modified_bessel_k0(x) + y / x), "d(K1(x))/dx=-K0(x)-K1(x)/x")
_un("special_scaled_modified_bessel_k0", _S.scaled_modified_bessel_k0,
    lambda g, x, y: g * (y - _S.scaled_modified_bessel_k1(x)), "d(e^x K0(x))/dx=e^x(K0(x)-K1(x))")
_un("special_scaled_modified_bessel_k1", _S.scaled_modified_bessel_k1,
    lambda g, x, y: g * (y * (1 - 1 / x) - _S.scaled_modified_bessel_k0(x)), "d(e^x K1(x))/dx=e^x(K1(x)(1-1/x)-K0(x))")
_un("special_spherical_bessel_j0", _S.spherical_bessel_j0,
    lambda g, x, y: g * _over_x(torch.cos(x) - y, x, 0.0), "d(sin(x)/x)/dx=(cos(x)-sin(x)/x)/x")
for _n in ("i0e", "i1", "i1e"):
    _alias("special_" + _n, _n)
# Ai'(x) is not expressible in the functions at hand; as in PyTorch the node carries no backward rule.
_nograd("special_airy_ai", _S.airy_ai, "no gradient (Ai' not available)")


# ---------------------------------------------------------------------------------- orthogonal polynomials (integer degree)
def _poly(name, fn, dfn, rule):
    _reg(name, lambda x, n=0: fn(x, int(n)), lambda g, i, o, kw: [g * dfn(i[0], int(kw.get("n", 0)), o)], rule)


def _cheb_u(x, n):
    return _S.chebyshev_polynomial_u(x, n)


def _legendre_d(x, n, pn):
    if n == 0:
        return torch.zeros_like(x)
    pnm1 = _S.legendre_polynomial_p(x, n - 1)
    edge = x.abs() == 1
    den = torch.where(edge, torch.ones_like(x), x * x - 1)
    d = n * (x * pn - pnm1) / den
    return torch.where(edge, torch.sign(x) ** (n + 1) * (n * (n + 1) / 2.0), d)


_poly("special_chebyshev_polynomial_t", _S.chebyshev_polynomial_t,
      lambda x, n, o: n * _cheb_u(x, n - 1) if n > 0 else torch.zeros_like(x), "d(T_n(x))/dx=n*U_{n-1}(x)")
_poly("special_hermite_polynomial_h", _S.hermite_polynomial_h,
      lambda x, n, o: 2 * n * _S.hermite_polynomial_h(x, n - 1) if n > 0 else torch.zeros_like(x), "d(H_n(x))/dx=2n*H_{n-1}(x)")
_poly("special_hermite_polynomial_he", _S.hermite_polynomial_he,
      lambda x, n, o: n * _S.hermite_polynomial_he(x, n - 1) if n > 0 else torch.zeros_like(x), "d(He_n(x))/dx=n*He_{n-1}(x)")
_poly("special_laguerre_polynomial_l", _S.laguerre_polynomial_l,
      lambda x, n, o: -sum((_S.laguerre_polynomial_l(x, k) for k in range(n)), torch.zeros_like(x)),
      "d(L_n(x))/dx=-sum_{k<n} L_k(x)")
_poly("special_legendre_polynomial_p", _S.legendre_polynomial_p, _legendre_d,
      "d(P_n(x))/dx=n*(x*P_n(x)-P_{n-1}(x))/(x^2-1); (+-1)^(n+1)*n(n+1)/2 at x=+-1")

# ---------------------------------------------------------------------------------- binary, elementwise
_reg("maximum", lambda a, b: torch.maximum(a, b), OPS["max"].vjp, OPS["max"].rule)
_reg("minimum", lambda a, b: torch.minimum(a, b), OPS["min"].vjp, OPS["min"].rule)
_alias("true_divide", "div")


def _nan_aware(a, b, cmp):
    # the non-NaN operand wins; where both are numbers ties split as for max / min
    a, b = torch.broadcast_tensors(a, b)
    w = _tie(a, b, cmp)
    return torch.where(torch.isnan(b), torch.ones_like(a), torch.where(torch.isnan(a), torch.zeros_like(a), w))


_bin("fmax", torch.fmax, lambda g, a, b, o: g * _nan_aware(a, b, torch.gt), lambda g, a, b, o: g * _nan_aware(b, a, torch.gt),
     "d(fmax(a,b)): as max, a NaN operand receives 0 and the other 1")
_bin("fmin", torch.fmin, lambda g, a, b, o: g * _nan_aware(a, b, torch.lt), lambda g, a, b, o: g * _nan_aware(b, a, torch.lt),
     "d(fmin(a,b)): as min, a NaN operand receives 0 and the other 1")
_bin("hypot", torch.hypot, lambda g, a, b, o: g * a / o, lambda g, a, b, o: g * b / o,
     "d(hypot(a,b))/da=a/hypot; db=b/hypot")
_bin("logaddexp", torch.logaddexp, lambda g, a, b, o: g * torch.exp(a - o), lambda g, a, b, o: g * torch.exp(b - o),
     "d(logaddexp(a,b))/da=exp(a-out); db=exp(b-out)")
_bin("logaddexp2", torch.logaddexp2, lambda g, a, b, o: g * torch.exp2(a - o), lambda g, a, b, o: g * torch.exp2(b - o),
     "d(logaddexp2(a,b))/da=2^(a-out); db=2^(b-out)")
_bin("xlogy", torch.xlogy, lambda g, a, b, o: g * torch.where(a == 0, torch.zeros_like(o), torch.log(b) + 0 * a),
     lambda g, a, b, o: g * a / b, "d(x*ln(y))/dx=ln(y) (0 where x=0); dy=x/y")
_bin("xlog1py", torch.special.xlog1py, lambda g, a, b, o: g * torch.where(a == 0, torch.zeros_like(o), torch.log1p(b) + 0 * a),
     lambda g, a, b, o: g * a / (1 + b), "d(x*log1p(y))/dx=log1p(y) (0 where x=0); dy=x/(1+y)")
_bin("copysign", torch.copysign,
     lambda g, a, b, o: g * torch.where(a == 0, torch.zeros_like(o), o / torch.where(a == 0, torch.ones_like(a), a) + 0 * b),
     lambda g, a, b, o: torch.zeros_like(o) * g, "d(copysign(a,b))/da=copysign(a,b)/a (0 at a=0); db=0")
_bin("heaviside", torch.heaviside, lambda g, a, b, o: torch.zeros_like(o) * g, lambda g, a, b, o: torch.zeros_like(o) * g,
     "d(heaviside(a,v))=0 for both operands")
_bin("floor_divide", torch.floor_divide, lambda g, a, b, o: torch.zeros_like(o) * g, lambda g, a, b, o: torch.zeros_like(o) * g,
     "d(floor(a/b))=0 for both operands")
_bin("ldexp", lambda x, e: x * torch.exp2(_as_float(e)), lambda g, a, b, o: g * torch.exp2(_as_float(b)),
     lambda g, a, b, o: g * o * _LN2, "d(x*2^e)/dx=2^e; de=x*2^e*ln2")
_bin("rel_entr", lambda x, y: torch.where(x > 0, x * (torch.log(x) - torch.log(y)), torch.where(x == 0, 0.0, math.inf) + 0 * (x + y)),
     lambda g, a, b, o: g * torch.where(a > 0, torch.log(a / b) + 1, torch.zeros_like(o)),
     lambda g, a, b, o: g * torch.where(a > 0, -a / b, torch.zeros_like(o)), "d(x*ln(x/y))/dx=ln(x/y)+1; dy=-x/y (x>0)")
_bin("zeta", torch.special.zeta, lambda g, a, b, o: torch.zeros_like(o) * g,
     lambda g, a, b, o: -g * a * torch.special.zeta(a + 1, b), "d(zeta(s,q))/dq=-s*zeta(s+1,q); ds not defined (0)")
_alias("special_zeta", "zeta")


def _igamma_dx(a, x):
    return torch.exp(-x + (a - 1) * torch.log(x) - torch.lgamma(a))


_bin("igamma", torch.special.gammainc, lambda g, a, b, o: torch.zeros_like(o) * g, lambda g, a, b, o: g * _igamma_dx(a, b),
     "d(P(a,x))/dx=exp(-x)*x^(a-1)/Gamma(a); da not defined (0)")
_bin("igammac", torch.special.gammaincc, lambda g, a, b, o: torch.zeros_like(o) * g, lambda g, a, b, o: -g * _igamma_dx(a, b),
     "d(Q(a,x))/dx=-exp(-x)*x^(a-1)/Gamma(a); da not defined (0)")
_alias("special_gammainc", "igamma")
_alias("special_gammaincc", "igammac")
_reg("vdot", lambda a, b: torch.dot(a, b), lambda g, i, o, kw: [g * i[1], g * i[0]], "d(vdot(a,b))/da=grad*b; db=grad*a (real)")


def _polar_vjp(g, i, o, kw):
    r, th = i
    gr, gi = g[..., 0], g[..., 1]       # complex values travel as [..., 2] (re, im)
    c, s = torch.cos(th), torch.sin(th)
    return [unbroadcast(gr * c + gi * s, r.shape), unbroadcast(r * (gi * c - gr * s), th.shape)]


_reg("polar", lambda r, theta: torch.stack([r * torch.cos(theta), r * torch.sin(theta)], -1), _polar_vjp,
     "d(r*e^{i t})/dr=g_re*cos(t)+g_im*sin(t); dt=r*(g_im*cos(t)-g_re*sin(t))")

for _n, _f in (("nextafter", lambda a, b: torch.nextafter(a, b)), ("gcd", lambda a, b: torch.gcd(a.long(), b.long())),
               ("lcm", lambda a, b: torch.lcm(a.long(), b.long())), ("logical_and", lambda a, b: torch.logical_and(a, b)),
               ("logical_or", lambda a, b: torch.logical_or(a, b)), ("logical_xor", lambda a, b: torch.logical_xor(a, b)),
               ("bitwise_and", lambda a, b: torch.bitwise_and(_bits(a), _bits(b))),
               ("bitwise_or", lambda a, b: torch.bitwise_or(_bits(a), _bits(b))),
               ("bitwise_xor", lambda a, b: torch.bitwise_xor(_bits(a), _bits(b))),
               ("isin", lambda e, t: torch.isin(e, t))):
    _nograd(_n, _f)
for _n, _f in (("logical_not", torch.logical_not), ("bitwise_not", lambda a: torch.bitwise_not(_bits(a))),
               ("signbit", torch.signbit), ("isinf", torch.isinf), ("isposinf", torch.isposinf),
               ("isneginf", torch.isneginf), ("count_nonzero", lambda x: torch.count_nonzero(x))):
    _nograd(_n, _f)
_nograd("isclose", lambda a, b, rtol=1e-5, atol=1e-8, equal_nan=False: torch.isclose(a, b, rtol, atol, equal_nan))
_nograd("one_hot", lambda idx, num_classes=-1: torch.nn.functional.one_hot(idx.long(), int(num_classes)))


def _bits(x):
    return x if not x.is_floating_point() else x.long()


# ---------------------------------------------------------------------------------- ternary
def _addc(name, fwd, d1, d2, rule):
    def vjp(g, i, o, kw):
        v = kw.get("value", 1.0)
        x, a, b = i
        return [unbroadcast(g, x.shape), unbroadcast(g * v * d1(a, b), a.shape), unbroadcast(g * v * d2(a, b), b.shape)]
    _reg(name, fwd, vjp, rule)


_addc("addcmul", lambda x, t1, t2, value=1.0: torch.addcmul(x, t1, t2, value=value), lambda a, b: b, lambda a, b: a,
      "d(x+v*a*b)/dx=1; da=v*b; db=v*a")
_addc("addcdiv", lambda x, t1, t2, value=1.0: torch.addcdiv(x, t1, t2, value=value), lambda a, b: 1 / b, lambda a, b: -a / (b * b),
      "d(x+v*a/b)/dx=1; da=v/b; db=-v*a/b^2")
_reg("addr", lambda x, v1, v2, beta=1.0, alpha=1.0: torch.addr(x, v1, v2, beta=beta, alpha=alpha),
     lambda g, i, o, kw: [unbroadcast(g * kw.get("beta", 1.0), i[0].shape), kw.get("alpha", 1.0) * (g @ i[2]),
                          kw.get("alpha", 1.0) * (g.t() @ i[1])],
     "d(beta*x+alpha*outer(a,b))/dx=beta*grad; da=alpha*grad@b; db=alpha*grad^T@a")
_reg("clamp_tensor", lambda x, lo, hi: torch.clamp(x, lo, hi),
     lambda g, i, o, kw: [unbroadcast(g * ((i[0] >= i[1]) & (i[0] <= i[2])), i[0].shape), unbroadcast(g * (i[0] < i[1]), i[1].shape),
                          unbroadcast(g * ((i[0] >= i[1]) & (i[0] > i[2])), i[2].shape)],
     "d(clamp(x,lo,hi))/dx=1(lo<=x<=hi); dlo=1(x<lo); dhi=1(x>hi)")
_reg("lerp_weighted", lambda s, e, w: torch.lerp(s, e, w),
     lambda g, i, o, kw: [unbroadcast(g * (1 - i[2]), i[0].shape), unbroadcast(g * i[2], i[1].shape),
                          unbroadcast(g * (i[1] - i[0]), i[2].shape)], "d(lerp(s,e,w))/ds=1-w; de=w; dw=e-s")


# ---------------------------------------------------------------------------------- norms
def _dist_vjp(g, i, o, kw):
    a, b = i
    p = float(kw.get("p", 2.0))
    d = a - b
    if p == 2.0:
        w = d / torch.where(o == 0, torch.ones_like(o), o)
    elif p == 1.0:
        w = torch.sign(d)
    elif math.isinf(p):
        m = (d.abs() == o).to(d.dtype)
        w = torch.sign(d) * m / m.sum()
    else:
        w = torch.sign(d) * d.abs().pow(p - 1) / torch.where(o == 0, torch.ones_like(o), o).pow(p - 1)
    w = g * w
    return [unbroadcast(w, a.shape), unbroadcast(-w, b.shape)]


_reg("dist", lambda a, b, p=2.0: torch.dist(a, b, p), _dist_vjp, "d(||a-b||_p)/da=sign(d)|d|^(p-1)/||d||_p^(p-1); db=-da")


def _pnorm_and_grad(x, p, dims):
    n = torch.linalg.vector_norm(x, ord=p, dim=dims, keepdim=True)
    safe = torch.where(n == 0, torch.ones_like(n), n)
    if p == 2.0:
        dn = x / safe
    elif p == 1.0:
        dn = torch.sign(x)
    else:
        dn = torch.sign(x) * x.abs().pow(p - 1) / safe.pow(p - 1)
    return n, dn


def _renorm_fwd(x, p=2.0, dim=0, maxnorm=1.0):
    return torch.renorm(x, p, int(dim), maxnorm)


def _renorm_vjp(g, i, o, kw):
    x = i[0]
    p, dim, m = float(kw.get("p", 2.0)), int(kw.get("dim", 0)) % i[0].dim(), float(kw.get("maxnorm", 1.0))
    dims = [d for d in range(x.dim()) if d != dim]
    n, dn = _pnorm_and_grad(x, p, dims)
    s = m / (n + 1e-7)
    gx = (g * x).sum(dims, keepdim=True)
    scaled = g * s - (m / (n + 1e-7) ** 2) * gx * dn
    return [torch.where(n > m, scaled, g)]


_reg("renorm", _renorm_fwd, _renorm_vjp,
     "rows with ||x||_p>m: y=x*m/(n+1e-7), dx=g*m/(n+eps)-m/(n+eps)^2*<g,x>*dn/dx; other rows dx=g")


def _normalize_fwd(x, p=2.0, dim=1, eps=1e-12):
    return torch.nn.functional.normalize(x, p=p, dim=int(dim), eps=eps)


def _normalize_vjp(g, i, o, kw):
    x = i[0]
    p, dim, eps = float(kw.get("p", 2.0)), int(kw.get("dim", 1)), float(kw.get("eps", 1e-12))
    n, dn = _pnorm_and_grad(x, p, [dim])
    gx = (g * x).sum(dim, keepdim=True)
    big = g / torch.clamp_min(n, eps) - gx * dn / torch.clamp_min(n, eps) ** 2
    return [torch.where(n > eps, big, g / eps)]


_reg("normalize", _normalize_fwd, _normalize_vjp, "y=x/max(||x||_p,eps): dx=g/n-<g,x>*dn/dx/n^2 (g/eps when n<=eps)")


# ---------------------------------------------------------------------------------- reductions
def _even_ties(g, x, out, dim, keepdim):
    if dim is None:
        mask = (x == out).to(g.dtype)
        return g * mask / mask.sum()
    if not keepdim:
        g, out = g.unsqueeze(dim), out.unsqueeze(dim)
    mask = (x == out).to(g.dtype)
    return g * mask / mask.sum(dim, keepdim=True)


def _ext(name, fn, rule):
    _reg(name, lambda x, dim=None, keepdim=False: fn(x) if dim is None else fn(x, dim=int(dim), keepdim=keepdim),
         lambda g, i, o, kw: [_even_ties(g, i[0], o, None if kw.get("dim") is None else int(kw["dim"]), kw.get("keepdim", False))],
         rule)


_ext("amax", torch.amax, "d(amax(x))/dx=grad/count on the positions equal to the maximum")
_ext("amin", torch.amin, "d(amin(x))/dx=grad/count on the positions equal to the minimum")


def _nan_fill(x, v):
    return torch.where(torch.isnan(x), torch.full_like(x, v), x)


_ext("nanmax", lambda x, **kw: torch.amax(_nan_fill(x, -math.inf), **kw), "as amax over the non-NaN elements")
_ext("nanmin", lambda x, **kw: torch.amin(_nan_fill(x, math.inf), **kw), "as amin over the non-NaN elements")


def _red_shape(g, x, dim, keepdim):
    if dim is None:
        return g.expand_as(x)
    return (g if keepdim else g.unsqueeze(dim)).expand_as(x)


def _dimkw(kw):
    return (None if kw.get("dim") is None else int(kw["dim"])), kw.get("keepdim", False)


_reg("nansum", lambda x, dim=None, keepdim=False: torch.nansum(x) if dim is None else torch.nansum(x, dim=int(dim), keepdim=keepdim),
     lambda g, i, o, kw: [_red_shape(g, i[0], *_dimkw(kw)) * ~torch.isnan(i[0])], "d(nansum(x))/dx=1 where x is not NaN")


def _nanmean_vjp(g, i, o, kw):
    x = i[0]
    dim, keepdim = _dimkw(kw)
    ok = ~torch.isnan(x)
    cnt = ok.sum() if dim is None else ok.sum(dim, keepdim=True)
    return [_red_shape(g, x, dim, keepdim) * ok / cnt]


_reg("nanmean", lambda x, dim=None, keepdim=False: torch.nanmean(x) if dim is None else torch.nanmean(x, dim=int(dim), keepdim=keepdim),
     _nanmean_vjp, "d(nanmean(x))/dx=1/count(non-NaN) where x is not NaN")


def _nanprod_fwd(x, dim=None, keepdim=False):
    y = _nan_fill(x, 1.0)
    return y.prod() if dim is None else y.prod(int(dim), keepdim=keepdim)


def _nanprod_vjp(g, i, o, kw):
    x = _nan_fill(i[0], 1.0)
    dim, keepdim = _dimkw(kw)
    flat = x.reshape(-1) if dim is None else x
    d = 0 if dim is None else dim
    # product of the others = exclusive prefix product * exclusive suffix product (no division: zeros are fine)
    ones = torch.ones_like(flat.narrow(d, 0, 1))
    pre = torch.cat([ones, flat.narrow(d, 0, flat.shape[d] - 1)], d).cumprod(d)
    suf = torch.cat([flat.narrow(d, 1, flat.shape[d] - 1), ones], d).flip(d).cumprod(d).flip(d)
    others = (pre * suf).reshape(x.shape)
    return [_red_shape(g, x, dim, keepdim) * others * ~torch.isnan(i[0])]


_reg("nanprod", _nanprod_fwd, _nanprod_vjp, "d(prod of non-NaN)/dx_i=prod_{j!=i} x_j (prefix*suffix products)")


def _nanvar_fwd(x, correction=1, dim=None, keepdim=False):
    ok = ~torch.isnan(x)
    xz = torch.where(ok, x, torch.zeros_like(x))
    if dim is None:
        cnt, mean = ok.sum(), xz.sum() / ok.sum()
        return (torch.where(ok, (x - mean) ** 2, torch.zeros_like(x))).sum() / (cnt - correction)
    cnt = ok.sum(int(dim), keepdim=True)
    mean = xz.sum(int(dim), keepdim=True) / cnt
    v = torch.where(ok, (x - mean) ** 2, torch.zeros_like(x)).sum(int(dim), keepdim=True) / (cnt - correction)
    return v if keepdim else v.squeeze(int(dim))


def _nanvar_vjp(g, i, o, kw):
    x = i[0]
    dim, keepdim = _dimkw(kw)
    c = kw.get("correction", 1)
    ok = ~torch.isnan(x)
    xz = torch.where(ok, x, torch.zeros_like(x))
    cnt = ok.sum() if dim is None else ok.sum(dim, keepdim=True)
    mean = xz.sum() / cnt if dim is None else xz.sum(dim, keepdim=True) / cnt
    return [_red_shape(g, x, dim, keepdim) * torch.where(ok, 2 * (x - mean) / (cnt - c), torch.zeros_like(x))]


_reg("nanvar", _nanvar_fwd, _nanvar_vjp, "d(var of non-NaN)/dx=2*(x-mean)/(count-correction) where x is not NaN")
_reg("nanstd", lambda x, correction=1, dim=None, keepdim=False: torch.sqrt(_nanvar_fwd(x, correction, dim, keepdim)),
     lambda g, i, o, kw: _nanvar_vjp(g / (2 * o), i, o, kw), "d(sqrt(var))/dx=dvar/(2*std)")


def _pick_vjp(idx_fn):
    """Rule of a reduction that returns one existing element per slice: the gradient goes to that element."""
    def vjp(g, i, o, kw):
        x = i[0]
        dim, keepdim, idx = idx_fn(x, kw)
        gx = torch.zeros_like(x, dtype=g.dtype)
        if dim is None:
            gx.reshape(-1)[idx] = g.reshape(())
            return [gx]
        return [gx.scatter(dim, idx if keepdim else idx.unsqueeze(dim), g if keepdim else g.unsqueeze(dim))]
    return vjp


def _nanmedian_idx(x, kw):
    dim, keepdim = _dimkw(kw)
    if dim is None:
        v = torch.nanmedian(x)
        flat = x.reshape(-1)
        return None, False, int(torch.nonzero(flat == v)[0]) if not torch.isnan(v) else 0
    return dim, keepdim, torch.nanmedian(x, dim=dim, keepdim=keepdim).indices


_reg("nanmedian", lambda x, dim=None, keepdim=False: torch.nanmedian(x) if dim is None else torch.nanmedian(x, dim=int(dim), keepdim=keepdim).values,
     _pick_vjp(_nanmedian_idx), "gradient flows to the element picked as the median of the non-NaN values")
_reg("kthvalue", lambda x, k=1, dim=-1, keepdim=False: torch.kthvalue(x, int(k), int(dim), keepdim).values,
     _pick_vjp(lambda x, kw: (int(kw.get("dim", -1)) % x.dim(), kw.get("keepdim", False),
                              torch.kthvalue(x, int(kw.get("k", 1)), int(kw.get("dim", -1)), kw.get("keepdim", False)).indices)),
     "gradient flows to the k-th smallest element of each slice")


def _quantile_fwd(x, q=0.5, dim=None, keepdim=False, interpolation="linear", ignore_nan=False):
    fn = torch.nanquantile if ignore_nan else torch.quantile
    qt = torch.as_tensor(q, dtype=x.dtype, device=x.device)
    return fn(x, qt, dim=None if dim is None else int(dim), keepdim=keepdim, interpolation=interpolation)


def _quantile_vjp(g, i, o, kw):
    """Quantiles are a fixed convex combination of two order statistics of each slice: the gradient is
    routed to their positions with the interpolation weights."""
    x = i[0]
    dim, keepdim = _dimkw(kw)
    interp, ignore_nan = kw.get("interpolation", "linear"), kw.get("ignore_nan", False)
    q = torch.as_tensor(kw.get("q", 0.5), dtype=x.dtype, device=x.device)
    multi = q.dim() > 0
    qs = q.reshape(-1)
    xs = x.reshape(1, -1) if dim is None else x.movedim(dim, -1).reshape(-1, x.shape[dim])
    srt, order = torch.sort(xs, dim=-1)           # NaNs sort last
    n = (~torch.isnan(xs)).sum(-1, keepdim=True) if ignore_nan else torch.full_like(order[:, :1], xs.shape[-1])
    gq = g if multi else g.unsqueeze(0)            # [Q, *reduced]
    if dim is not None and keepdim:
        gq = gq.squeeze(dim + 1)
    gq = gq.reshape(qs.numel(), -1)                # [Q, rows]
    gx = torch.zeros_like(xs, dtype=g.dtype)
    for k in range(qs.numel()):
        pos = qs[k] * (n - 1).to(x.dtype)           # [rows, 1]
        lo, hi = torch.floor(pos), torch.ceil(pos)
        if interp == "lower":
            w_hi = torch.zeros_like(pos)
        elif interp == "higher":
            w_hi = torch.ones_like(pos)
        elif interp == "nearest":
            w_hi = (torch.round(pos) == hi).to(pos.dtype) * (hi != lo)
        elif interp == "midpoint":
            w_hi = torch.full_like(pos, 0.5) * (hi != lo)
        else:
            w_hi = pos - lo
        lo_i = order.gather(-1, lo.long().clamp_min(0))
        hi_i = order.gather(-1, hi.long().clamp_min(0))
        gk = gq[k].unsqueeze(-1)
        gx.scatter_add_(-1, lo_i, gk * (1 - w_hi))
        gx.scatter_add_(-1, hi_i, gk * w_hi)
    if dim is None:
        return [gx.reshape(x.shape)]
    return [gx.reshape(x.movedim(dim, -1).shape).movedim(-1, dim)]


_reg("quantile_full", _quantile_fwd, _quantile_vjp,
     "d(quantile)/dx: weights (1-w, w) on the two order statistics that bracket q*(n-1)")


def _logcumsumexp_vjp(g, i, o, kw):
    x, dim = i[0], int(kw.get("dim", 0))
    # dx_i = exp(x_i) * sum_{j>=i} g_j*exp(-out_j); positive and negative parts of g are carried in log space
    def part(gp):
        lg = torch.log(gp) - o
        return torch.exp(x + torch.logcumsumexp(lg.flip(dim), dim).flip(dim))
    zero = torch.zeros_like(g)
    return [part(torch.maximum(g, zero)) - part(torch.maximum(-g, zero))]


_reg("logcumsumexp", lambda x, dim=0: torch.logcumsumexp(x, int(dim)), _logcumsumexp_vjp,
     "d(logcumsumexp(x))/dx_i=exp(x_i)*sum_{j>=i} grad_j*exp(-out_j)")


# ---------------------------------------------------------------------------------- finite differences / quadrature
def _diff_adj(g, dim):
    """Adjoint of a first difference along ``dim``: ``[-g_0, g_0-g_1, ..., g_{n-2}]``."""
    z = torch.zeros_like(g.narrow(dim, 0, 1))
    return torch.cat([z, g], dim) - torch.cat([g, z], dim)


def _diff_fwd(x, n=1, dim=-1, prepend=None, append=None):
    return torch.diff(x, n=int(n), dim=int(dim), prepend=prepend, append=append)


def _diff_vjp_for(layout):
    def vjp(g, i, o, kw):
        n, dim = int(kw.get("n", 1)), int(kw.get("dim", -1))
        for _ in range(n):
            g = _diff_adj(g, dim)
        parts = dict(zip(layout, i))
        sizes = [(k, parts[k].shape[dim]) for k in ("prepend", "x", "append") if k in parts]
        outs, off = {}, 0
        for k, s in sizes:
            outs[k] = g.narrow(dim, off, s)
            off += s
        return [outs[k] for k in layout]
    return vjp


_reg("diff", lambda x, dim=-1: torch.diff(x, dim=int(dim)), _diff_vjp_for(("x",)),
     "d(x[i+1]-x[i])/dx: adjoint of the first difference, [-g_0, g_0-g_1, ..., g_{n-2}]")
_reg("diff_full", lambda x, n=1, dim=-1: _diff_fwd(x, n, dim), _diff_vjp_for(("x",)), "n-th difference: the adjoint applied n times")
_reg("diff_full_prepend", lambda x, prepend, n=1, dim=-1: _diff_fwd(x, n, dim, prepend=prepend), _diff_vjp_for(("x", "prepend")),
     "n-th difference of cat(prepend,x): the adjoint applied n times, then split")
_reg("diff_full_append", lambda x, append, n=1, dim=-1: _diff_fwd(x, n, dim, append=append), _diff_vjp_for(("x", "append")),
     "n-th difference of cat(x,append): the adjoint applied n times, then split")
_reg("diff_full_both", lambda x, prepend, append, n=1, dim=-1: _diff_fwd(x, n, dim, prepend, append),
     _diff_vjp_for(("x", "prepend", "append")), "n-th difference of cat(prepend,x,append): the adjoint applied n times, then split")


def _trap_vjp(g, i, o, kw):
    y, dim = i[0], int(kw.get("dim", -1)) % i[0].dim()
    n = y.shape[dim]
    ge = g.unsqueeze(dim)
    if len(i) == 1:
        w = torch.full((n,), float(kw.get("dx", 1.0)), dtype=g.dtype, device=g.device)
        w[0] *= 0.5
        w[-1] *= 0.5
        shape = [1] * y.dim()
        shape[dim] = n
        return [ge * w.reshape(shape)]
    x = i[1]
    xb = x if x.dim() == y.dim() else x.reshape([-1 if d == dim else 1 for d in range(y.dim())])
    dx = torch.diff(xb, dim=dim)                                     # spacing of each panel
    z = torch.zeros_like(dx.narrow(dim, 0, 1))
    wy = 0.5 * (torch.cat([dx, z], dim) + torch.cat([z, dx], dim))    # weight of y_i = (dx_{i-1}+dx_i)/2
    ysum = 0.5 * (y.narrow(dim, 0, n - 1) + y.narrow(dim, 1, n - 1))  # d/d(dx_i)
    gx = _diff_adj(ge * ysum, dim)
    return [(ge * wy).expand(y.shape), unbroadcast(gx, xb.shape).reshape(x.shape)]


_reg("trapezoid", lambda y, dx=1.0, dim=-1: torch.trapezoid(y, dx=dx, dim=int(dim)), _trap_vjp,
     "d(trapz(y))/dy=dx*[1/2,1,...,1,1/2]")
_reg("trapezoid_x", lambda y, x, dim=-1: torch.trapezoid(y, x, dim=int(dim)), _trap_vjp,
     "d(trapz(y,x))/dy_i=(x_{i+1}-x_{i-1})/2 (one-sided at the ends); dx: adjoint difference of grad*(y_i+y_{i+1})/2")


def _cumtrap_vjp(g, i, o, kw):
    y, dim = i[0], int(kw.get("dim", -1)) % i[0].dim()
    n = y.shape[dim]
    h = g.flip(dim).cumsum(dim).flip(dim)                 # h_i = sum_{j>=i} g_j: panel i feeds every later output
    if len(i) == 1:
        hd = h * float(kw.get("dx", 1.0))
        z = torch.zeros_like(hd.narrow(dim, 0, 1))
        return [0.5 * (torch.cat([hd, z], dim) + torch.cat([z, hd], dim))]
    x = i[1]
    xb = x if x.dim() == y.dim() else x.reshape([-1 if d == dim else 1 for d in range(y.dim())])
    dx = torch.diff(xb, dim=dim)
    hd = h * dx
    z = torch.zeros_like(hd.narrow(dim, 0, 1))
    ysum = 0.5 * (y.narrow(dim, 0, n - 1) + y.narrow(dim, 1, n - 1))
    return [0.5 * (torch.cat([hd, z], dim) + torch.cat([z, hd], dim)), unbroadcast(_diff_adj(h * ysum, dim), xb.shape).reshape(x.shape)]


_reg("cumulative_trapezoid", lambda y, dx=1.0, dim=-1: torch.cumulative_trapezoid(y, dx=dx, dim=int(dim)), _cumtrap_vjp,
     "d(cumtrapz(y))/dy_i=dx/2*(h_i+h_{i-1}), h=reverse cumsum of grad")
_reg("cumulative_trapezoid_x", lambda y, x, dim=-1: torch.cumulative_trapezoid(y, x, dim=int(dim)), _cumtrap_vjp,
     "as cumtrapz with panel widths x_{i+1}-x_i; dx: adjoint difference of h*(y_i+y_{i+1})/2")


def _gradient_stencil(n: int, h: float, edge_order: int, dtype, device) -> torch.Tensor:
    """Matrix ``D`` with ``gradient(x) = D @ x`` for uniform spacing ``h`` (second-order interior)."""
    D = torch.zeros(n, n, dtype=dtype, device=device)
    r = torch.arange(1, n - 1)
    D[r, r + 1], D[r, r - 1] = 0.5 / h, -0.5 / h
    if edge_order == 1:
        D[0, 0], D[0, 1] = -1.0 / h, 1.0 / h
        D[-1, -2], D[-1, -1] = -1.0 / h, 1.0 / h
    else:
        D[0, 0], D[0, 1], D[0, 2] = -1.5 / h, 2.0 / h, -0.5 / h
        D[-1, -3], D[-1, -2], D[-1, -1] = 0.5 / h, -2.0 / h, 1.5 / h
    return D


def _gradient_dim_vjp(g, i, o, kw):
    x, dim = i[0], int(kw.get("dim", 0))
    D = _gradient_stencil(x.shape[dim], float(kw.get("spacing", 1.0)), int(kw.get("edge_order", 1)), g.dtype, g.device)
    return [torch.movedim(torch.movedim(g, dim, -1) @ D, -1, dim)]      # D^T applied along dim


_reg("gradient_dim", lambda x, dim=0, spacing=1.0, edge_order=1:
     torch.gradient(x, spacing=float(spacing), dim=int(dim), edge_order=int(edge_order))[0], _gradient_dim_vjp,
     "gradient(x)=D@x along dim (central differences, one-sided ends): dx=D^T@grad")


# ---------------------------------------------------------------------------------- selection / scatter
def _sel_vjp(g, i, o, kw):
    gx = torch.zeros_like(i[0], dtype=g.dtype)
    gx.select(int(kw.get("dim", 0)), int(kw.get("index", 0))).copy_(g)
    return [gx]


_reg("select", lambda x, dim=0, index=0: torch.select(x, int(dim), int(index)), _sel_vjp, "d(select)/dx: grad placed in the selected slice, 0 elsewhere")
_reg("select_scatter", lambda x, src, dim=0, index=0: torch.select_scatter(x, src, int(dim), int(index)),
     lambda g, i, o, kw: [torch.select_scatter(g, torch.zeros_like(i[1], dtype=g.dtype), int(kw.get("dim", 0)), int(kw.get("index", 0))),
                          g.select(int(kw.get("dim", 0)), int(kw.get("index", 0)))],
     "d/dx=grad with the slice zeroed; d/dsrc=the slice of grad")


def _ss_kw(kw):
    return dict(dim=int(kw.get("dim", 0)), start=kw.get("start"), end=kw.get("end"), step=int(kw.get("step", 1)))


_reg("slice_scatter", lambda x, src, dim=0, start=None, end=None, step=1: torch.slice_scatter(x, src, int(dim), start, end, int(step)),
     lambda g, i, o, kw: [torch.slice_scatter(g, torch.zeros_like(i[1], dtype=g.dtype), **_ss_kw(kw)),
                          g[(slice(None),) * (_ss_kw(kw)["dim"] % g.dim()) + (slice(kw.get("start"), kw.get("end"), int(kw.get("step", 1))),)]],
     "d/dx=grad with the slice zeroed; d/dsrc=the slice of grad")
_reg("diagonal_scatter", lambda x, src, offset=0: torch.diagonal_scatter(x, src, int(offset)),
     lambda g, i, o, kw: [torch.diagonal_scatter(g, torch.zeros_like(i[1], dtype=g.dtype), int(kw.get("offset", 0))),
                          torch.diagonal(g, int(kw.get("offset", 0)))],
     "d/dx=grad with the diagonal zeroed; d/dsrc=the diagonal of grad")
def _diag_vjp(g, i, o, kw):
    x, k = i[0], int(kw.get("diagonal", 0))
    if x.dim() == 1:
        return [torch.diagonal(g, k)]
    return [torch.diagonal_scatter(torch.zeros_like(x, dtype=g.dtype), g, k)]


_reg("diag", lambda x, diagonal=0: torch.diag(x, int(diagonal)), _diag_vjp,
     "d(diag(x,k))/dx: vector -> the k-th diagonal of grad; matrix -> grad placed on the k-th diagonal")
_reg("diag_embed", lambda x, offset=0: torch.diag_embed(x, int(offset)),
     lambda g, i, o, kw: [torch.diagonal(g, int(kw.get("offset", 0)), -2, -1)], "d(diag_embed(x,k))/dx=diagonal(grad,k)")
_reg("diagflat", lambda x, offset=0: torch.diagflat(x, int(offset)),
     lambda g, i, o, kw: [torch.diagonal(g, int(kw.get("offset", 0))).reshape(i[0].shape)], "d(diagflat(x,k))/dx=diagonal(grad,k)")
_reg("rot90", lambda x, k=1, dims=(0, 1): torch.rot90(x, int(k), list(dims)),
     lambda g, i, o, kw: [torch.rot90(g, -int(kw.get("k", 1)), list(kw.get("dims", (0, 1))))], "d(rot90(x,k))/dx=rot90(grad,-k)")
_reg("fliplr", torch.fliplr, lambda g, i, o, kw: [torch.fliplr(g)], "d(fliplr(x))/dx=fliplr(grad)")
_reg("flipud", torch.flipud, lambda g, i, o, kw: [torch.flipud(g)], "d(flipud(x))/dx=flipud(grad)")
_reg("matrix_transpose", lambda x: x.mT, lambda g, i, o, kw: [g.mT], "d(x^T)/dx=grad^T")
_reg("ravel", lambda x: x.reshape(-1), lambda g, i, o, kw: [g.reshape(i[0].shape)], "d(ravel(x))/dx=reshape(grad)")
_reg("squeeze_all", lambda x: x.squeeze(), lambda g, i, o, kw: [g.reshape(i[0].shape)], "d(squeeze(x))/dx=reshape(grad)")
for _k, _f in ((1, lambda x: torch.atleast_1d(x)), (2, lambda x: torch.atleast_2d(x)), (3, lambda x: torch.atleast_3d(x))):
    _reg(f"atleast_{_k}d", _f, lambda g, i, o, kw: [g.reshape(i[0].shape)], "d(atleast_kd(x))/dx=reshape(grad)")
_reg("view_as", lambda x, other: x.reshape(other.shape), lambda g, i, o, kw: [g.reshape(i[0].shape), None],
     "d(view_as(x,o))/dx=reshape(grad)")
_reg("msort", torch.msort, lambda g, i, o, kw: [torch.zeros_like(g).scatter(0, torch.argsort(i[0], dim=0, stable=True), g)],
     "d(sort along dim 0)/dx: grad scattered back through the sorting permutation")


def _ri_fwd(x, repeats=1, dim=None):
    return torch.repeat_interleave(x, int(repeats), dim=None if dim is None else int(dim))


def _ri_vjp(g, i, o, kw):
    x, r, dim = i[0], int(kw.get("repeats", 1)), kw.get("dim")
    if dim is None:
        return [g.reshape(-1, r).sum(-1).reshape(x.shape)]
    dim = int(dim) % x.dim()
    return [g.reshape(x.shape[:dim] + (x.shape[dim], r) + x.shape[dim + 1:]).sum(dim + 1)]


_reg("repeat_interleave", _ri_fwd, _ri_vjp, "d(repeat_interleave(x,r))/dx=sum of each run of r copies")


def _rit_fwd(x, repeats=(), dim=None):
    return torch.repeat_interleave(x, torch.as_tensor(list(repeats), dtype=torch.long, device=x.device), dim=None if dim is None else int(dim))


def _rit_vjp(g, i, o, kw):
    x, dim = i[0], kw.get("dim")
    reps = torch.as_tensor(list(kw.get("repeats", ())), dtype=torch.long, device=g.device)
    src = torch.repeat_interleave(torch.arange(reps.numel(), device=g.device), reps)
    if dim is None:
        return [torch.zeros(x.numel(), dtype=g.dtype, device=g.device).index_add_(0, src, g.reshape(-1)).reshape(x.shape)]
    return [torch.zeros_like(x, dtype=g.dtype).index_add_(int(dim), src, g)]


_reg("repeat_interleave_tensor", _rit_fwd, _rit_vjp, "d/dx: index_add of grad by the source position of each copy")


def _take_vjp(g, i, o, kw):
    x, idx = i[0], i[1].long()
    return [torch.zeros(x.numel(), dtype=g.dtype, device=g.device).index_add_(0, idx.reshape(-1) % x.numel(), g.reshape(-1)).reshape(x.shape), None]


_reg("take", lambda x, idx: torch.take(x, idx.long()), _take_vjp, "d(take(x,idx))/dx=index_add of grad at the flat indices")
_reg("take_along_dim", lambda x, idx, dim=0: torch.take_along_dim(x, idx.long(), int(dim)),
     lambda g, i, o, kw: [torch.zeros_like(i[0], dtype=g.dtype).scatter_add_(int(kw.get("dim", 0)), i[1].long().expand_as(g) if i[1].shape != g.shape else i[1].long(), g), None],
     "d(take_along_dim)/dx=scatter_add of grad at idx")
_reg("put", lambda x, idx, values, accumulate=False: torch.put(x, idx.long(), values, bool(accumulate)),
     lambda g, i, o, kw: [g if kw.get("accumulate", False) else torch.put(g, i[1].long(), torch.zeros_like(i[2], dtype=g.dtype)), None,
                          torch.take(g, i[1].long()).reshape(i[2].shape)],
     "d/dx=grad (zeroed at idx unless accumulating); d/dvalues=take(grad,idx)")
_reg("index_add", lambda x, idx, src, dim=0, alpha=1.0: torch.index_add(x, int(dim), idx.long(), src, alpha=alpha),
     lambda g, i, o, kw: [g, None, kw.get("alpha", 1.0) * g.index_select(int(kw.get("dim", 0)), i[1].long())],
     "d/dx=grad; d/dsrc=alpha*index_select(grad,idx)")
_reg("index_copy", lambda x, idx, src, dim=0: torch.index_copy(x, int(dim), idx.long(), src),
     lambda g, i, o, kw: [g.index_fill(int(kw.get("dim", 0)), i[1].long(), 0), None, g.index_select(int(kw.get("dim", 0)), i[1].long())],
     "d/dx=grad zeroed at idx; d/dsrc=index_select(grad,idx)")
_reg("index_fill", lambda x, idx, dim=0, value=0.0: torch.index_fill(x, int(dim), idx.long(), value),
     lambda g, i, o, kw: [g.index_fill(int(kw.get("dim", 0)), i[1].long(), 0), None], "d/dx=grad zeroed at idx")


def _masked_scatter_vjp(g, i, o, kw):
    x, mask, src = i
    mb = mask.bool().expand_as(x)
    gs = torch.zeros(src.numel(), dtype=g.dtype, device=g.device)
    picked = g[mb]
    gs[:picked.numel()] = picked
    return [g.masked_fill(mb, 0), None, gs.reshape(src.shape)]


_reg("masked_scatter", lambda x, mask, src: torch.masked_scatter(x, mask.bool(), src), _masked_scatter_vjp,
     "d/dx=grad zeroed under the mask; d/dsrc=the masked elements of grad, in order")
_reg("where_scalar", lambda cond, x=0.0, y=0.0: torch.where(cond.bool(), torch.as_tensor(float(x), dtype=torch.float64, device=cond.device),
                                                            torch.as_tensor(float(y), dtype=torch.float64, device=cond.device)),
     None, "no gradient (both branches are constants)")


def _reduce_scatter_like(g, x, idx, src, out, dim, mode, include_self, gather_fn, scatter_add_fn):
    """Shared rule of ``scatter_reduce`` / ``index_reduce``; ``gather_fn(t)`` reads ``t`` at the scattered
    positions (shape of ``src``), ``scatter_add_fn(zeros, t)`` adds ``t`` (shape of ``src``) into them."""
    if mode in ("sum", "add"):
        return (g if include_self else g * (scatter_add_fn(torch.zeros_like(x, dtype=g.dtype), torch.ones_like(src, dtype=g.dtype)) == 0)), gather_fn(g)
    hit = scatter_add_fn(torch.zeros_like(x, dtype=g.dtype), torch.ones_like(src, dtype=g.dtype))
    if mode == "mean":
        n = hit + (1.0 if include_self else 0.0)
        n = torch.where(n == 0, torch.ones_like(n), n)
        gs = g / n
        return (gs if include_self else torch.where(hit == 0, g, torch.zeros_like(g))), gather_fn(gs)
    if mode == "prod":
        go = g * out
        gx = go / x if include_self else torch.where(hit == 0, g, torch.zeros_like(g))
        return gx, gather_fn(go) / src
    # amax / amin: the gradient is shared evenly by every contribution equal to the result
    x_eq = (x == out).to(g.dtype)
    if not include_self:
        x_eq = torch.where(hit == 0, x_eq, torch.zeros_like(x_eq))
    s_eq = (src == gather_fn(out)).to(g.dtype)
    cnt = scatter_add_fn(x_eq.clone(), s_eq)
    share = g / torch.where(cnt == 0, torch.ones_like(cnt), cnt)
    return share * x_eq, gather_fn(share) * s_eq


def _scatter_reduce_vjp(g, i, o, kw):
    x, idx, src = i[0], i[1].long(), i[2]
    dim, mode, inc = int(kw.get("dim", 0)), kw.get("reduce", "sum"), kw.get("include_self", True)
    gx, gs = _reduce_scatter_like(g, x, idx, src, o, dim, mode, inc, lambda t: t.gather(dim, idx),
                                  lambda z, t: z.scatter_add(dim, idx, t))
    return [gx, None, gs]


_reg("scatter_reduce", lambda x, idx, src, dim=0, reduce="sum", include_self=True:
     torch.scatter_reduce(x, int(dim), idx.long(), src, reduce, include_self=include_self), _scatter_reduce_vjp,
     "sum: grad / gather(grad); mean: divided by the contribution count; prod: grad*out/operand; amax|amin: shared evenly by the ties")


def _index_reduce_vjp(g, i, o, kw):
    x, idx, src = i[0], i[1].long(), i[2]
    dim, mode, inc = int(kw.get("dim", 0)), kw.get("reduce", "prod"), kw.get("include_self", True)
    gx, gs = _reduce_scatter_like(g, x, idx, src, o, dim, mode, inc, lambda t: t.index_select(dim, idx),
                                  lambda z, t: z.index_add(dim, idx, t))
    return [gx, None, gs]


_reg("index_reduce", lambda x, idx, src, dim=0, reduce="prod", include_self=True:
     torch.index_reduce(x, int(dim), idx.long(), src, reduce, include_self=include_self), _index_reduce_vjp,
     "as scatter_reduce with whole slices addressed by idx")


# ---------------------------------------------------------------------------------- constructions from several tensors
def _block_diag_vjp(g, i, o, kw):
    outs, r, c = [], 0, 0
    for x in i:
        h, w = (1, 1) if x.dim() == 0 else ((1, x.shape[0]) if x.dim() == 1 else tuple(x.shape))
        outs.append(g[r:r + h, c:c + w].reshape(x.shape))
        r, c = r + h, c + w
    return outs


_reg("block_diag", lambda *xs: torch.block_diag(*xs), _block_diag_vjp, "d(block_diag)/dx_k=the k-th diagonal block of grad")


def _cartesian_vjp(g, i, o, kw):
    if len(i) == 1:
        return [g.reshape(i[0].shape)]
    sizes = [x.shape[0] for x in i]
    gg = g.reshape(*sizes, len(i))
    return [gg[..., k].sum([d for d in range(len(i)) if d != k]) for k in range(len(i))]


_reg("cartesian_prod", lambda *xs: torch.cartesian_prod(*xs), _cartesian_vjp,
     "d/dx_k=column k of grad summed over the other factors' positions")
_reg("column_stack", lambda *xs: torch.column_stack(xs),
     lambda g, i, o, kw: [p.reshape(x.shape) for p, x in zip(torch.split(g, [1 if x.dim() < 2 else x.shape[1] for x in i], 1), i)],
     "d(column_stack)/dx_k=the columns of grad that x_k filled")


def _comb_index(n, r, with_replacement, device):
    import itertools
    it = itertools.combinations_with_replacement(range(n), r) if with_replacement else itertools.combinations(range(n), r)
    rows = list(it)
    return torch.tensor(rows, dtype=torch.long, device=device).reshape(len(rows), r)


_reg("combinations", lambda x, r=2, with_replacement=False: torch.combinations(x, int(r), bool(with_replacement)),
     lambda g, i, o, kw: [torch.zeros_like(i[0], dtype=g.dtype).index_add_(
         0, _comb_index(i[0].shape[0], int(kw.get("r", 2)), kw.get("with_replacement", False), g.device).reshape(-1), g.reshape(-1))],
     "d(combinations(x))/dx=index_add of grad at the source index of every entry")


def _vander_fwd(x, n=None, increasing=False):
    return torch.vander(x, N=None if n is None else int(n), increasing=bool(increasing))


def _vander_vjp(g, i, o, kw):
    x = i[0]
    n = x.shape[0] if kw.get("n") is None else int(kw["n"])
    p = torch.arange(n, dtype=g.dtype, device=g.device)
    if not kw.get("increasing", False):
        p = p.flip(0)
    xe = x.unsqueeze(-1)
    d = p * torch.where(p == 0, torch.zeros_like(xe * p), torch.pow(xe, torch.clamp_min(p - 1, 0)))
    return [(g * d).sum(-1)]


_reg("vander", _vander_fwd, _vander_vjp, "d(x_i^p_j)/dx_i=sum_j grad_ij*p_j*x_i^(p_j-1)")


# ---------------------------------------------------------------------------------- matrices
def _inv_vjp(g, i, o, kw):
    yt = o.mT
    return [-(yt @ g @ yt)]


_reg("inverse", torch.linalg.inv, _inv_vjp, "d(A^-1)/dA=-A^-T@grad@A^-T")
_reg("det", torch.linalg.det, lambda g, i, o, kw: [(g * o)[..., None, None] * torch.linalg.inv(i[0]).mT], "d(det(A))/dA=det(A)*A^-T")
_reg("logdet", torch.logdet, lambda g, i, o, kw: [g[..., None, None] * torch.linalg.inv(i[0]).mT], "d(logdet(A))/dA=A^-T")


def _chol_inv_fwd(l, upper=False):
    return torch.cholesky_inverse(l, upper=bool(upper))


def _chol_inv_vjp(g, i, o, kw):
    l, upper = i[0], bool(kw.get("upper", False))
    # out = (L L^T)^-1 (or (U^T U)^-1); d(out) = -out dA out, dA = dL L^T + L dL^T
    ga = -(o.mT @ g @ o.mT)
    gs = ga + ga.mT
    # only the named triangle of the factor is read
    return [torch.triu(l @ gs) if upper else torch.tril(gs @ l)]


_reg("cholesky_inverse", _chol_inv_fwd, _chol_inv_vjp, "out=(L L^T)^-1: dA=-out^T@grad@out^T, dL=(dA+dA^T)@L (U: U@(dA+dA^T))")


# ---------------------------------------------------------------------------------- losses with the full argument list
def _ce_full_fwd(logits, target, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
    return torch.nn.functional.cross_entropy(logits, target.long(), weight=weight, ignore_index=int(ignore_index),
                                             reduction=reduction, label_smoothing=float(label_smoothing))


def _class_weights(logits, t, weight, ignore_index):
    """Per-sample weight (0 on ignored targets) and the safe target index."""
    keep = t != ignore_index
    ts = torch.where(keep, t, torch.zeros_like(t))
    w = torch.ones_like(ts, dtype=logits.dtype) if weight is None else weight.to(logits.dtype)[ts]
    return w * keep, ts, keep


def _ce_full_vjp(g, i, o, kw):
    logits, t = i[0], i[1].long()
    weight = i[2] if len(i) > 2 else None
    ii, red, eps = int(kw.get("ignore_index", -100)), kw.get("reduction", "mean"), float(kw.get("label_smoothing", 0.0))
    C = logits.shape[1] if logits.dim() > 1 else logits.shape[0]
    cdim = 1 if logits.dim() > 1 else 0
    w, ts, keep = _class_weights(logits, t, weight, ii)
    p = torch.softmax(logits, cdim)
    onehot = torch.zeros_like(p).scatter_(cdim, ts.unsqueeze(cdim), 1.0)
    wu = w.unsqueeze(cdim)
    # nll part: w_t * (p - onehot); smoothing part: sum_c w_c/C * (p - onehot_c) = (sum_c w_c / C) * p - w_c / C
    d = (1 - eps) * wu * (p - onehot)
    if eps > 0:
        wc = torch.ones(C, dtype=p.dtype, device=p.device) if weight is None else weight.to(p.dtype)
        shape = [1] * p.dim()
        shape[cdim] = C
        wcb = wc.reshape(shape)
        d = d + eps / C * (wcb.sum() * p - wcb) * keep.unsqueeze(cdim)
    if red == "mean":
        d = d * (g / w.sum())
    elif red == "sum":
        d = d * g
    else:
        d = d * g.unsqueeze(cdim)
    return [d, None] + ([None] if weight is not None else [])


_reg("cross_entropy_full", _ce_full_fwd, _ce_full_vjp,
     "d(CE)/dlogits=w_t*(softmax-onehot) (label smoothing: the mixture with the uniform target), 0 on ignored targets; mean divides by sum of w_t")


def _nll_full_fwd(lp, target, weight=None, ignore_index=-100, reduction="mean"):
    return torch.nn.functional.nll_loss(lp, target.long(), weight=weight, ignore_index=int(ignore_index), reduction=reduction)


def _nll_full_vjp(g, i, o, kw):
    lp, t = i[0], i[1].long()
    weight = i[2] if len(i) > 2 else None
    cdim = 1 if lp.dim() > 1 else 0
    w, ts, _ = _class_weights(lp, t, weight, int(kw.get("ignore_index", -100)))
    red = kw.get("reduction", "mean")
    scale = g / w.sum() if red == "mean" else (g if red == "sum" else g)
    d = torch.zeros_like(lp, dtype=g.dtype).scatter_(cdim, ts.unsqueeze(cdim), (-(w * scale)).unsqueeze(cdim))
    return [d, None] + ([None] if weight is not None else [])


_reg("nll_loss_full", _nll_full_fwd, _nll_full_vjp, "d(NLL)/dlp[n,t_n]=-w_t (mean: /sum of w_t), 0 on ignored targets")


def _bce_pw_fwd(x, t, pos_weight=1.0, reduction="mean"):
    pw = torch.as_tensor(float(pos_weight), dtype=x.dtype, device=x.device)
    return torch.nn.functional.binary_cross_entropy_with_logits(x, t, pos_weight=pw, reduction=reduction)


def _bce_pw_vjp(g, i, o, kw):
    x, t = i
    pw, red = float(kw.get("pos_weight", 1.0)), kw.get("reduction", "mean")
    s = torch.sigmoid(x)
    # loss = -pw*t*log(s) - (1-t)*log(1-s)
    dx = (1 - t) * s - pw * t * (1 - s)
    dt = -pw * torch.nn.functional.logsigmoid(x) + torch.nn.functional.logsigmoid(-x)
    k = g / x.numel() if red == "mean" else g
    return [dx * k, dt * k]


_reg("bce_with_logits_pos_weight", _bce_pw_fwd, _bce_pw_vjp, "d/dx=(1-t)*sigmoid(x)-pw*t*(1-sigmoid(x)); d/dt=-pw*ln(s)+ln(1-s)")


# ---------------------------------------------------------------------------------- real FFTs over several dimensions
def _cplx(x):
    return torch.view_as_complex(x.contiguous())


def _norm_scale(norm, n_total, inverse):
    """Factor that the transform applies on top of the unnormalised sum."""
    if norm == "ortho":
        return 1.0 / math.sqrt(n_total)
    if (norm == "forward") != inverse:      # forward transform under "forward", inverse under "backward" / None
        return 1.0 / n_total
    return 1.0


def _rfftn_fwd(x, s=None, dim=None, norm=None):
    return torch.view_as_real(torch.fft.rfftn(x, s=s, dim=dim, norm=norm)).contiguous()


def _fft_dims(x_ndim, s, dim):
    if dim is not None:
        return [d % x_ndim for d in dim]
    if s is not None:
        return list(range(x_ndim - len(s), x_ndim))
    return list(range(x_ndim))


def _fit(t, shape):
    """Crop or zero-pad ``t`` to ``shape`` (the adjoint of the transform's own pad / crop of its input)."""
    for d, n in enumerate(shape):
        if t.shape[d] > n:
            t = t.narrow(d, 0, n)
        elif t.shape[d] < n:
            pad = [0, 0] * t.dim()
            pad[2 * (t.dim() - 1 - d) + 1] = n - t.shape[d]
            t = torch.nn.functional.pad(t, pad)
    return t


def _rfftn_vjp(g, i, o, kw):
    x = i[0]
    dims = _fft_dims(x.dim(), kw.get("s"), kw.get("dim"))
    sizes = list(kw["s"]) if kw.get("s") is not None else [x.shape[d] for d in dims]
    n_total = math.prod(sizes)
    gc = _cplx(g)
    full = list(gc.shape)
    full[dims[-1]] = sizes[-1]
    gfull = _fit(gc, full)                                # the missing half of the spectrum contributes nothing
    # y_k = c * sum_n x_n e^{-i th}  =>  dx_n = c * Re(sum_k g_k e^{+i th}) = c * N * Re(ifftn(g))
    dx = torch.fft.ifftn(gfull, dim=dims).real * (n_total * _norm_scale(kw.get("norm"), n_total, False))
    return [_fit(dx, x.shape)]


_reg("rfftn", _rfftn_fwd, _rfftn_vjp, "d(rfftn(x))/dx=N*c*Re(ifftn(zero-extended grad)), c the norm factor")
_reg("rfft2", lambda x, s=None, norm=None: _rfftn_fwd(x, s, (-2, -1), norm),
     lambda g, i, o, kw: _rfftn_vjp(g, i, o, dict(kw, dim=(-2, -1))), "d(rfft2(x))/dx=N*c*Re(ifft2(zero-extended grad))")


def _irfft2_fwd(z, s=None, norm=None):
    return torch.fft.irfft2(_cplx(z), s=s, norm=norm)


def _irfft2_vjp(g, i, o, kw):
    z = i[0]
    zc_shape = z.shape[:-1]
    n0, n1 = g.shape[-2], g.shape[-1]
    n_total = n0 * n1
    m = n1 // 2 + 1                                      # half-spectrum bins the transform reads
    w = torch.full((m,), 2.0, dtype=g.dtype, device=g.device)
    w[0] = 1.0
    if n1 % 2 == 0:
        w[-1] = 1.0
    # out_n = c * sum_k w_k Re(z_k e^{+i th})  =>  dz_k = c * w_k * rfft2(grad)_k
    gz = torch.fft.rfft2(g) * w * _norm_scale(kw.get("norm"), n_total, True)
    return [torch.view_as_real(_fit(gz, zc_shape)).contiguous()]


_reg("irfft2", _irfft2_fwd, _irfft2_vjp, "d(irfft2(z))/dz_k=c*w_k*rfft2(grad)_k, w=1 at DC and Nyquist else 2")


# ---------------------------------------------------------------------------------- second batch
# Operators named in the reference's parity matrix and profiling notes (FEATURE_PARITY.md, docs/NEGATIVE_EVIDENCE.md):
# soft-target cross-entropy, multi-dimension variance, the remaining Chebyshev families, clamps against tensors,
# vecdot, inverse real FFTs, boolean reductions.
def _ce_soft_fwd(logits, probs, reduction="mean"):
    return torch.nn.functional.cross_entropy(logits, probs, reduction=reduction)


def _ce_soft_vjp(g, i, o, kw):
    logits, p = i
    cdim = 1 if logits.dim() > 1 else 0
    red = kw.get("reduction", "mean")
    ls = torch.log_softmax(logits, cdim)
    n = logits.numel() // logits.shape[cdim] if logits.dim() > 1 else 1
    k = g / n if red == "mean" else (g if red == "sum" else g.unsqueeze(cdim))
    return [k * (torch.exp(ls) * p.sum(cdim, keepdim=True) - p), -k * ls]


_reg("cross_entropy_soft", _ce_soft_fwd, _ce_soft_vjp,
     "loss=-sum_c p_c*log_softmax(x)_c: dx=softmax(x)*sum_c(p_c)-p; dp=-log_softmax(x); mean divides by the batch")


def _dims_tuple(dims, ndim):
    return tuple(sorted(int(d) % ndim for d in dims))


def _var_dims_fwd(x, dims=(0,), correction=1, keepdim=False):
    return torch.var(x, dim=_dims_tuple(dims, x.dim()), correction=correction, keepdim=keepdim)


def _var_dims_vjp(g, i, o, kw):
    x = i[0]
    dims = _dims_tuple(kw.get("dims", (0,)), x.dim())
    n = 1
    for d in dims:
        n *= x.shape[d]
    if not kw.get("keepdim", False):
        for d in dims:
            g = g.unsqueeze(d)
    return [g * 2.0 * (x - x.mean(dims, keepdim=True)) / (n - kw.get("correction", 1))]


_reg("var_dims", _var_dims_fwd, _var_dims_vjp, "d(var over dims)/dx=2*(x-mean)/(n-correction)")


def _std_dims_vjp(g, i, o, kw):
    og = o
    if not kw.get("keepdim", False):
        for d in _dims_tuple(kw.get("dims", (0,)), i[0].dim()):
            og = og.unsqueeze(d)
            g = g.unsqueeze(d)
        kw = dict(kw, keepdim=True)
    return _var_dims_vjp(g / (2.0 * og), i, o, kw)


_reg("std_dims", lambda x, dims=(0,), correction=1, keepdim=False: torch.std(x, dim=_dims_tuple(dims, x.dim()), correction=correction, keepdim=keepdim),
     _std_dims_vjp, "d(std over dims)/dx=(x-mean)/((n-correction)*std)")


def _cheb_u_d(x, n, un=None):
    """U_n'(x) = ((n+1)*T_{n+1}(x) - x*U_n(x)) / (x^2 - 1); (+-1)^(n+1) * n(n+1)(n+2)/3 at x = +-1."""
    if n <= 0:
        return torch.zeros_like(x)
    un = _S.chebyshev_polynomial_u(x, n) if un is None else un
    edge = x.abs() == 1
    den = torch.where(edge, torch.ones_like(x), x * x - 1)
    d = ((n + 1) * _S.chebyshev_polynomial_t(x, n + 1) - x * un) / den
    return torch.where(edge, torch.sign(x) ** (n + 1) * (n * (n + 1) * (n + 2) / 3.0), d)


def _cheb_t_d(x, n):
    return n * _S.chebyshev_polynomial_u(x, n - 1) if n > 0 else torch.zeros_like(x)


_poly("special_chebyshev_polynomial_u", _S.chebyshev_polynomial_u, lambda x, n, o: _cheb_u_d(x, n, o),
      "d(U_n(x))/dx=((n+1)*T_{n+1}(x)-x*U_n(x))/(x^2-1)")
# V_n = U_n - U_{n-1}, W_n = U_n + U_{n-1}
_poly("special_chebyshev_polynomial_v", _S.chebyshev_polynomial_v, lambda x, n, o: _cheb_u_d(x, n) - _cheb_u_d(x, n - 1),
      "d(V_n)/dx=U_n'-U_{n-1}'")
_poly("special_chebyshev_polynomial_w", _S.chebyshev_polynomial_w, lambda x, n, o: _cheb_u_d(x, n) + _cheb_u_d(x, n - 1),
      "d(W_n)/dx=U_n'+U_{n-1}'")
# shifted families: P*_n(x) = P_n(2x - 1), so the derivative carries a factor 2
_poly("special_shifted_chebyshev_polynomial_t", _S.shifted_chebyshev_polynomial_t, lambda x, n, o: 2 * _cheb_t_d(2 * x - 1, n),
      "d(T*_n(x))/dx=2*T_n'(2x-1)")
_poly("special_shifted_chebyshev_polynomial_u", _S.shifted_chebyshev_polynomial_u, lambda x, n, o: 2 * _cheb_u_d(2 * x - 1, n),
      "d(U*_n(x))/dx=2*U_n'(2x-1)")
_poly("special_shifted_chebyshev_polynomial_v", _S.shifted_chebyshev_polynomial_v,
      lambda x, n, o: 2 * (_cheb_u_d(2 * x - 1, n) - _cheb_u_d(2 * x - 1, n - 1)), "d(V*_n(x))/dx=2*V_n'(2x-1)")
_poly("special_shifted_chebyshev_polynomial_w", _S.shifted_chebyshev_polynomial_w,
      lambda x, n, o: 2 * (_cheb_u_d(2 * x - 1, n) + _cheb_u_d(2 * x - 1, n - 1)), "d(W*_n(x))/dx=2*W_n'(2x-1)")

_bin("clamp_min_tensor", torch.maximum, lambda g, a, b, o: g * (a >= b), lambda g, a, b, o: g * (a < b),
     "d(max(x,lo))/dx=1(x>=lo); dlo=1(x<lo)")
_bin("clamp_max_tensor", torch.minimum, lambda g, a, b, o: g * (a <= b), lambda g, a, b, o: g * (a > b),
     "d(min(x,hi))/dx=1(x<=hi); dhi=1(x>hi)")


def _vecdot_vjp(g, i, o, kw):
    a, b = i
    ge = g.unsqueeze(int(kw.get("dim", -1)))
    return [unbroadcast(ge * b, a.shape), unbroadcast(ge * a, b.shape)]


_reg("vecdot", lambda a, b, dim=-1: torch.linalg.vecdot(a, b, dim=int(dim)), _vecdot_vjp, "d(sum_k a_k*b_k)/da=grad*b; db=grad*a (real)")
_nograd("any", lambda x, dim=None, keepdim=False: torch.any(x != 0) if dim is None else torch.any(x != 0, dim=int(dim), keepdim=keepdim))
_nograd("all", lambda x, dim=None, keepdim=False: torch.all(x != 0) if dim is None else torch.all(x != 0, dim=int(dim), keepdim=keepdim))
_reg("roll_flat", lambda x, shift=1: torch.roll(x, int(shift)), lambda g, i, o, kw: [torch.roll(g, -int(kw.get("shift", 1)))],
     "d(roll of the flattened tensor)/dx=roll(grad,-shift)")
_reg("frobenius_norm", lambda x: torch.linalg.vector_norm(x, 2.0),
     lambda g, i, o, kw: [g * i[0] / torch.where(o == 0, torch.ones_like(o), o)], "d(||x||_F)/dx=x/||x||_F")


def _tensorinv_vjp(g, i, o, kw):
    x, ind = i[0], int(kw.get("ind", 2))
    n = 1
    for d in x.shape[:ind]:
        n *= d
    y = o.reshape(n, n)            # inverse of the flattened square matrix
    ga = -(y.mT @ g.reshape(n, n) @ y.mT)
    return [ga.reshape(x.shape)]


_reg("linalg_tensorinv", lambda x, ind=2: torch.linalg.tensorinv(x, ind=int(ind)), _tensorinv_vjp,
     "tensorinv = inverse of the matrix flattened at ind: dA=-A^-T@grad@A^-T, reshaped")


def _irfftn_fwd(z, s=None, dim=None, norm=None):
    return torch.fft.irfftn(_cplx(z), s=s, dim=dim, norm=norm)


def _irfftn_vjp(g, i, o, kw):
    z = i[0]
    dims = _fft_dims(z.dim() - 1, kw.get("s"), kw.get("dim"))
    n_total = 1
    for d in dims:
        n_total *= g.shape[d]
    n_last = g.shape[dims[-1]]
    m = n_last // 2 + 1
    w = torch.full((m,), 2.0, dtype=g.dtype, device=g.device)
    w[0] = 1.0
    if n_last % 2 == 0:
        w[-1] = 1.0
    shape = [1] * g.dim()
    shape[dims[-1]] = m
    gz = torch.fft.rfftn(g, dim=dims) * w.reshape(shape) * _norm_scale(kw.get("norm"), n_total, True)
    return [torch.view_as_real(_fit(gz, z.shape[:-1])).contiguous()]


_reg("irfftn", _irfftn_fwd, _irfftn_vjp, "d(irfftn(z))/dz_k=c*w_k*rfftn(grad)_k, w=1 at DC and Nyquist of the last dimension else 2")


def _ihfft_fwd(x, n=None, dim=-1, norm=None):
    return torch.view_as_real(torch.fft.ihfft(x, n=n, dim=int(dim), norm=norm).resolve_conj()).contiguous()


def _ihfft_vjp(g, i, o, kw):
    # ihfft(x) = conj(rfft(x)) / n (under the default norm): linear in the real input
    x, dim = i[0], int(kw.get("dim", -1)) % i[0].dim()
    n = x.shape[dim] if kw.get("n") is None else int(kw["n"])
    gc = torch.conj(_cplx(g))
    full = list(gc.shape)
    full[dim] = n
    scale = {"forward": 1.0, "ortho": 1.0 / math.sqrt(n)}.get(kw.get("norm"), 1.0 / n)
    dx = torch.fft.ifft(_fit(gc, full), dim=dim).real * (n * scale)
    return [_fit(dx, x.shape)]


_reg("ihfft", _ihfft_fwd, _ihfft_vjp, "ihfft(x)=conj(rfft(x))*c: dx=n*c*Re(ifft(zero-extended conj(grad)))")
