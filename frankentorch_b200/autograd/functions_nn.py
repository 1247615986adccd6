"""VJP rules, part 3: neural-network functionals, losses, linalg / FFT / misc long tail.

Fused CPU formulas follow the reference kernels: Linear (ft-kernel-cpu/src/lib.rs:17162, bwd
:17226), LayerNorm (:5824 / :6052), RMSNorm (:6418 / :6503: dx = rstd*g - rstd^3*c/N*x),
cross-entropy (:6649 / :6679), SDPA with recomputed probabilities (:4572 / :5300).  The rest
of the long tail differentiates a re-run of the single node (``local_vjp``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from .functions import OPS, OpDef, _reg, local_vjp, unbroadcast


# ---------------------------------------------------------------------------------- linear
def _linear_fwd(x, w, b=None):
    return TF.linear(x, w, b)


def _linear_vjp(g, i, o, kw):
    x, w = i[0], i[1]
    g2, x2 = g.reshape(-1, g.shape[-1]), x.reshape(-1, x.shape[-1])
    out = [(g2 @ w).reshape(x.shape), g2.t() @ x2]          # dx = dy.W ; dW = dy^T.x
    if len(i) > 2:
        out.append(g2.sum(0))                                 # db = row sum
    return out


_reg("linear", _linear_fwd, _linear_vjp, "d(A@B)/dA=dOut@B^T; d(A@B)/dB=A^T@dOut [+bias]")


# ---------------------------------------------------------------------------------- layer norm / rms norm
def _ln_fwd(x, w=None, b=None, eps=1e-5, ndim=1):
    return TF.layer_norm(x, x.shape[-ndim:], w, b, eps)


def _ln_vjp(g, i, o, kw):
    x = i[0]
    w = i[1] if len(i) > 1 else None
    nd, eps = kw.get("ndim", 1), kw.get("eps", 1e-5)
    dims = tuple(range(x.dim() - nd, x.dim()))
    mean = x.mean(dims, keepdim=True)
    rstd = torch.rsqrt(((x - mean) ** 2).mean(dims, keepdim=True) + eps)
    xhat = (x - mean) * rstd
    gw = g * w if w is not None else g
    dx = rstd * (gw - gw.mean(dims, keepdim=True) - xhat * (gw * xhat).mean(dims, keepdim=True))
    out = [dx]
    red = tuple(range(x.dim() - nd))
    if len(i) > 1:
        out.append((g * xhat).sum(red))
    if len(i) > 2:
        out.append(g.sum(red))
    return out


_reg("layer_norm", _ln_fwd, _ln_vjp, "d(layer_norm(x))/dx,dgamma,dbeta")


def _rms_fwd(x, w=None, eps=1e-6):
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * w if w is not None else y


def _rms_vjp(g, i, o, kw):
    x = i[0]
    w = i[1] if len(i) > 1 else None
    n = x.shape[-1]
    rstd = torch.rsqrt((x * x).mean(-1, keepdim=True) + kw.get("eps", 1e-6))
    gw = g * w if w is not None else g
    c = (gw * x).sum(-1, keepdim=True)
    out = [rstd * gw - rstd ** 3 * c / n * x]
    if w is not None:
        out.append((g * x * rstd).reshape(-1, n).sum(0))
    return out


_reg("rms_norm", _rms_fwd, _rms_vjp, "d(rms_norm(x))/dx,dgamma")


# ---------------------------------------------------------------------------------- attention
def _sdpa_fwd(q, k, v, mask=None, is_causal=False, scale=None):
    return TF.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=is_causal, scale=scale)


def _sdpa_vjp(g, i, o, kw):
    q, k, v = i[0], i[1], i[2]
    mask = i[3] if len(i) > 3 else None
    scale = kw.get("scale") or 1.0 / math.sqrt(q.shape[-1])
    s = (q @ k.transpose(-1, -2)) * scale
    if kw.get("is_causal", False):
        S, T = s.shape[-2], s.shape[-1]
        s = s.masked_fill(torch.triu(torch.ones(S, T, dtype=torch.bool), 1), float("-inf"))
    if mask is not None:
        s = s + mask if mask.dtype != torch.bool else s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)                      # recompute P
    dv = p.transpose(-1, -2) @ g                  # dV = P^T dO
    dp = g @ v.transpose(-1, -2)                  # dP = dO V^T
    du = p * (dp - (p * dp).sum(-1, keepdim=True))
    out = [scale * du @ k, scale * du.transpose(-1, -2) @ q, dv]
    if mask is not None:
        out.append(None)
    return out


_reg("sdpa", _sdpa_fwd, _sdpa_vjp, "d(sdpa(q,k,v))/dq,dk,dv [recompute P]")


# ---------------------------------------------------------------------------------- losses
def _ce_fwd(logits, target, reduction="mean"):
    return TF.cross_entropy(logits, target.long(), reduction=reduction)


def _ce_vjp(g, i, o, kw):
    x, t = i[0], i[1].long()
    sm = torch.softmax(x, -1)
    onehot = torch.zeros_like(sm).scatter_(-1, t.unsqueeze(-1), 1.0)
    red = kw.get("reduction", "mean")
    if red == "mean":
        return [g * (sm - onehot) / x.shape[0], None]
    if red == "sum":
        return [g * (sm - onehot), None]
    return [g.unsqueeze(-1) * (sm - onehot), None]


_reg("cross_entropy", _ce_fwd, _ce_vjp, "d(cross_entropy)/dlogits=g*(softmax-onehot)")


def _mse_vjp(g, i, o, kw):
    d = i[0] - i[1]
    red = kw.get("reduction", "mean")
    s = 2.0 / d.numel() if red == "mean" else 2.0
    return [g * s * d, -g * s * d]


_reg("mse_loss", lambda a, b, reduction="mean": TF.mse_loss(a, b, reduction=reduction), _mse_vjp,
     "d(mse(p,t))/dp=2(p-t)/n")


def _l1_vjp(g, i, o, kw):
    d = torch.sign(i[0] - i[1])
    s = 1.0 / d.numel() if kw.get("reduction", "mean") == "mean" else 1.0
    return [g * s * d, -g * s * d]


_reg("l1_loss", lambda a, b, reduction="mean": TF.l1_loss(a, b, reduction=reduction), _l1_vjp,
     "d(l1(p,t))/dp=sign(p-t)/n")


def _generic(name, fwd, rule=None):
    OPS[name] = OpDef(name, fwd, local_vjp(fwd), rule or f"d({name})/d_inputs [single-node differentiation]")


_generic("nll_loss", lambda lp, t, reduction="mean": TF.nll_loss(lp, t.long(), reduction=reduction))
_generic("bce_loss", lambda p, t, reduction="mean": TF.binary_cross_entropy(p, t, reduction=reduction))
_generic("bce_with_logits_loss", lambda x, t, reduction="mean": TF.binary_cross_entropy_with_logits(x, t, reduction=reduction))
_generic("smooth_l1_loss", lambda a, b, beta=1.0, reduction="mean": TF.smooth_l1_loss(a, b, beta=beta, reduction=reduction))
_generic("huber_loss", lambda a, b, delta=1.0, reduction="mean": TF.huber_loss(a, b, delta=delta, reduction=reduction))
_generic("kl_div", lambda a, b, reduction="batchmean", log_target=False: TF.kl_div(a, b, reduction=reduction, log_target=log_target))
_generic("cosine_embedding_loss", lambda a, b, y, margin=0.0: TF.cosine_embedding_loss(a, b, y, margin=margin))
_generic("triplet_margin_loss", lambda a, p, n, margin=1.0: TF.triplet_margin_loss(a, p, n, margin=margin))
_generic("multi_margin_loss", lambda x, t, margin=1.0: TF.multi_margin_loss(x, t.long(), margin=margin))
_generic("gaussian_nll_loss", lambda x, t, var, eps=1e-6: TF.gaussian_nll_loss(x, t, var, eps=eps))
_generic("poisson_nll_loss", lambda x, t, log_input=True: TF.poisson_nll_loss(x, t, log_input=log_input))
_generic("hinge_embedding_loss", lambda x, y, margin=1.0: TF.hinge_embedding_loss(x, y, margin=margin))
_generic("soft_margin_loss", lambda x, y: TF.soft_margin_loss(x, y))
_generic("margin_ranking_loss", lambda a, b, y, margin=0.0: TF.margin_ranking_loss(a, b, y, margin=margin))
_generic("ctc_loss", lambda lp, t, il, tl, blank=0, reduction="mean", zero_infinity=False:
         TF.ctc_loss(lp, t.long(), il.long(), tl.long(), blank=blank, reduction=reduction, zero_infinity=zero_infinity))


def _focal(x, t, alpha=0.25, gamma=2.0):
    p = torch.sigmoid(x)
    ce = TF.binary_cross_entropy_with_logits(x, t, reduction="none")
    pt = p * t + (1 - p) * (1 - t)
    return ((alpha * t + (1 - alpha) * (1 - t)) * (1 - pt) ** gamma * ce).mean()


def _dice(p, t, eps=1.0):
    inter = (p * t).sum()
    return 1 - (2 * inter + eps) / (p.sum() + t.sum() + eps)


_generic("focal_loss", _focal)
_generic("dice_loss", _dice)

# ---------------------------------------------------------------------------------- conv / pool / misc nn
_generic("conv1d", lambda x, w, b=None, stride=1, padding=0, dilation=1, groups=1: TF.conv1d(x, w, b, stride, padding, dilation, groups))
_generic("conv2d", lambda x, w, b=None, stride=1, padding=0, dilation=1, groups=1: TF.conv2d(x, w, b, stride, padding, dilation, groups))
_generic("conv3d", lambda x, w, b=None, stride=1, padding=0, dilation=1, groups=1: TF.conv3d(x, w, b, stride, padding, dilation, groups))
_generic("conv_transpose1d", lambda x, w, b=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1: TF.conv_transpose1d(x, w, b, stride, padding, output_padding, groups, dilation))
_generic("conv_transpose2d", lambda x, w, b=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1: TF.conv_transpose2d(x, w, b, stride, padding, output_padding, groups, dilation))
_generic("conv_transpose3d", lambda x, w, b=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1: TF.conv_transpose3d(x, w, b, stride, padding, output_padding, groups, dilation))
for _d in (1, 2, 3):
    _generic(f"avg_pool{_d}d", (lambda f: (lambda x, kernel_size=2, stride=None, padding=0, ceil_mode=False, count_include_pad=True:
                                           f(x, kernel_size, stride, padding, ceil_mode, count_include_pad)))(getattr(TF, f"avg_pool{_d}d")))
    _generic(f"max_pool{_d}d", (lambda f: (lambda x, kernel_size=2, stride=None, padding=0, dilation=1, ceil_mode=False:
                                           f(x, kernel_size, stride, padding, dilation, ceil_mode)))(getattr(TF, f"max_pool{_d}d")))
    _generic(f"adaptive_avg_pool{_d}d", (lambda f: (lambda x, output_size=1: f(x, output_size)))(getattr(TF, f"adaptive_avg_pool{_d}d")))
    _generic(f"adaptive_max_pool{_d}d", (lambda f: (lambda x, output_size=1: f(x, output_size)))(getattr(TF, f"adaptive_max_pool{_d}d")))
_generic("lp_pool1d", lambda x, norm_type=2.0, kernel_size=2: TF.lp_pool1d(x, norm_type, kernel_size))
_generic("lp_pool2d", lambda x, norm_type=2.0, kernel_size=2: TF.lp_pool2d(x, norm_type, kernel_size))
_generic("group_norm", lambda x, w=None, b=None, groups=1, eps=1e-5: TF.group_norm(x, groups, w, b, eps))
_generic("batch_norm", lambda x, w=None, b=None, eps=1e-5: TF.batch_norm(x, None, None, w, b, True, 0.0, eps))
_generic("instance_norm", lambda x, w=None, b=None, eps=1e-5: TF.instance_norm(x, None, None, w, b, True, 0.0, eps))
_generic("local_response_norm", lambda x, size=5, alpha=1e-4, beta=0.75, k=1.0: TF.local_response_norm(x, size, alpha, beta, k))
_generic("interpolate", lambda x, size=None, scale_factor=None, mode="nearest", align_corners=None:
         TF.interpolate(x, size=size, scale_factor=scale_factor, mode=mode, align_corners=align_corners))
_generic("grid_sample", lambda x, grid, mode="bilinear", padding_mode="zeros", align_corners=False: TF.grid_sample(x, grid, mode=mode, padding_mode=padding_mode, align_corners=align_corners))
_generic("affine_grid", lambda theta, size=(), align_corners=False: TF.affine_grid(theta, list(size), align_corners=align_corners))
_generic("pixel_shuffle", lambda x, r=2: TF.pixel_shuffle(x, r))
_generic("pixel_unshuffle", lambda x, r=2: TF.pixel_unshuffle(x, r))
_generic("unfold", lambda x, kernel_size=1, dilation=1, padding=0, stride=1: TF.unfold(x, kernel_size, dilation, padding, stride))
_generic("fold", lambda x, output_size=(), kernel_size=1, dilation=1, padding=0, stride=1: TF.fold(x, output_size, kernel_size, dilation, padding, stride))
_generic("pad_mode", lambda x, padding=(), mode="reflect": TF.pad(x, list(padding), mode=mode))
_generic("embedding_bag", lambda w, ids, offsets, mode="mean": TF.embedding_bag(ids.long(), w, offsets.long(), mode=mode))
_generic("bilinear", lambda a, b, w, bias=None: TF.bilinear(a, b, w, bias))
_generic("cosine_similarity", lambda a, b, dim=1, eps=1e-8: TF.cosine_similarity(a, b, dim, eps))
_generic("pairwise_distance", lambda a, b, p=2.0, eps=1e-6, keepdim=False: TF.pairwise_distance(a, b, p, eps, keepdim))
_generic("cdist", lambda a, b, p=2.0: torch.cdist(a, b, p))
_generic("pdist", lambda a, p=2.0: TF.pdist(a, p))
_generic("glu", lambda x, dim=-1: TF.glu(x, dim))
_generic("swiglu", lambda x, dim=-1: (lambda a, b: TF.silu(a) * b)(*x.chunk(2, dim)))
_generic("geglu", lambda x, dim=-1: (lambda a, b: TF.gelu(a) * b)(*x.chunk(2, dim)))
_generic("reglu", lambda x, dim=-1: (lambda a, b: torch.relu(a) * b)(*x.chunk(2, dim)))
for _n in ("selu", "celu", "relu6", "hardtanh", "hardswish", "hardsigmoid", "logsigmoid", "softsign", "tanhshrink",
           "softshrink", "hardshrink", "softmin", "threshold", "prelu", "rrelu"):
    if _n == "softmin":
        _generic(_n, lambda x, dim=-1: TF.softmin(x, dim))
    elif _n == "threshold":
        _generic(_n, lambda x, threshold=0.0, value=0.0: TF.threshold(x, threshold, value))
    elif _n == "prelu":
        _generic(_n, lambda x, w: TF.prelu(x, w))
    elif _n == "rrelu":
        _generic(_n, lambda x, lower=1.0 / 8, upper=1.0 / 3: TF.rrelu(x, lower, upper, False))
    else:
        _generic(_n, getattr(TF, _n))


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], -1)
    return x * cos + rot * sin


_generic("rotary_pos_emb", _rope)

# ---------------------------------------------------------------------------------- linalg / fft / special
for _n in ("det", "inv", "pinv", "cholesky", "matrix_exp", "slogdet_abs"):
    pass
_generic("linalg_det", torch.linalg.det)
_generic("linalg_inv", torch.linalg.inv)
_generic("linalg_pinv", torch.linalg.pinv)
_generic("linalg_cholesky", torch.linalg.cholesky)
_generic("linalg_matrix_exp", torch.linalg.matrix_exp)
_generic("linalg_logdet", torch.logdet)
_generic("linalg_solve", torch.linalg.solve)
_generic("linalg_triangular_solve", lambda a, b, upper=True: torch.linalg.solve_triangular(a, b, upper=upper))
_generic("linalg_lstsq", lambda a, b: torch.linalg.lstsq(a, b).solution)
_generic("linalg_eigvalsh", torch.linalg.eigvalsh)
_generic("linalg_svdvals", torch.linalg.svdvals)
_generic("linalg_matrix_norm", lambda x, ord="fro": torch.linalg.matrix_norm(x, ord))
_generic("linalg_cond", lambda x: torch.linalg.cond(x))
_generic("linalg_qr_r", lambda x: torch.linalg.qr(x).R)
_generic("linalg_qr_q", lambda x: torch.linalg.qr(x).Q)
_generic("linalg_eigh_vectors", lambda x: torch.linalg.eigh(x).eigenvectors)
_generic("einsum", lambda *xs, equation="": torch.einsum(equation, *xs))
_generic("tensordot", lambda a, b, dims=2: torch.tensordot(a, b, dims))
_generic("kron", torch.kron)
_generic("cross", lambda a, b, dim=-1: torch.linalg.cross(a, b, dim=dim))
_generic("inner", torch.inner)
_generic("mv", torch.mv)
_generic("baddbmm", lambda inp, a, b, beta=1.0, alpha=1.0: torch.baddbmm(inp, a, b, beta=beta, alpha=alpha))
_generic("addbmm", lambda inp, a, b, beta=1.0, alpha=1.0: torch.addbmm(inp, a, b, beta=beta, alpha=alpha))
_generic("fft_real", lambda x, n=None, dim=-1: torch.view_as_real(torch.fft.fft(x, n, dim)))
_generic("rfft_real", lambda x, n=None, dim=-1: torch.view_as_real(torch.fft.rfft(x, n, dim)))
_generic("irfft", lambda x, n=None, dim=-1: torch.fft.irfft(torch.view_as_complex(x.contiguous()), n, dim))
_generic("special_digamma", torch.special.digamma)
_generic("special_lgamma", torch.lgamma)
_generic("special_erfc", torch.special.erfc)
_generic("special_erfinv", torch.special.erfinv)
_generic("special_i0", torch.special.i0)
_generic("special_xlogy", torch.special.xlogy)
_generic("special_logit", lambda x, eps=None: torch.special.logit(x, eps))
_generic("special_sinc", torch.special.sinc)
_generic("special_expit", torch.special.expit)
_generic("diagonal", lambda x, offset=0, dim1=0, dim2=1: torch.diagonal(x, offset, dim1, dim2).contiguous())
_generic("movedim", lambda x, source=0, destination=0: torch.movedim(x, source, destination).contiguous())
_generic("unfold_dim", lambda x, dim=0, size=1, step=1: x.unfold(dim, size, step).contiguous())
_generic("index_put", lambda x, idx, vals, accumulate=False: x.index_put((idx.long(),), vals, accumulate=accumulate))
_generic("masked_select", lambda x, mask: torch.masked_select(x, mask.bool()))
_generic("median", lambda x: x.median())
_generic("quantile", lambda x, q=0.5: torch.quantile(x, q))
_generic("cummax", lambda x, dim=0: torch.cummax(x, dim).values)
_generic("cummin", lambda x, dim=0: torch.cummin(x, dim).values)
_generic("cov", lambda x: torch.cov(x))
_generic("corrcoef", lambda x: torch.corrcoef(x))
