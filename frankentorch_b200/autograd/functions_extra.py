"""Operators added after the core rule tables: complex-valued FFTs, full linalg factorisations,
fake quantisation, complex views, box / point-cloud utilities and box losses.

Complex tensors are carried on the tape as real tensors with a trailing dimension of 2
(``view_as_real`` layout), because tape values, the gradient space and the serialisers are
real-typed; every operator below converts at its boundary.  The reference exposes the same
families on its session (``tensor_fft/ifft/rfft/fft2/fftn/stft/istft``, ``tensor_linalg_*`` with
gradients, ``tensor_quantize_per_tensor/channel``, ``tensor_complex/real/imag/view_as_*``, ``nms``,
``roi_pool``, ``ball_query``, ``farthest_point_sampling``; FEATURE_PARITY.md and
crates/ft-kernel-cpu/src/lib.rs families "linalg", "fft", "vision").
"""
from __future__ import annotations

import torch

from .functions import OPS, OpDef, local_vjp


def _generic(name, fwd, rule=None):
    OPS[name] = OpDef(name, fwd, local_vjp(fwd), rule or f"d({name})/d_inputs [single-node differentiation]")


def _nograd(name, fwd, rule=None):
    OPS[name] = OpDef(name, fwd, None, rule or f"{name}: piecewise constant, no gradient")


def _c(x):       # real [..., 2] -> complex
    return torch.view_as_complex(x.contiguous())


def _r(z):       # complex -> real [..., 2]
    return torch.view_as_real(z).contiguous()


def _dim_c(dim, ndim_c):
    """Dimension index of the complex tensor for an index given on the complex shape."""
    return dim if dim >= 0 else dim + ndim_c


# ------------------------------------------------------------------------------------- complex
_generic("complex", lambda re, im: torch.stack([re, im], -1), "d(complex(re,im)) = (g[...,0], g[...,1])")
_generic("real", lambda z: z[..., 0].contiguous(), "d(real(z))/dz = (g, 0)")
_generic("imag", lambda z: z[..., 1].contiguous(), "d(imag(z))/dz = (0, g)")
_generic("view_as_real", lambda z: z.contiguous(), "identity on the [...,2] layout")
_generic("view_as_complex", lambda x: x.contiguous(), "identity on the [...,2] layout")
_generic("complex_mul", lambda a, b: _r(_c(a) * _c(b)), "d(ab) = (g conj(b), g conj(a))")
_generic("complex_conj", lambda z: torch.stack([z[..., 0], -z[..., 1]], -1), "d(conj z) = conj(g)")
_generic("complex_abs", lambda z: torch.sqrt(z[..., 0] ** 2 + z[..., 1] ** 2), "d|z| = g z / |z|")
_generic("complex_angle", lambda z: torch.atan2(z[..., 1], z[..., 0]), "d(arg z) = g (-im, re) / |z|^2")

# ------------------------------------------------------------------------------------- fft
# inputs: real tensors ("fft" of a real signal) or [...,2] complex layout (flag complex_input)


def _as_c(x, complex_input):
    return _c(x) if complex_input else x


_generic("fft", lambda x, n=None, dim=-1, norm=None, complex_input=False:
         _r(torch.fft.fft(_as_c(x, complex_input), n, dim, norm)))
_generic("ifft", lambda x, n=None, dim=-1, norm=None, complex_input=True:
         _r(torch.fft.ifft(_as_c(x, complex_input), n, dim, norm)))
_generic("rfft", lambda x, n=None, dim=-1, norm=None: _r(torch.fft.rfft(x, n, dim, norm)))
_generic("fft2", lambda x, norm=None, complex_input=False:
         _r(torch.fft.fft2(_as_c(x, complex_input), norm=norm)))
_generic("ifft2", lambda x, norm=None, complex_input=True:
         _r(torch.fft.ifft2(_as_c(x, complex_input), norm=norm)))
_generic("fftn", lambda x, norm=None, complex_input=False:
         _r(torch.fft.fftn(_as_c(x, complex_input), norm=norm)))
_generic("ifftn", lambda x, norm=None, complex_input=True:
         _r(torch.fft.ifftn(_as_c(x, complex_input), norm=norm)))
_generic("hfft", lambda x, n=None, dim=-1: torch.fft.hfft(_c(x), n, dim))


def _stft(x, n_fft=16, hop_length=None, win_length=None, window=None, center=True, normalized=False,
          onesided=True):
    w = window if window is not None else torch.ones(win_length or n_fft, dtype=x.dtype, device=x.device)
    return _r(torch.stft(x, n_fft, hop_length, win_length, w, center=center, normalized=normalized,
                         onesided=onesided, return_complex=True))


def _istft(z, n_fft=16, hop_length=None, win_length=None, window=None, center=True, normalized=False,
           onesided=True, length=None):
    w = window if window is not None else torch.ones(win_length or n_fft, dtype=z.dtype, device=z.device)
    return torch.istft(_c(z), n_fft, hop_length, win_length, w, center=center, normalized=normalized,
                       onesided=onesided, length=length)


OPS["stft"] = OpDef("stft", _stft, local_vjp(_stft), "d(stft)/dx [frames x window x DFT, single-node differentiation]")
OPS["istft"] = OpDef("istft", _istft, local_vjp(_istft), "d(istft)/dz [overlap-add inverse, single-node differentiation]")

# ------------------------------------------------------------------------------------- linalg
_generic("linalg_svd_u", lambda x: torch.linalg.svd(x, full_matrices=False).U)
_generic("linalg_svd_vh", lambda x: torch.linalg.svd(x, full_matrices=False).Vh)
_generic("linalg_eigh_values", lambda x: torch.linalg.eigh(x).eigenvalues)
_generic("linalg_eig_values", lambda x: _r(torch.linalg.eig(x).eigenvalues))
_generic("linalg_eig_vectors", lambda x: _r(torch.linalg.eig(x).eigenvectors))
_generic("linalg_eigvals", lambda x: _r(torch.linalg.eigvals(x)))
_generic("linalg_slogdet_logabs", lambda x: torch.linalg.slogdet(x).logabsdet)
_nograd("linalg_slogdet_sign", lambda x: torch.linalg.slogdet(x).sign)
_generic("linalg_matrix_power", lambda x, n=2: torch.linalg.matrix_power(x, n))
_generic("linalg_vector_norm", lambda x, ord=2.0: torch.linalg.vector_norm(x, ord))
_generic("linalg_lu_l", lambda x: torch.linalg.lu(x).L)
_generic("linalg_lu_u", lambda x: torch.linalg.lu(x).U)
_nograd("linalg_lu_p", lambda x: torch.linalg.lu(x).P)
_nograd("linalg_matrix_rank", lambda x: torch.linalg.matrix_rank(x).to(x.dtype))
_generic("linalg_cholesky_solve", lambda b, l, upper=False: torch.cholesky_solve(b, l, upper=upper))
_generic("linalg_householder_product", lambda v, tau: torch.linalg.householder_product(v, tau))
_generic("linalg_multi_dot", lambda *xs: torch.linalg.multi_dot(list(xs)))


# ------------------------------------------------------------------------------------- quantisation
def _qrange(bits, signed):
    return (-(1 << (bits - 1)), (1 << (bits - 1)) - 1) if signed else (0, (1 << bits) - 1)


def _fake_quant_tensor(x, scale=1.0, zero_point=0, bits=8, signed=True):
    lo, hi = _qrange(bits, signed)
    q = torch.clamp(torch.round(x / scale) + zero_point, lo, hi)
    return (q - zero_point) * scale


def _fake_quant_vjp(g, inputs, out, kw):
    # straight-through estimator inside the representable range, zero outside
    x = inputs[0]
    lo, hi = _qrange(kw.get("bits", 8), kw.get("signed", True))
    scale, zp = kw.get("scale", 1.0), kw.get("zero_point", 0)
    q = torch.round(x / scale) + zp
    return [g * ((q >= lo) & (q <= hi)).to(g.dtype)]


OPS["fake_quantize_per_tensor"] = OpDef("fake_quantize_per_tensor", _fake_quant_tensor, _fake_quant_vjp,
                                        "straight-through: g inside [qmin, qmax], 0 outside")


def _quantize_per_tensor(x, scale=1.0, zero_point=0, bits=8, signed=True):
    lo, hi = _qrange(bits, signed)
    return torch.clamp(torch.round(x / scale) + zero_point, lo, hi)


def _quantize_per_channel(x, scales, zero_points, axis=0, bits=8, signed=True):
    lo, hi = _qrange(bits, signed)
    shape = [1] * x.dim()
    shape[axis] = -1
    return torch.clamp(torch.round(x / scales.reshape(shape)) + zero_points.reshape(shape), lo, hi)


def _dequantize_per_channel(q, scales, zero_points, axis=0):
    shape = [1] * q.dim()
    shape[axis] = -1
    return (q - zero_points.reshape(shape)) * scales.reshape(shape)


_nograd("quantize_per_tensor", _quantize_per_tensor, "integer codes: round(x/scale)+zp clamped; no gradient")
_nograd("quantize_per_channel", _quantize_per_channel, "integer codes per channel; no gradient")
_generic("dequantize_per_tensor", lambda q, scale=1.0, zero_point=0: (q - zero_point) * scale)
_generic("dequantize_per_channel", _dequantize_per_channel)


# ------------------------------------------------------------------------------------- boxes
def box_area(b):
    return (b[..., 2] - b[..., 0]).clamp(min=0) * (b[..., 3] - b[..., 1]).clamp(min=0)


def _pair_iou(a, b):
    """IoU and union of boxes ``a[N,4]`` against ``b[M,4]`` (xyxy)."""
    lt = torch.maximum(a[:, None, :2], b[None, :, :2])
    rb = torch.minimum(a[:, None, 2:], b[None, :, 2:])
    wh = (rb - lt).clamp(min=0)
    inter = wh[..., 0] * wh[..., 1]
    union = box_area(a)[:, None] + box_area(b)[None, :] - inter
    return inter / union.clamp(min=torch.finfo(a.dtype).tiny), union


def _box_iou(a, b):
    return _pair_iou(a, b)[0]


def _generalized_box_iou(a, b):
    iou, union = _pair_iou(a, b)
    lt = torch.minimum(a[:, None, :2], b[None, :, :2])
    rb = torch.maximum(a[:, None, 2:], b[None, :, 2:])
    wh = (rb - lt).clamp(min=0)
    hull = wh[..., 0] * wh[..., 1]
    return iou - (hull - union) / hull.clamp(min=torch.finfo(a.dtype).tiny)


def _elementwise_iou(p, t):
    lt = torch.maximum(p[..., :2], t[..., :2])
    rb = torch.minimum(p[..., 2:], t[..., 2:])
    wh = (rb - lt).clamp(min=0)
    inter = wh[..., 0] * wh[..., 1]
    union = box_area(p) + box_area(t) - inter
    return inter, union


def _iou_loss(p, t, reduction="mean", eps=1e-7):
    inter, union = _elementwise_iou(p, t)
    loss = 1 - inter / (union + eps)
    return loss.mean() if reduction == "mean" else (loss.sum() if reduction == "sum" else loss)


def _giou_loss(p, t, reduction="mean", eps=1e-7):
    inter, union = _elementwise_iou(p, t)
    iou = inter / (union + eps)
    lt = torch.minimum(p[..., :2], t[..., :2])
    rb = torch.maximum(p[..., 2:], t[..., 2:])
    hull = (rb - lt).clamp(min=0).prod(-1)
    loss = 1 - (iou - (hull - union) / (hull + eps))
    return loss.mean() if reduction == "mean" else (loss.sum() if reduction == "sum" else loss)


_generic("box_iou", _box_iou)
_generic("generalized_box_iou", _generalized_box_iou)
_generic("iou_loss", _iou_loss, "d(1 - IoU)/d_boxes")
_generic("giou_loss", _giou_loss, "d(1 - GIoU)/d_boxes")


def nms_indices(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float) -> torch.Tensor:
    """Greedy non-maximum suppression; ties in score are broken by the lower index (stable sort), so
    the kept set is deterministic."""
    order = torch.sort(scores, descending=True, stable=True).indices.tolist()
    iou = _box_iou(boxes, boxes)
    keep, dead = [], set()
    for i in order:
        if i in dead:
            continue
        keep.append(i)
        over = (iou[i] > iou_threshold).nonzero().flatten().tolist()
        dead.update(over)
    return torch.tensor(keep, dtype=torch.int64, device=boxes.device)


def _roi_pool(feat, rois, output_size=(2, 2), spatial_scale=1.0):
    """Max pooling of regions ``rois[K,5] = (batch, x1, y1, x2, y2)`` of ``feat[N,C,H,W]`` to
    ``[K, C, oh, ow]`` with the usual rounding to whole cells; the gradient goes to the arg-max cell."""
    oh, ow = (output_size, output_size) if isinstance(output_size, int) else output_size
    N, C, H, W = feat.shape
    outs = []
    for k in range(rois.shape[0]):
        bi = int(rois[k, 0])
        x1, y1, x2, y2 = [int(round(float(v) * spatial_scale)) for v in rois[k, 1:5]]
        rw, rh = max(x2 - x1 + 1, 1), max(y2 - y1 + 1, 1)
        cells = []
        for i in range(oh):
            hs = min(max(y1 + (i * rh) // oh, 0), H)
            he = min(max(y1 + -((-(i + 1) * rh) // oh), 0), H)
            row = []
            for j in range(ow):
                ws = min(max(x1 + (j * rw) // ow, 0), W)
                we = min(max(x1 + -((-(j + 1) * rw) // ow), 0), W)
                if he <= hs or we <= ws:
                    row.append(feat.new_zeros(C))
                else:
                    row.append(feat[bi, :, hs:he, ws:we].amax((-1, -2)))
            cells.append(torch.stack(row, -1))
        outs.append(torch.stack(cells, -2))
    return torch.stack(outs, 0) if outs else feat.new_zeros((0, C, oh, ow))


OPS["roi_pool"] = OpDef("roi_pool", _roi_pool, None, "roi max pool: gradient to the arg-max cell")


def _roi_pool_vjp(g, inputs, out, kw):
    feat, rois = inputs
    x = feat.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        y = _roi_pool(x, rois, **kw)
    return [torch.autograd.grad(y, x, g.to(y.dtype))[0], None]


OPS["roi_pool"] = OpDef("roi_pool", _roi_pool, _roi_pool_vjp, "roi max pool: gradient to the arg-max cell")


def ball_query_indices(xyz: torch.Tensor, centers: torch.Tensor, radius: float, k: int) -> torch.Tensor:
    """For each centre the first ``k`` point indices (ascending index) within ``radius``; rows with
    fewer hits repeat their first hit, rows with none hold 0 (the PointNet++ convention).
    ``xyz[B,N,3]``, ``centers[B,M,3]`` -> ``[B,M,k]`` int64."""
    d2 = torch.cdist(centers, xyz) ** 2
    B, M, N = d2.shape
    inside = d2 <= radius * radius
    idx = torch.arange(N, device=xyz.device).expand(B, M, N).clone()
    idx[~inside] = N
    idx = torch.sort(idx, -1).values[..., :k]
    if idx.shape[-1] < k:
        idx = torch.cat([idx, idx.new_full((B, M, k - idx.shape[-1]), N)], -1)
    first = idx[..., :1].clone()
    first[first == N] = 0
    return torch.where(idx == N, first.expand_as(idx), idx)


def farthest_point_sampling_indices(xyz: torch.Tensor, m: int, start: int = 0) -> torch.Tensor:
    """Iterative farthest point sampling from index ``start``; ties pick the lowest index.
    ``xyz[B,N,3]`` -> ``[B,m]`` int64."""
    B, N, _ = xyz.shape
    out = torch.zeros((B, m), dtype=torch.int64, device=xyz.device)
    dist = torch.full((B, N), float("inf"), dtype=xyz.dtype, device=xyz.device)
    cur = torch.full((B,), start, dtype=torch.int64, device=xyz.device)
    ar = torch.arange(B, device=xyz.device)
    for i in range(m):
        out[:, i] = cur
        d = ((xyz - xyz[ar, cur][:, None, :]) ** 2).sum(-1)
        dist = torch.minimum(dist, d)
        cur = torch.argmax(dist, -1)       # argmax returns the first maximal index
    return out


# ------------------------------------------------------------------------------------- norms
_generic("batch_norm_eval", lambda x, mean, var, w=None, b=None, eps=1e-5:
         torch.nn.functional.batch_norm(x, mean, var, w, b, False, 0.0, eps),
         "d(batch_norm with fixed statistics)/dx,dw,db")

# ------------------------------------------------------------------------------------- pooling
def _fractional_max_pool2d(x, kernel_size=2, output_size=None, output_ratio=None, samples=None):
    """Fractional max pooling with caller-supplied ``samples[N,C,2]`` in [0,1) (deterministic)."""
    if samples is None:
        samples = torch.full((x.shape[0], x.shape[1], 2), 0.5, dtype=x.dtype, device=x.device)
    return torch.nn.functional.fractional_max_pool2d(x, kernel_size, output_size, output_ratio,
                                                     _random_samples=samples)


_generic("fractional_max_pool2d", _fractional_max_pool2d, "max pool over pseudo-random windows: gradient to the arg-max")
_nograd("max_pool2d_indices", lambda x, kernel_size=2, stride=None, padding=0:
        torch.nn.functional.max_pool2d(x, kernel_size, stride, padding, return_indices=True)[1].to(torch.float64),
        "flat arg-max positions of max_pool2d; no gradient")
_generic("max_unpool1d", lambda x, indices, kernel_size=2, stride=None, padding=0, output_size=None:
         torch.nn.functional.max_unpool1d(x, indices.long(), kernel_size, stride, padding, output_size),
         "d(max_unpool)/dx = gather of g at the indices")
_generic("max_unpool3d", lambda x, indices, kernel_size=2, stride=None, padding=0, output_size=None:
         torch.nn.functional.max_unpool3d(x, indices.long(), kernel_size, stride, padding, output_size),
         "d(max_unpool)/dx = gather of g at the indices")
_nograd("max_pool1d_indices", lambda x, kernel_size=2, stride=None, padding=0:
        torch.nn.functional.max_pool1d(x, kernel_size, stride, padding, return_indices=True)[1].to(torch.float64),
        "flat arg-max positions of max_pool1d; no gradient")
_nograd("max_pool3d_indices", lambda x, kernel_size=2, stride=None, padding=0:
        torch.nn.functional.max_pool3d(x, kernel_size, stride, padding, return_indices=True)[1].to(torch.float64),
        "flat arg-max positions of max_pool3d; no gradient")


def _fractional_max_pool3d(x, kernel_size=2, output_size=None, output_ratio=None, samples=None):
    """Fractional max pooling over volumes with caller-supplied ``samples[N,C,3]`` in [0,1) (deterministic)."""
    if samples is None:
        samples = torch.full((x.shape[0], x.shape[1], 3), 0.5, dtype=x.dtype, device=x.device)
    return torch.nn.functional.fractional_max_pool3d(x, kernel_size, output_size, output_ratio,
                                                     _random_samples=samples)


_generic("fractional_max_pool3d", _fractional_max_pool3d, "max pool over pseudo-random windows: gradient to the arg-max")
_generic("lp_pool3d", lambda x, norm_type=2.0, kernel_size=2, stride=None:
         torch.nn.functional.lp_pool3d(x, norm_type, kernel_size, stride),
         "d((sum |x|^p)^(1/p))/dx over each window")
_generic("multilabel_margin_loss", lambda x, t, reduction="mean":
         torch.nn.functional.multilabel_margin_loss(x, t.long(), reduction=reduction),
         "d(sum_j sum_i max(0, 1 - (x[y_j] - x_i)) / C)/dx")
_generic("multilabel_soft_margin_loss", lambda x, t, reduction="mean":
         torch.nn.functional.multilabel_soft_margin_loss(x, t, reduction=reduction),
         "d(-mean_c [y log sigmoid(x) + (1-y) log sigmoid(-x)])/dx")
_generic("max_unpool2d", lambda x, indices, kernel_size=2, stride=None, padding=0, output_size=None:
         torch.nn.functional.max_unpool2d(x, indices.long(), kernel_size, stride, padding, output_size),
         "d(max_unpool)/dx = gather of g at the indices")
