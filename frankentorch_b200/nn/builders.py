"""Builder-style constructors and named forwards of the reference's modules.

The reference configures a module with chained ``with_*`` calls and names the forward of a multi-input module
after its inputs (``forward_pair``, ``forward_with_var`` ...).  The modules here take keyword arguments and have
one ``forward``; this file adds the reference's spellings on top of them, so code written against either reads
the same.  Reference: ft-nn/src/lib.rs - ``LocalResponseNorm::with_params`` :2227, ``Embedding::with_options``
:2916, ``EmbeddingBag::forward_with_offsets`` :3244, ``Conv1d / Conv2d::new_grouped`` :4114 / :7406,
``MaxPool2d::ceil_mode`` :7785, ``MaxUnpool1d / 2d::forward_with_indices`` :9281 / :9400, ``Upsample`` builders
:10265-10330, ``UpsamplingNearest2d / Bilinear2d`` :10528-10600, ``Bilinear::forward_bilinear`` :1260,
``CosineEmbeddingLoss / MarginRankingLoss::forward_triplet`` :15775 / :15840, ``HingeEmbeddingLoss::forward_hinge``
:16033, ``GaussianNLLLoss::forward_with_var`` :16128, ``CTCLoss`` builders and ``forward_ctc`` :16198-16222,
``CosineSimilarity / PairwiseDistance`` builders and ``forward_pair`` :18878-18984, ``MinMaxObserver::compute_qparams``
:20161.

A ``with_*`` call returns the module itself after setting the field (the reference consumes and returns the
value; the effect for a caller that keeps the result is the same).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import extra as _x
from . import layers as _l
from . import transformer as _t
from . import utils as _u
from .enums import CTCReduction, UpsampleMode


def _setter(field: str, conv=lambda v: v, into_kw: bool = False):
    def with_(self, value):
        if into_kw:
            self.kw[field] = conv(value)
        else:
            setattr(self, field, conv(value))
        return self
    with_.__name__ = "with_" + field
    return with_


def _mode_str(m) -> str:
    return m.value if hasattr(m, "value") else str(m)


# ------------------------------------------------------------------------------------ similarity / distance
_l.CosineSimilarity.with_eps = _setter("eps", float)
_l.CosineSimilarity.with_dim = _setter("dim", int)
_l.CosineSimilarity.forward_pair = lambda self, session, x1, x2: self.forward(session, x1, x2)


def _pd_forward(self, session, a, b):
    return session.tensor_pairwise_distance(a, b, p=self.p, eps=self.eps, keepdim=getattr(self, "keepdim", False))


_l.PairwiseDistance.forward = _pd_forward
_l.PairwiseDistance.with_p = _setter("p", float)
_l.PairwiseDistance.with_eps = _setter("eps", float)
_l.PairwiseDistance.with_keepdim = _setter("keepdim", bool)
_l.PairwiseDistance.forward_pair = lambda self, session, x1, x2: self.forward(session, x1, x2)

# ------------------------------------------------------------------------------------ losses
_t.CosineEmbeddingLoss.forward_triplet = lambda self, session, x1, x2, target: self.forward(session, x1, x2, target)
_t.MarginRankingLoss.forward_triplet = lambda self, session, x1, x2, target: self.forward(session, x1, x2, target)
_t.GaussianNLLLoss.forward_with_var = lambda self, session, input, target, var: self.forward(session, input, target, var)


def _forward_hinge(self, session, input, target):
    margin = self.kw.get("margin", 1.0)
    if not math.isfinite(margin):
        raise ValueError("HingeEmbeddingLoss margin must be finite")
    return self.forward(session, input, target)


_t.HingeEmbeddingLoss.forward_hinge = _forward_hinge
_t.CTCLoss.with_blank = _setter("blank", int, into_kw=True)
_t.CTCLoss.with_reduction = _setter("reduction", lambda r: _mode_str(CTCReduction(r) if not isinstance(r, CTCReduction) else r),
                                    into_kw=True)
_t.CTCLoss.with_zero_infinity = _setter("zero_infinity", bool, into_kw=True)
_t.CTCLoss.forward_ctc = lambda self, session, log_probs, targets, input_lengths, target_lengths: \
    self.forward(session, log_probs, targets, input_lengths, target_lengths)

_l.Bilinear.forward_bilinear = lambda self, session, x1, x2: self.forward(session, x1, x2)


# ------------------------------------------------------------------------------------ local response norm
def _lrn_with_params(size: int, alpha: float, beta: float, k: float):
    if size <= 0:
        raise ValueError("LocalResponseNorm requires size > 0")
    if not all(math.isfinite(v) for v in (alpha, beta, k)):
        raise ValueError("LocalResponseNorm parameters must be finite")
    return _l.LocalResponseNorm(size, alpha, beta, k)


_l.LocalResponseNorm.with_params = staticmethod(_lrn_with_params)


# ------------------------------------------------------------------------------------ embeddings
def _embedding_with_options(session, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                            max_norm: Optional[float] = None, norm_type: float = 2.0, sparse: bool = False):
    """Embedding with the full option set.  With ``max_norm`` every row that a lookup touches is first rescaled,
    in place and outside the graph, so that its ``norm_type`` norm is at most ``max_norm`` (torch's rule)."""
    if num_embeddings <= 0 or embedding_dim <= 0:
        raise ValueError("Embedding requires num_embeddings > 0 and embedding_dim > 0")
    if padding_idx is not None and not (0 <= padding_idx < num_embeddings):
        raise ValueError("Embedding padding_idx must be less than num_embeddings")
    if max_norm is not None and not (math.isfinite(max_norm) and max_norm > 0):
        raise ValueError("Embedding max_norm must be finite and positive")
    if not (norm_type > 0):
        raise ValueError("Embedding norm_type must be positive")
    m = _l.Embedding(session, num_embeddings, embedding_dim, padding_idx, sparse)
    m.max_norm, m.norm_type = max_norm, float(norm_type)
    return m


_embedding_forward_plain = _l.Embedding.forward


def _embedding_forward(self, session, ids):
    max_norm = getattr(self, "max_norm", None)
    if max_norm is not None:
        wid = self._parameters["weight"]
        rows = torch.unique(session.tensor(ids).reshape(-1).long())

        def renorm(w):
            sub = w[rows]
            norms = torch.linalg.vector_norm(sub, ord=self.norm_type, dim=1, keepdim=True)
            scale = torch.where(norms > max_norm, max_norm / (norms + 1e-7), torch.ones_like(norms))
            w[rows] = sub * scale
        session.tensor_tape.update_tensor_values_with(wid, renorm)
    return _embedding_forward_plain(self, session, ids)


_l.Embedding.forward = _embedding_forward
_l.Embedding.with_options = staticmethod(_embedding_with_options)


def _bag_forward_with_offsets(self, session, indices, offsets, per_sample_weights=None):
    """Bags given as one flat index list plus the start of each bag.  ``per_sample_weights`` (one weight per
    index, ``sum`` mode only) scales each looked-up row before the bag is summed; it receives a gradient."""
    if len(session.tensor_shape(indices)) != 1:
        raise ValueError("EmbeddingBag: indices must be 1D")
    if len(session.tensor_shape(offsets)) != 1:
        raise ValueError("EmbeddingBag: offsets must be 1D")
    if per_sample_weights is None:
        return self.forward(session, indices, offsets)
    if _mode_str(self.mode) != "sum":
        raise ValueError("EmbeddingBag: per_sample_weights is only supported in sum mode")
    n = session.tensor_shape(indices)[0]
    if session.tensor_shape(per_sample_weights) != [n]:
        raise ValueError("EmbeddingBag: per_sample_weights must have the shape of indices")
    off = session.tensor(offsets).long()
    if off.numel() and (int(off[0]) != 0 or bool((off[1:] < off[:-1]).any()) or int(off[-1]) > n):
        raise ValueError("EmbeddingBag: offsets must start at 0, be non-decreasing and stay inside indices")
    bags = off.numel()
    bag_of = torch.searchsorted(off, torch.arange(n, device=off.device), right=True) - 1
    rows = session.tensor_embedding(self._parameters["weight"], indices)                    # [n, D]
    rows = session.tensor_mul(rows, session.tensor_unsqueeze(per_sample_weights, dim=1))
    dim = session.tensor_shape(rows)[1]
    zero = session.zeros([bags, dim], dtype=session.tensor_dtype(rows))
    return session.tensor_index_add(zero, 0, session.tensor_tape.leaf(bag_of, False), rows)


_l.EmbeddingBag.forward_with_offsets = _bag_forward_with_offsets


# ------------------------------------------------------------------------------------ convolution / pooling
def _new_grouped(cls):
    def new_grouped(session, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0,
                    use_bias: bool = True, groups: int = 1):
        if in_channels <= 0 or out_channels <= 0 or (isinstance(kernel_size, int) and kernel_size <= 0):
            raise ValueError(f"{cls.__name__} requires positive channel counts and kernel size")
        if groups <= 0 or in_channels % groups or out_channels % groups:
            raise ValueError(f"{cls.__name__}: in_channels and out_channels must be divisible by groups")
        return cls(session, in_channels, out_channels, kernel_size, stride=stride, padding=padding, bias=use_bias,
                   groups=groups)
    return staticmethod(new_grouped)


_l.Conv1d.new_grouped = _new_grouped(_l.Conv1d)
_l.Conv2d.new_grouped = _new_grouped(_l.Conv2d)


def _ceil_mode(self, ceil_mode: bool):
    self.kw["ceil_mode"] = bool(ceil_mode)
    return self


_l.MaxPool2d.ceil_mode = _ceil_mode
_l.MaxPool1d.ceil_mode = _ceil_mode


def _unpool_forward_with_indices(self, session, input, indices: Sequence[int], output_size):
    """Unpooling with the argmax positions given as a host list (flattened, one per input element)."""
    shape = session.tensor_shape(input)
    want = 3 if isinstance(self, _x.MaxUnpool1d) else 4
    if len(shape) != want:
        raise ValueError(f"{type(self).__name__} expects a {want}-D input")
    idx = torch.as_tensor(list(indices), dtype=torch.long)
    if idx.numel() != math.prod(shape):
        raise ValueError(f"{type(self).__name__}: {idx.numel()} indices for {math.prod(shape)} input elements")
    out = (int(output_size),) if isinstance(output_size, int) else tuple(int(v) for v in output_size)
    if len(out) != want - 2:
        raise ValueError(f"{type(self).__name__}: output_size must give {want - 2} spatial extents")
    limit = math.prod(out)
    if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= limit):
        raise ValueError(f"{type(self).__name__}: an index lies outside the output of {limit} positions")
    leaf = session.tensor_tape.leaf(idx.reshape(shape).to(session.device), False)
    return self.forward(session, input, leaf, output_size=list(out))


_x.MaxUnpool1d.forward_with_indices = _unpool_forward_with_indices
_x.MaxUnpool2d.forward_with_indices = _unpool_forward_with_indices


# ------------------------------------------------------------------------------------ upsampling
def _upsample_from_options(cls):
    def from_options(size=None, scale_factor=None, mode=UpsampleMode.Nearest, align_corners=None):
        if size is not None and scale_factor is not None:
            raise ValueError(f"{cls.__name__} accepts either size or scale_factor, not both")
        if size is None and scale_factor is None:
            raise ValueError(f"{cls.__name__} requires size or scale_factor")
        return cls(size=size, scale_factor=scale_factor, mode=_mode_str(mode), align_corners=align_corners)
    return staticmethod(from_options)


def _fixed_from_options(cls):
    def from_options(size=None, scale_factor=None):
        if size is not None and scale_factor is not None:
            raise ValueError(f"{cls.__name__} accepts either size or scale_factor, not both")
        if size is None and scale_factor is None:
            raise ValueError(f"{cls.__name__} requires size or scale_factor")
        return cls(size=None if size is None else tuple(size), scale_factor=None if scale_factor is None else tuple(scale_factor))
    return staticmethod(from_options)


_x.Upsample.from_options = _upsample_from_options(_x.Upsample)
_x.Upsample.with_uniform_size = staticmethod(lambda size: _x.Upsample(size=int(size)))
_x.Upsample.with_size = staticmethod(lambda size: _x.Upsample(size=tuple(int(v) for v in size)))
_x.Upsample.with_uniform_scale_factor = staticmethod(lambda f: _x.Upsample(scale_factor=float(f)))
_x.Upsample.with_scale_factor = staticmethod(lambda f: _x.Upsample(scale_factor=tuple(float(v) for v in f)))
_x.Upsample.with_mode = _setter("mode", _mode_str, into_kw=True)
_x.Upsample.with_align_corners = _setter("align_corners", into_kw=True)
for _cls in (_x.UpsamplingNearest2d, _x.UpsamplingBilinear2d):
    _cls.with_size = staticmethod(lambda output_h, output_w, _c=_cls: _c(size=(int(output_h), int(output_w))))
    _cls.with_scale_factors = staticmethod(lambda scale_h, scale_w, _c=_cls: _c(scale_factor=(float(scale_h), float(scale_w))))
    _cls.with_scale_factor = staticmethod(lambda f, _c=_cls: _c(scale_factor=(float(f), float(f))))
    _cls.from_options = _fixed_from_options(_cls)


# ------------------------------------------------------------------------------------ observers
def _compute_qparams(self):
    """The affine parameters of the observed range, or None before the first observation.  The range is widened
    to contain 0 so that a floating-point zero has an exact code."""
    if not (self.min_val <= self.max_val):
        return None
    return self.calculate_qparams()


_u.MinMaxObserver.compute_qparams = _compute_qparams
_u.MinMaxObserver.initialized = property(lambda self: self.min_val <= self.max_val)
_u.qint8_range = lambda: _u.QuantizedStorageDType.QInt8.qrange()
_u.quint8_range = lambda: _u.QuantizedStorageDType.QUInt8.qrange()
