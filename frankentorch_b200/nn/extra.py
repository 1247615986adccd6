"""Modules completing the reference's ft-nn list: lazy convolutions, fractional max pooling,
max unpooling and the adaptive softmax (crates/ft-nn/src/lib.rs: LazyConv*, FractionalMaxPool2d,
MaxUnpool*, AdaptiveLogSoftmaxWithLoss ``:5371``)."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

from .layers import Linear, _ConvNd
from .module import Module, ModuleList


def _lazy_conv(nd: int):
    class _Lazy(Module):
        """Convolution whose ``in_channels`` is taken from the first input."""

        def __init__(self, session, out_channels: int, kernel_size, **kw):
            super().__init__()
            self.out_channels, self.kernel_size, self.kw, self._inner = out_channels, kernel_size, kw, None

        def is_materialized(self) -> bool:
            return self._inner is not None

        def materialize(self, session, in_channels: int) -> None:
            if self._inner is None:
                object.__setattr__(self, "_inner", _ConvNd(session, nd, in_channels, self.out_channels, self.kernel_size, **self.kw))
                self.register_parameter("weight", self._inner._parameters["weight"])
                self.register_parameter("bias", self._inner._parameters["bias"])

        def forward(self, session, x):
            shape = session.tensor_shape(x)
            if len(shape) != nd + 2:
                raise ValueError(f"LazyConv{nd}d expects a {nd + 2}-D input [N, C, ...]")
            self.materialize(session, shape[1])
            return self._inner.forward(session, x)

        forward_lazy = forward
    _Lazy.__name__ = f"LazyConv{nd}d"
    return _Lazy


LazyConv1d, LazyConv2d, LazyConv3d = _lazy_conv(1), _lazy_conv(2), _lazy_conv(3)


class FractionalMaxPool2d(Module):
    """Fractional max pooling.  The window offsets come from ``samples[N, C, 2]`` in [0, 1): drawn
    from the session's deterministic PRNG in training mode, fixed at 0.5 in evaluation mode, so a
    replay with the same seed pools the same windows."""

    def __init__(self, kernel_size, output_size=None, output_ratio=None):
        super().__init__()
        if (output_size is None) == (output_ratio is None):
            raise ValueError("give exactly one of output_size and output_ratio")
        self.kernel_size, self.output_size, self.output_ratio = kernel_size, output_size, output_ratio

    def forward(self, session, x):
        samples = None
        if self.training:
            n, c = session.tensor_shape(x)[:2]
            samples = session.tensor(session.rand([n, c, 2])).to(session.tensor(x).dtype)
        return session.tensor_fractional_max_pool2d(x, kernel_size=self.kernel_size, output_size=self.output_size,
                                                    output_ratio=self.output_ratio, samples=samples)


class MaxPool2dWithIndices(Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.kw = dict(kernel_size=kernel_size, stride=stride, padding=padding)

    def forward(self, session, x) -> Tuple[int, int]:
        return (session.tensor_max_pool2d(x, self.kw["kernel_size"], self.kw["stride"] or self.kw["kernel_size"],
                                          self.kw["padding"]),
                session.tensor_max_pool2d_indices(x, **self.kw))


class MaxUnpool2d(Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.kw = dict(kernel_size=kernel_size, stride=stride, padding=padding)

    def forward(self, session, x, indices, output_size=None):
        return session.tensor_max_unpool2d(x, indices, output_size=output_size, **self.kw)


class AdaptiveLogSoftmaxWithLoss(Module):
    """Efficient softmax approximation (Grave et al.): a head over the frequent classes plus one
    entry per tail cluster, and a down-projected classifier per cluster.

    ``forward(session, x[N, in], target[N]) -> (output[N], loss)`` where ``output`` holds each
    sample's target log-probability and ``loss`` is their negative mean; ``log_prob`` returns the
    full ``[N, n_classes]`` table.  Cluster ``i`` projects to ``in / div_value**(i+1)`` features.
    """

    def __init__(self, session, in_features: int, n_classes: int, cutoffs: Sequence[int], div_value: float = 4.0,
                 head_bias: bool = False):
        super().__init__()
        cutoffs = list(cutoffs)
        if (not cutoffs or cutoffs != sorted(set(cutoffs)) or cutoffs[0] <= 0 or cutoffs[-1] > n_classes - 1):
            raise ValueError("cutoffs must be unique, increasing and inside (0, n_classes - 1]")
        self.in_features, self.n_classes, self.div_value = in_features, n_classes, div_value
        self.cutoffs = cutoffs + [n_classes]
        self.shortlist, self.n_clusters = cutoffs[0], len(cutoffs)
        self.head = Linear(session, in_features, self.shortlist + self.n_clusters, head_bias)
        tails = []
        for i in range(self.n_clusters):
            hsz = max(1, int(in_features // (div_value ** (i + 1))))
            osz = self.cutoffs[i + 1] - self.cutoffs[i]
            tails.append(ModuleList([Linear(session, in_features, hsz, False), Linear(session, hsz, osz, False)]))
        self.tail = ModuleList(tails)

    def log_prob(self, session, x) -> int:
        head_lp = session.tensor_log_softmax(self.head.forward(session, x), -1)
        parts = [session.tensor_narrow(head_lp, 1, 0, self.shortlist)]
        for i in range(self.n_clusters):
            proj, out = self.tail[i][0], self.tail[i][1]
            cl = session.tensor_log_softmax(out.forward(session, proj.forward(session, x)), -1)
            gate = session.tensor_narrow(head_lp, 1, self.shortlist + i, 1)
            parts.append(session.tensor_add(cl, gate))
        return session.tensor_cat(parts, 1)

    def forward(self, session, x, target) -> Tuple[int, int]:
        lp = self.log_prob(session, x)
        n = session.tensor_shape(x)[0]
        idx = session.tensor_reshape(target, [n, 1])
        out = session.tensor_reshape(session.tensor_gather(lp, idx, 1), [n])
        loss = session.tensor_neg(session.tensor_mean(out))
        return out, loss

    def predict(self, session, x) -> int:
        return session.tensor_argmax(self.log_prob(session, x), 1)


# ---------------------------------------------------------------------------------- remaining pools / unpools
class FractionalMaxPool3d(FractionalMaxPool2d):
    """Volume form of :class:`FractionalMaxPool2d` (``samples[N, C, 3]``)."""

    def forward(self, session, x):
        samples = None
        if self.training:
            n, c = session.tensor_shape(x)[:2]
            samples = session.tensor(session.rand([n, c, 3])).to(session.tensor(x).dtype)
        return session.tensor_fractional_max_pool3d(x, kernel_size=self.kernel_size, output_size=self.output_size,
                                                    output_ratio=self.output_ratio, samples=samples)


class LPPool3d(Module):
    def __init__(self, norm_type: float, kernel_size, stride=None):
        super().__init__()
        self.kw = dict(norm_type=float(norm_type), kernel_size=kernel_size, stride=stride)

    def forward(self, session, x):
        return session.tensor_lp_pool3d(x, **self.kw)


class MaxUnpool1d(MaxUnpool2d):
    def forward(self, session, x, indices, output_size=None):
        return session.tensor_max_unpool1d(x, indices, output_size=output_size, **self.kw)


class MaxUnpool3d(MaxUnpool2d):
    def forward(self, session, x, indices, output_size=None):
        return session.tensor_max_unpool3d(x, indices, output_size=output_size, **self.kw)


# ---------------------------------------------------------------------------------- upsampling
class Upsample(Module):
    """``interpolate`` as a module: give ``size`` or ``scale_factor``; ``mode`` as in ``tensor_interpolate``."""

    ndim = 0        # 0: any

    def __init__(self, size=None, scale_factor=None, mode: str = "nearest", align_corners=None):
        super().__init__()
        if (size is None) == (scale_factor is None):
            raise ValueError("give exactly one of size and scale_factor")
        self.kw = dict(size=size, scale_factor=scale_factor, mode=mode, align_corners=align_corners)

    def forward(self, session, x):
        if self.ndim and len(session.tensor_shape(x)) != self.ndim + 2:
            raise ValueError(f"{type(self).__name__} expects a [N, C, {self.ndim} spatial dims] input")
        return session.tensor_interpolate(x, **{k: v for k, v in self.kw.items() if v is not None})


class Upsample1d(Upsample):
    ndim = 1


class Upsample2d(Upsample):
    ndim = 2


class Upsample3d(Upsample):
    ndim = 3


class UpsamplingNearest2d(Upsample2d):
    def __init__(self, size=None, scale_factor=None):
        super().__init__(size, scale_factor, mode="nearest")


class UpsamplingBilinear2d(Upsample2d):
    def __init__(self, size=None, scale_factor=None):
        super().__init__(size, scale_factor, mode="bilinear", align_corners=True)


# ---------------------------------------------------------------------------------- losses
class MultiLabelMarginLoss(Module):
    def __init__(self, reduction: str = "mean"):
        super().__init__()
        self.reduction = reduction

    def forward(self, session, x, target):
        return session.tensor_multilabel_margin_loss(x, target, reduction=self.reduction)


class MultiLabelSoftMarginLoss(Module):
    def __init__(self, reduction: str = "mean"):
        super().__init__()
        self.reduction = reduction

    def forward(self, session, x, target):
        return session.tensor_multilabel_soft_margin_loss(x, target, reduction=self.reduction)


class TripletMarginWithDistanceLoss(Module):
    """``mean(max(d(a, p) - d(a, n) + margin, 0))`` with a caller-supplied distance
    ``distance_function(session, x, y) -> node`` (default: pairwise L2 distance); ``swap`` uses
    ``min(d(a, n), d(p, n))`` for the negative distance."""

    def __init__(self, distance_function=None, margin: float = 1.0, swap: bool = False, reduction: str = "mean"):
        super().__init__()
        self.distance_function, self.margin, self.swap, self.reduction = distance_function, float(margin), swap, reduction

    def forward(self, session, anchor, positive, negative):
        dist = self.distance_function or (lambda s, x, y: s.tensor_pairwise_distance(x, y))
        d_ap, d_an = dist(session, anchor, positive), dist(session, anchor, negative)
        if self.swap:
            d_pn = dist(session, positive, negative)           # min(a, b) = a - relu(a - b)
            d_an = session.tensor_sub(d_an, session.tensor_relu(session.tensor_sub(d_an, d_pn)))
        loss = session.tensor_relu(session.tensor_add_scalar(session.tensor_sub(d_ap, d_an), self.margin))
        if self.reduction == "mean":
            return session.tensor_mean(loss)
        if self.reduction == "sum":
            return session.tensor_sum(loss)
        return loss


# ---------------------------------------------------------------------------------- recurrent records
from dataclasses import dataclass as _dataclass  # noqa: E402
from typing import NamedTuple as _NamedTuple  # noqa: E402


@_dataclass(frozen=True)
class RNNConfig:
    """Constructor arguments of the recurrent stacks (ft-nn's ``RNNConfig``); ``build`` makes the module."""
    input_size: int
    hidden_size: int
    num_layers: int = 1
    bias: bool = True
    batch_first: bool = False
    dropout: float = 0.0
    bidirectional: bool = False

    def build(self, session, kind: str = "rnn"):
        from . import transformer as _t
        cls = {"rnn": _t.RNN, "gru": _t.GRU, "lstm": _t.LSTM}[kind]
        import inspect
        allowed = set(inspect.signature(cls.__init__).parameters)
        kw = {k: v for k, v in self.__dict__.items() if k in allowed}
        return cls(session, **kw)


class RNNOutput(_NamedTuple):
    output: int          # node id of the output sequence
    h_n: int             # node id of the final hidden state


class GRUOutput(_NamedTuple):
    output: int
    h_n: int


class LSTMOutput(_NamedTuple):
    output: int
    h_n: int
    c_n: int
