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

        def forward(self, session, x):
            if self._inner is None:
                in_ch = session.tensor_shape(x)[1]
                object.__setattr__(self, "_inner", _ConvNd(session, nd, in_ch, self.out_channels, self.kernel_size, **self.kw))
                self.register_parameter("weight", self._inner._parameters["weight"])
                self.register_parameter("bias", self._inner._parameters["bias"])
            return self._inner.forward(session, x)
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
