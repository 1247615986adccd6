"""Layers, part 1: linear family, activations, normalisation, dropout, embeddings, conv / pool.

Reference: ft-nn/src/lib.rs - Linear :902 (weight [out,in], bias [out], init U(+-1/sqrt(in))
:929-955), Bilinear :1190, activations :5855-6562, LayerNorm :2042 (weight ones / bias zeros),
Dropout family :2303-2761, Embedding :2873 (init N(0,1)), EmbeddingBag :3152, BatchNorm
:3574/:9643/:10105, GroupNorm :6661, RMSNorm :6843, InstanceNorm, Conv / ConvTranspose, pools,
Flatten / Unflatten / Identity, padding modules :17592-18627, PixelShuffle, ChannelShuffle.
Every forward goes through session operators, i.e. through the DAC tape.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

from .module import Module


def _param(session, shape, init: str = "zeros", bound: float = 0.0, std: float = 1.0) -> int:
    p = session.zeros(list(shape), requires_grad=False)
    if init == "uniform":
        session.init_uniform_(p, -bound, bound)
    elif init == "normal":
        session.init_normal_(p, 0.0, std)
    elif init == "ones":
        session.init_ones_(p)
    session.tensor_requires_grad_(p, True)
    return p


class Identity(Module):
    def forward(self, session, x):
        return x


class Linear(Module):
    def __init__(self, session, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        bound = 1.0 / math.sqrt(in_features)
        self.register_parameter("weight", _param(session, (out_features, in_features), "uniform", bound))
        self.register_parameter("bias", _param(session, (out_features,), "uniform", bound) if bias else None)

    @property
    def weight(self):
        return self._parameters["weight"]

    @property
    def bias(self):
        return self._parameters["bias"]

    def forward(self, session, x):
        return session.tensor_linear(x, self.weight, self.bias)


class LazyLinear(Module):
    """Linear whose ``in_features`` is taken from the first input."""

    def __init__(self, session, out_features: int, bias: bool = True):
        super().__init__()
        self.out_features, self._bias, self._inner = out_features, bias, None

    def is_materialized(self) -> bool:
        return self._inner is not None

    def materialize(self, session, in_features: int) -> None:
        """Create the parameters for ``in_features`` now instead of at the first forward (no-op when they exist)."""
        if self._inner is None:
            object.__setattr__(self, "_inner", Linear(session, in_features, self.out_features, self._bias))
            self.register_parameter("weight", self._inner._parameters["weight"])
            self.register_parameter("bias", self._inner._parameters["bias"])

    def forward(self, session, x):
        if self._inner is None:
            # bypass child registration: the parameters are registered on this module itself
            object.__setattr__(self, "_inner", Linear(session, session.tensor_shape(x)[-1], self.out_features, self._bias))
            self.register_parameter("weight", self._inner._parameters["weight"])
            self.register_parameter("bias", self._inner._parameters["bias"])
        return session.tensor_linear(x, self._parameters["weight"], self._parameters["bias"])


class Bilinear(Module):
    def __init__(self, session, in1: int, in2: int, out: int, bias: bool = True):
        super().__init__()
        bound = 1.0 / math.sqrt(in1)
        self.register_parameter("weight", _param(session, (out, in1, in2), "uniform", bound))
        self.register_parameter("bias", _param(session, (out,), "uniform", bound) if bias else None)

    def forward(self, session, a, b):
        return session.tensor_bilinear(a, b, self._parameters["weight"], self._parameters["bias"])


def _activation(op: str, **fixed):
    class _Act(Module):
        def __init__(self, **kw):
            super().__init__()
            self.kw = {**fixed, **kw}

        def forward(self, session, x):
            return getattr(session, "tensor_" + op)(x, **self.kw)
    _Act.__name__ = op
    return _Act


ReLU = _activation("relu")
ReLU6 = _activation("relu6")
Sigmoid = _activation("sigmoid")
Tanh = _activation("tanh")
GELU = _activation("gelu")              # exact erf form (reference default, ft-nn :1927)
GELUTanh = _activation("gelu_tanh")
SiLU = _activation("silu")
LeakyReLU = _activation("leaky_relu")
ELU = _activation("elu")
Mish = _activation("mish")
Softplus = _activation("softplus")
CELU = _activation("celu")
SELU = _activation("selu")
GLU = _activation("glu")
Hardtanh = _activation("hardtanh")
Softshrink = _activation("softshrink")
Hardshrink = _activation("hardshrink")
Tanhshrink = _activation("tanhshrink")
Softsign = _activation("softsign")
Hardswish = _activation("hardswish")
Hardsigmoid = _activation("hardsigmoid")
LogSigmoid = _activation("logsigmoid")
Threshold = _activation("threshold")
RReLU = _activation("rrelu")
SwiGLU = _activation("swiglu")
GEGLU = _activation("geglu")
ReGLU = _activation("reglu")


class PReLU(Module):
    def __init__(self, session, num_parameters: int = 1, init: float = 0.25):
        super().__init__()
        p = session.full([num_parameters], init)
        session.tensor_requires_grad_(p, True)
        self.register_parameter("weight", p)

    def forward(self, session, x):
        return session.tensor_prelu(x, self._parameters["weight"])


class Softmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, session, x):
        return session.tensor_softmax(x, dim=self.dim)


class Softmin(Softmax):
    def forward(self, session, x):
        return session.tensor_softmin(x, dim=self.dim)


class LogSoftmax(Softmax):
    def forward(self, session, x):
        return session.tensor_log_softmax(x, dim=self.dim)


class Softmax2d(Module):
    def forward(self, session, x):
        return session.tensor_softmax(x, dim=-3)


class Flatten(Module):
    def __init__(self, start_dim: int = 1, end_dim: int = -1):
        super().__init__()
        self.start, self.end = start_dim, end_dim

    def forward(self, session, x):
        return session.tensor_flatten(x, start=self.start, end=self.end)


class Unflatten(Module):
    def __init__(self, dim: int, sizes: Sequence[int]):
        super().__init__()
        self.dim, self.sizes = dim, tuple(sizes)

    def forward(self, session, x):
        return session.tensor_unflatten(x, self.dim, self.sizes)


# -------------------------------------------------------------------------------------- normalisation
class LayerNorm(Module):
    def __init__(self, session, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True):
        super().__init__()
        self.shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.eps = eps
        self.register_parameter("weight", _param(session, self.shape, "ones") if elementwise_affine else None)
        self.register_parameter("bias", _param(session, self.shape, "zeros") if elementwise_affine else None)

    def forward(self, session, x):
        return session.tensor_layer_norm(x, self._parameters["weight"], self._parameters["bias"], eps=self.eps,
                                         ndim=len(self.shape))


class RMSNorm(Module):
    def __init__(self, session, dim: int, eps: float = 1e-6, elementwise_affine: bool = True):
        super().__init__()
        self.eps = eps
        self.register_parameter("weight", _param(session, (dim,), "ones") if elementwise_affine else None)

    def forward(self, session, x):
        return session.tensor_rms_norm(x, self._parameters["weight"], eps=self.eps)


class GroupNorm(Module):
    def __init__(self, session, num_groups: int, num_channels: int, eps: float = 1e-5, affine: bool = True):
        super().__init__()
        self.groups, self.eps = num_groups, eps
        self.register_parameter("weight", _param(session, (num_channels,), "ones") if affine else None)
        self.register_parameter("bias", _param(session, (num_channels,), "zeros") if affine else None)

    def forward(self, session, x):
        return session.tensor_group_norm(x, self._parameters["weight"], self._parameters["bias"], groups=self.groups,
                                         eps=self.eps)


class _BatchNorm(Module):
    """Training: batch statistics through the tape, running stats updated under no_grad;
    eval: the running statistics as constants."""

    def __init__(self, session, num_features: int, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True,
                 track_running_stats: bool = True):
        super().__init__()
        self.eps, self.momentum, self.track = eps, momentum, track_running_stats
        self.register_parameter("weight", _param(session, (num_features,), "ones") if affine else None)
        self.register_parameter("bias", _param(session, (num_features,), "zeros") if affine else None)
        if track_running_stats:
            self.register_buffer("running_mean", session.zeros([num_features]))
            self.register_buffer("running_var", session.ones([num_features]))
            self.register_buffer("num_batches_tracked", session.zeros([1]))

    def forward(self, session, x):
        w, b = self._parameters["weight"], self._parameters["bias"]
        if self.training or not self.track:
            y = session.tensor_batch_norm(x, w, b, eps=self.eps)
            if self.track:
                xt = session.tensor(x).detach()
                dims = [d for d in range(xt.dim()) if d != 1]
                with session.no_grad():
                    rm, rv = session.tensor(self._buffers["running_mean"][0]), session.tensor(self._buffers["running_var"][0])
                    n = xt.numel() / xt.shape[1]
                    rm.mul_(1 - self.momentum).add_(self.momentum * xt.mean(dims).to(rm.dtype))
                    rv.mul_(1 - self.momentum).add_(self.momentum * (xt.var(dims, unbiased=False) * n / max(n - 1, 1)).to(rv.dtype))
                    session.tensor(self._buffers["num_batches_tracked"][0]).add_(1)
            return y
        rm, rv = session.tensor(self._buffers["running_mean"][0]), session.tensor(self._buffers["running_var"][0])
        shape = [1, -1] + [1] * (len(session.tensor_shape(x)) - 2)
        scale = session.tensor_tape.leaf((1.0 / torch.sqrt(rv + self.eps)).reshape(shape), False)
        shift = session.tensor_tape.leaf(rm.reshape(shape), False)
        y = session.tensor_mul(session.tensor_sub(x, shift), scale)
        if w is not None:
            y = session.tensor_add(session.tensor_mul(y, session.tensor_reshape(w, shape=tuple(shape))),
                                   session.tensor_reshape(b, shape=tuple(shape)))
        return y


class BatchNorm1d(_BatchNorm):
    pass


class BatchNorm2d(_BatchNorm):
    pass


class BatchNorm3d(_BatchNorm):
    pass


class _InstanceNorm(Module):
    def __init__(self, session, num_features: int, eps: float = 1e-5, affine: bool = False):
        super().__init__()
        self.eps = eps
        self.register_parameter("weight", _param(session, (num_features,), "ones") if affine else None)
        self.register_parameter("bias", _param(session, (num_features,), "zeros") if affine else None)

    def forward(self, session, x):
        return session.tensor_instance_norm(x, self._parameters["weight"], self._parameters["bias"], eps=self.eps)


InstanceNorm1d = InstanceNorm2d = InstanceNorm3d = _InstanceNorm


class LocalResponseNorm(Module):
    def __init__(self, size: int, alpha: float = 1e-4, beta: float = 0.75, k: float = 1.0):
        super().__init__()
        self.kw = dict(size=size, alpha=alpha, beta=beta, k=k)

    def forward(self, session, x):
        return session.tensor_local_response_norm(x, **self.kw)


# -------------------------------------------------------------------------------------- dropout
class Dropout(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        if not (0.0 <= p < 1.0):
            raise ValueError("dropout probability must be in [0, 1)")
        self.p = p

    def forward(self, session, x):
        return session.functional_dropout(x, self.p, self.training)


class _ChannelDropout(Dropout):
    """Drops whole channels (dim 1): the mask is drawn per (N, C) and broadcast."""

    def forward(self, session, x):
        if not self.training or self.p == 0.0:
            return x
        shp = session.tensor_shape(x)
        mshape = shp[:2] + [1] * (len(shp) - 2)
        u = session.rng.uniform(shp[0] * shp[1]).reshape(mshape)
        m = session.tensor_tape.leaf(((u > self.p).to(torch.float64) / (1 - self.p)).to(session.tensor(x).dtype).to(session.device), False)
        return session.tensor_mul(x, m)


Dropout1d = Dropout2d = Dropout3d = FeatureAlphaDropout = _ChannelDropout


class AlphaDropout(Dropout):
    def forward(self, session, x):
        if not self.training or self.p == 0.0:
            return x
        alpha = -1.7580993408473766
        a = (1 - self.p + self.p * alpha * alpha * (1 - self.p)) ** -0.5
        b = -a * alpha * self.p
        keep = (session.rng.uniform(session.tensor_numel(x)).reshape(session.tensor_shape(x)) > self.p).to(torch.float64)
        k = session.tensor_tape.leaf(keep.to(session.tensor(x).dtype).to(session.device), False)
        nk = session.tensor_tape.leaf(((1 - keep) * alpha).to(session.tensor(x).dtype).to(session.device), False)
        y = session.tensor_add(session.tensor_mul(x, k), nk)
        return session.tensor_add_scalar(session.tensor_mul_scalar(y, c=a), c=b)


# -------------------------------------------------------------------------------------- embeddings
class Embedding(Module):
    def __init__(self, session, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 sparse: bool = False):
        super().__init__()
        self.padding_idx = padding_idx
        self.sparse = sparse        # row-sparse weight gradient for SparseAdam (ft-nn/src/lib.rs:2873 "+sparse")
        w = _param(session, (num_embeddings, embedding_dim), "normal", std=1.0)
        if padding_idx is not None:
            with session.no_grad():
                session.tensor(w)[padding_idx].zero_()
        self.register_parameter("weight", w)

    def forward(self, session, ids):
        if self.sparse:
            out = session.tensor_index_select_sparse(self._parameters["weight"], ids)
        else:
            out = session.tensor_embedding(self._parameters["weight"], ids)
        if self.padding_idx is not None:
            h = session.register_tensor_hook  # gradient of the padding row is forced to zero
            pid, wid = self.padding_idx, self._parameters["weight"]

            def zero_pad_row(g):
                g = g.clone()
                g[pid].zero_()
                return g
            if not getattr(self, "_pad_hook", None):
                object.__setattr__(self, "_pad_hook", h(wid, zero_pad_row))
        return out


class EmbeddingBag(Module):
    def __init__(self, session, num_embeddings: int, embedding_dim: int, mode: str = "mean"):
        super().__init__()
        self.mode = mode
        self.register_parameter("weight", _param(session, (num_embeddings, embedding_dim), "normal", std=1.0))

    def forward(self, session, ids, offsets):
        return session.tensor_embedding_bag(self._parameters["weight"], ids, offsets, mode=self.mode)


# -------------------------------------------------------------------------------------- conv / pool
class _ConvNd(Module):
    def __init__(self, session, nd, in_ch, out_ch, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 transposed=False, output_padding=0):
        super().__init__()
        ks = (kernel_size,) * nd if isinstance(kernel_size, int) else tuple(kernel_size)
        self.nd, self.transposed = nd, transposed
        self.kw = dict(stride=stride, padding=padding, dilation=dilation, groups=groups)
        if transposed:
            self.kw["output_padding"] = output_padding
            wshape = (in_ch, out_ch // groups) + ks
        else:
            wshape = (out_ch, in_ch // groups) + ks
        fan_in = (in_ch // groups) * math.prod(ks)
        bound = 1.0 / math.sqrt(fan_in)
        self.register_parameter("weight", _param(session, wshape, "uniform", bound))
        self.register_parameter("bias", _param(session, (out_ch,), "uniform", bound) if bias else None)

    def forward(self, session, x):
        name = f"tensor_conv{'_transpose' if self.transposed else ''}{self.nd}d"
        return getattr(session, name)(x, self._parameters["weight"], self._parameters["bias"], **self.kw)


def _conv(nd, transposed=False):
    class _C(_ConvNd):
        def __init__(self, session, in_ch, out_ch, kernel_size, **kw):
            super().__init__(session, nd, in_ch, out_ch, kernel_size, transposed=transposed, **kw)
    _C.__name__ = f"Conv{'Transpose' if transposed else ''}{nd}d"
    return _C


Conv1d, Conv2d, Conv3d = _conv(1), _conv(2), _conv(3)
ConvTranspose1d, ConvTranspose2d, ConvTranspose3d = _conv(1, True), _conv(2, True), _conv(3, True)


def _pool(op: str, **defaults):
    class _P(Module):
        def __init__(self, *args, **kw):
            super().__init__()
            self.args, self.kw = args, {**defaults, **kw}

        def forward(self, session, x):
            return getattr(session, "tensor_" + op)(x, *self.args, **self.kw)
    _P.__name__ = op
    return _P


AvgPool1d, AvgPool2d, AvgPool3d = _pool("avg_pool1d"), _pool("avg_pool2d"), _pool("avg_pool3d")
MaxPool1d, MaxPool2d, MaxPool3d = _pool("max_pool1d"), _pool("max_pool2d"), _pool("max_pool3d")
AdaptiveAvgPool1d, AdaptiveAvgPool2d, AdaptiveAvgPool3d = (_pool("adaptive_avg_pool1d"), _pool("adaptive_avg_pool2d"),
                                                          _pool("adaptive_avg_pool3d"))
AdaptiveMaxPool1d, AdaptiveMaxPool2d, AdaptiveMaxPool3d = (_pool("adaptive_max_pool1d"), _pool("adaptive_max_pool2d"),
                                                          _pool("adaptive_max_pool3d"))
LPPool1d, LPPool2d = _pool("lp_pool1d"), _pool("lp_pool2d")
PixelShuffle, PixelUnshuffle = _pool("pixel_shuffle"), _pool("pixel_unshuffle")
Unfold, Fold = _pool("unfold"), _pool("fold")
Upsample = _pool("interpolate")


class _Pad(Module):
    def __init__(self, padding, mode: str = "constant", value: float = 0.0):
        super().__init__()
        self.padding = (padding,) * 2 if isinstance(padding, int) else tuple(padding)
        self.mode, self.value = mode, value

    def forward(self, session, x):
        if self.mode == "constant":
            return session.tensor_pad(x, padding=self.padding, value=self.value)
        return session.tensor_pad_mode(x, padding=self.padding, mode=self.mode)


def _pad_cls(mode, nd):
    class _P(_Pad):
        def __init__(self, padding, value: float = 0.0):
            pad = (padding,) * (2 * nd) if isinstance(padding, int) else tuple(padding)
            super().__init__(pad, mode, value)
    return _P


ConstantPad1d, ConstantPad2d, ConstantPad3d = (_pad_cls("constant", n) for n in (1, 2, 3))
ZeroPad1d, ZeroPad2d, ZeroPad3d = (_pad_cls("constant", n) for n in (1, 2, 3))
ReflectionPad1d, ReflectionPad2d, ReflectionPad3d = (_pad_cls("reflect", n) for n in (1, 2, 3))
ReplicationPad1d, ReplicationPad2d, ReplicationPad3d = (_pad_cls("replicate", n) for n in (1, 2, 3))
CircularPad1d, CircularPad2d, CircularPad3d = (_pad_cls("circular", n) for n in (1, 2, 3))


class ChannelShuffle(Module):
    def __init__(self, groups: int):
        super().__init__()
        self.groups = groups

    def forward(self, session, x):
        shp = session.tensor_shape(x)
        n, c = shp[0], shp[1]
        y = session.tensor_reshape(x, shape=(n, self.groups, c // self.groups, *shp[2:]))
        y = session.tensor_transpose(y, dim0=1, dim1=2)
        return session.tensor_reshape(y, shape=tuple(shp))


class CosineSimilarity(Module):
    def __init__(self, dim: int = 1, eps: float = 1e-8):
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, session, a, b):
        return session.tensor_cosine_similarity(a, b, dim=self.dim, eps=self.eps)


class PairwiseDistance(Module):
    def __init__(self, p: float = 2.0, eps: float = 1e-6):
        super().__init__()
        self.p, self.eps = p, eps

    def forward(self, session, a, b):
        return session.tensor_pairwise_distance(a, b, p=self.p, eps=self.eps)
