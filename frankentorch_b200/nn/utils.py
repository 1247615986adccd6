"""nn utilities: packed sequences, weight / spectral norm, quantisation helpers.

Reference: ft-nn/src/lib.rs - PackedSequence + pack/pad utils :19022-19401, weight_norm /
spectral_norm :19457-19601, QParams / MinMaxObserver / QuantizedLinear :20024-20530.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .layers import Linear
from .module import Module


@dataclass
class PackedSequence:
    data: torch.Tensor           # [sum(lengths), *]
    batch_sizes: List[int]       # number of sequences alive at each time step
    sorted_indices: List[int]
    unsorted_indices: List[int]


def pad_sequence(seqs: Sequence[torch.Tensor], batch_first: bool = True, padding_value: float = 0.0) -> torch.Tensor:
    return torch.nn.utils.rnn.pad_sequence(list(seqs), batch_first=batch_first, padding_value=padding_value)


def pack_padded_sequence(padded: torch.Tensor, lengths: Sequence[int], batch_first: bool = True) -> PackedSequence:
    if not batch_first:
        padded = padded.transpose(0, 1)
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])      # stable: ties keep batch order
    unsort = [0] * len(order)
    for k, i in enumerate(order):
        unsort[i] = k
    maxlen = max(lengths)
    chunks, batch_sizes = [], []
    for t in range(maxlen):
        alive = [i for i in order if lengths[i] > t]
        batch_sizes.append(len(alive))
        chunks.append(padded[alive, t])
    return PackedSequence(torch.cat(chunks, 0), batch_sizes, order, unsort)


def pad_packed_sequence(packed: PackedSequence, batch_first: bool = True, padding_value: float = 0.0) -> Tuple[torch.Tensor, List[int]]:
    n, maxlen = packed.batch_sizes[0], len(packed.batch_sizes)
    out = torch.full((n, maxlen) + tuple(packed.data.shape[1:]), padding_value, dtype=packed.data.dtype)
    lengths_sorted = [sum(1 for b in packed.batch_sizes if b > k) for k in range(n)]
    off = 0
    for t, b in enumerate(packed.batch_sizes):
        out[:b, t] = packed.data[off: off + b]
        off += b
    out = out[packed.unsorted_indices]
    lengths = [lengths_sorted[packed.unsorted_indices[i]] for i in range(n)]
    return (out if batch_first else out.transpose(0, 1)), lengths


def pack_sequence(seqs: Sequence[torch.Tensor]) -> PackedSequence:
    return pack_padded_sequence(pad_sequence(seqs), [s.shape[0] for s in seqs])


class WeightNorm(Module):
    """w = g * v / ||v|| (norm over all dims but 0), re-materialised on every forward."""

    def __init__(self, session, linear: Linear):
        super().__init__()
        w = session.tensor(linear.weight).detach()
        g = session.tensor_tape.leaf(w.reshape(w.shape[0], -1).norm(dim=1, keepdim=True).clone(), True)
        v = session.tensor_tape.leaf(w.clone(), True)
        self.register_parameter("weight_g", g)
        self.register_parameter("weight_v", v)
        self.register_parameter("bias", linear.bias)

    def forward(self, session, x):
        v, g = self._parameters["weight_v"], self._parameters["weight_g"]
        nrm = session.tensor_norm_dim(v, p=2.0, dim=1, keepdim=True)
        w = session.tensor_mul(session.tensor_div(v, nrm), g)
        return session.tensor_linear(x, w, self._parameters["bias"])


def weight_norm(session, linear: Linear) -> WeightNorm:
    return WeightNorm(session, linear)


def _wn_check(session, t, dim):
    shape = session.tensor_shape(t)
    if not 0 <= dim < len(shape):
        raise ValueError("weight_norm: dim out of range")
    if shape[dim] == 0:
        raise ValueError("weight_norm: dimension size must be > 0")
    return shape


def weight_norm_decompose(session, weight: int, dim: int = 0) -> Tuple[int, int]:
    """``w = g * v / ||v||`` with the norm over every dimension but ``dim`` (ft-nn/src/lib.rs:19457): returns two
    new trainable leaves, the magnitudes ``g`` ``[shape[dim]]`` (floored at 1e-12) and the direction ``v = w``."""
    shape = _wn_check(session, weight, dim)
    w = session.tensor(weight).detach()
    others = [d for d in range(len(shape)) if d != dim]
    g = torch.sqrt((w.to(torch.float64) ** 2).sum(others)) if others else w.to(torch.float64).abs()
    g = g.clamp_min(1e-12).to(w.dtype)
    return session.tensor_tape.leaf(g.clone(), True), session.tensor_tape.leaf(w.clone(), True)


def weight_norm_reconstruct(session, g: int, v: int, dim: int = 0) -> int:
    """``g * v / ||v||`` built from session operators, so gradients reach both ``g`` and ``v``
    (ft-nn/src/lib.rs:19508)."""
    shape = _wn_check(session, v, dim)
    if session.tensor_numel(g) != shape[dim]:
        raise ValueError("weight_norm: magnitude length mismatch")
    bshape = [1] * len(shape)
    bshape[dim] = shape[dim]
    sq = session.tensor_square(v)
    for d in sorted((d for d in range(len(shape)) if d != dim), reverse=True):
        sq = session.tensor_sum_dim(sq, dim=d, keepdim=True)
    nrm = session.tensor_clamp_min(session.tensor_sqrt(sq), 1e-12)
    scale = session.tensor_div(session.tensor_reshape(g, shape=tuple(bshape)), session.tensor_reshape(nrm, shape=tuple(bshape)))
    return session.tensor_mul(v, scale)


class SpectralNorm(Module):
    """Divides the weight by its largest singular value estimated by power iteration."""

    def __init__(self, session, linear: Linear, n_power_iterations: int = 1, eps: float = 1e-12):
        super().__init__()
        self.inner, self.iters, self.eps = linear, n_power_iterations, eps
        w = session.tensor(linear.weight)
        u = session.rng.normal(w.shape[0]).to(w.dtype)
        self.register_buffer("u", session.tensor_tape.leaf((u / (u.norm() + eps)).to(session.device), False))

    def forward(self, session, x):
        w = session.tensor(self.inner.weight).detach()
        u = session.tensor(self._buffers["u"][0])
        with session.no_grad():
            for _ in range(self.iters):
                v = torch.nn.functional.normalize(w.t() @ u, dim=0, eps=self.eps)
                u.copy_(torch.nn.functional.normalize(w @ v, dim=0, eps=self.eps))
        sigma = float(u @ (w @ v))
        wn = session.tensor_mul_scalar(self.inner.weight, c=1.0 / sigma)
        return session.tensor_linear(x, wn, self.inner.bias)


def spectral_norm(session, linear: Linear, n_power_iterations: int = 1) -> SpectralNorm:
    return SpectralNorm(session, linear, n_power_iterations)


# -------------------------------------------------------------------------------------- quantisation
@dataclass
class QParams:
    scale: float
    zero_point: int
    qmin: int = -128
    qmax: int = 127


class MinMaxObserver:
    def __init__(self, qmin: int = -128, qmax: int = 127):
        self.qmin, self.qmax = qmin, qmax
        self.min_val, self.max_val = float("inf"), float("-inf")

    def observe(self, t: torch.Tensor) -> None:
        self.min_val = min(self.min_val, float(t.min()))
        self.max_val = max(self.max_val, float(t.max()))

    def calculate_qparams(self) -> QParams:
        lo, hi = min(self.min_val, 0.0), max(self.max_val, 0.0)
        scale = max((hi - lo) / (self.qmax - self.qmin), 1e-12)
        zp = int(round(self.qmin - lo / scale))
        return QParams(scale, max(self.qmin, min(self.qmax, zp)), self.qmin, self.qmax)


def quantize_per_tensor(t: torch.Tensor, qp: QParams) -> torch.Tensor:
    return torch.clamp(torch.round(t / qp.scale) + qp.zero_point, qp.qmin, qp.qmax).to(torch.int8)


def dequantize(q: torch.Tensor, qp: QParams) -> torch.Tensor:
    return (q.to(torch.float32) - qp.zero_point) * qp.scale


class QuantizedStorageDType(enum.Enum):
    """Physical dtype of packed affine-quantized weights (ft-nn/src/lib.rs:20192)."""
    QInt8 = "qint8"
    QUInt8 = "quint8"

    def qrange(self) -> Tuple[int, int]:
        return (-128, 127) if self is QuantizedStorageDType.QInt8 else (0, 255)

    def torch_dtype(self) -> torch.dtype:
        return torch.int8 if self is QuantizedStorageDType.QInt8 else torch.uint8

    def validate_qparams(self, qp: QParams) -> None:
        if not math.isfinite(qp.scale) or qp.scale <= 0:
            raise ValueError("QuantizedLinear: scale must be finite and > 0")
        if qp.qmin >= qp.qmax:
            raise ValueError("QuantizedLinear: qmin must be < qmax")
        if not qp.qmin <= qp.zero_point <= qp.qmax:
            raise ValueError("QuantizedLinear: zero_point must lie in [qmin, qmax]")
        lo, hi = self.qrange()
        if qp.qmin < lo or qp.qmax > hi:
            raise ValueError("QuantizedLinear: qparams exceed storage dtype range")


@dataclass
class QuantizedLinearQParams:
    """Layout of the weight's quantization parameters (ft-nn/src/lib.rs:20233): one set for the whole tensor, or
    one per slice of ``axis`` (0 = per output feature, 1 = per input feature)."""
    per_tensor: Optional[QParams] = None
    axis: Optional[int] = None
    channels: Optional[List[QParams]] = None

    @staticmethod
    def PerTensor(qp: QParams) -> "QuantizedLinearQParams":
        return QuantizedLinearQParams(per_tensor=qp)

    @staticmethod
    def PerChannel(axis: int, channels: Sequence[QParams]) -> "QuantizedLinearQParams":
        return QuantizedLinearQParams(axis=int(axis), channels=list(channels))

    @property
    def is_per_channel(self) -> bool:
        return self.channels is not None

    def validate(self, dtype: QuantizedStorageDType, in_features: int, out_features: int) -> None:
        if not self.is_per_channel:
            dtype.validate_qparams(self.per_tensor)
            return
        if self.axis not in (0, 1):
            raise ValueError("QuantizedLinear: per-channel axis must be 0 (out_features) or 1 (in_features)")
        want = out_features if self.axis == 0 else in_features
        if len(self.channels) != want:
            raise ValueError(f"QuantizedLinear: {len(self.channels)} channel qparams for {want} channels")
        for qp in self.channels:
            dtype.validate_qparams(qp)

    def broadcast(self, out_features: int, in_features: int, dtype=torch.float64):
        """``(scale, zero_point, qmin, qmax)`` tensors broadcastable against the ``[out, in]`` weight."""
        if not self.is_per_channel:
            q = self.per_tensor
            return (torch.tensor(q.scale, dtype=dtype), torch.tensor(float(q.zero_point), dtype=dtype),
                    torch.tensor(float(q.qmin), dtype=dtype), torch.tensor(float(q.qmax), dtype=dtype))
        shape = (out_features, 1) if self.axis == 0 else (1, in_features)
        col = lambda f: torch.tensor([float(f(q)) for q in self.channels], dtype=dtype).reshape(shape)   # noqa: E731
        return col(lambda q: q.scale), col(lambda q: q.zero_point), col(lambda q: q.qmin), col(lambda q: q.qmax)


class QuantizedLinearWeightStorage:
    """Packed integer codes of a quantized ``[out, in]`` weight (ft-nn/src/lib.rs:20310): int8 or uint8."""

    def __init__(self, dtype: QuantizedStorageDType, codes: torch.Tensor):
        if codes.dtype != dtype.torch_dtype():
            raise ValueError(f"{dtype.name} storage needs {dtype.torch_dtype()} codes")
        self.dtype, self.codes = dtype, codes.contiguous()

    @staticmethod
    def from_float_values(values: torch.Tensor, dtype: QuantizedStorageDType, layout: QuantizedLinearQParams) -> "QuantizedLinearWeightStorage":
        """Round-to-nearest-even affine quantisation, clamped to ``[qmin, qmax]``."""
        w = values.to(torch.float64)
        if not torch.isfinite(w).all():
            raise ValueError("QuantizedLinear: weights must be finite")
        scale, zp, qmin, qmax = layout.broadcast(*w.shape)
        q = torch.minimum(torch.maximum(torch.round(w / scale) + zp, qmin), qmax)
        return QuantizedLinearWeightStorage(dtype, q.to(dtype.torch_dtype()))

    def __len__(self) -> int:
        return self.codes.numel()

    def qint8_values(self) -> Optional[List[int]]:
        return self.codes.reshape(-1).tolist() if self.dtype is QuantizedStorageDType.QInt8 else None

    def quint8_values(self) -> Optional[List[int]]:
        return self.codes.reshape(-1).tolist() if self.dtype is QuantizedStorageDType.QUInt8 else None

    def dequantized(self, layout: QuantizedLinearQParams) -> torch.Tensor:
        scale, zp, _, _ = layout.broadcast(*self.codes.shape)
        return (self.codes.to(torch.float64) - zp) * scale

    def dequantized_values(self, qp: QParams) -> List[float]:
        return self.dequantized(QuantizedLinearQParams.PerTensor(qp)).reshape(-1).tolist()


class QuantizedLinear(Module):
    """Linear layer with an affine-quantized weight.

    Two forms (ft-nn/src/lib.rs:20530):

    * ``QuantizedLinear(session, linear)`` quantizes an existing layer per tensor to int8 and quantizes the
      activations dynamically per call (integer-valued product, fp32 accumulate); its output is a leaf.
    * ``from_float_weights`` / ``from_float_weights_per_channel`` pack given float weights with given quantization
      parameters (int8 or uint8 storage).  The forward dequantizes the weight and runs ``x @ W^T + b`` through the
      session's operators, so a gradient reaches the input; the module has no trainable parameters.
    """

    def __init__(self, session=None, linear: Optional[Linear] = None):
        super().__init__()
        self._packed = None
        if linear is None:
            return
        w = session.tensor(linear.weight).detach().float()
        obs = MinMaxObserver()
        obs.observe(w)
        self.wq_params = obs.calculate_qparams()
        self.wq = quantize_per_tensor(w, self.wq_params)
        self.bias = None if linear.bias is None else session.tensor(linear.bias).detach().float()

    # ------------------------------------------------------------------ packed constructors
    @classmethod
    def _pack(cls, weight_values, bias, in_features, out_features, dtype, layout) -> "QuantizedLinear":
        if in_features <= 0:
            raise ValueError("QuantizedLinear: in_features must be > 0")
        if out_features <= 0:
            raise ValueError("QuantizedLinear: out_features must be > 0")
        w = torch.as_tensor(weight_values, dtype=torch.float64).reshape(-1)
        if w.numel() != in_features * out_features:
            raise ValueError("QuantizedLinear: weight length must equal out_features * in_features")
        if bias is not None and len(bias) != out_features:
            raise ValueError("QuantizedLinear: bias length must equal out_features")
        layout.validate(dtype, in_features, out_features)
        m = cls()
        storage = QuantizedLinearWeightStorage.from_float_values(w.reshape(out_features, in_features), dtype, layout)
        m._packed = (storage, layout, None if bias is None else [float(b) for b in bias], int(in_features), int(out_features))
        return m

    @classmethod
    def from_float_weights(cls, weight_values, bias, in_features: int, out_features: int,
                           weight_dtype: QuantizedStorageDType, weight_qparams: QParams) -> "QuantizedLinear":
        return cls._pack(weight_values, bias, in_features, out_features, weight_dtype,
                         QuantizedLinearQParams.PerTensor(weight_qparams))

    @classmethod
    def from_float_weights_per_channel(cls, weight_values, bias, in_features: int, out_features: int,
                                       weight_dtype: QuantizedStorageDType, channel_axis: int,
                                       channel_qparams: Sequence[QParams]) -> "QuantizedLinear":
        return cls._pack(weight_values, bias, in_features, out_features, weight_dtype,
                         QuantizedLinearQParams.PerChannel(channel_axis, channel_qparams))

    # ------------------------------------------------------------------ accessors of the packed form
    def _need_packed(self):
        if self._packed is None:
            raise ValueError("this QuantizedLinear was built from a Linear layer, not from packed weights")
        return self._packed

    def weight_storage(self) -> QuantizedLinearWeightStorage:
        return self._need_packed()[0]

    def weight_tensor(self) -> torch.Tensor:
        """The integer codes as an ``[out, in]`` tensor."""
        return self._need_packed()[0].codes

    def weight_qparam_layout(self) -> QuantizedLinearQParams:
        return self._need_packed()[1]

    def weight_qparams(self) -> Optional[QParams]:
        return self._need_packed()[1].per_tensor

    def weight_quantization_axis(self) -> Optional[int]:
        return self._need_packed()[1].axis

    def weight_channel_qparams(self) -> Optional[List[QParams]]:
        return self._need_packed()[1].channels

    def bias_values(self) -> Optional[List[float]]:
        return self._need_packed()[2]

    def in_features(self) -> int:
        return self._need_packed()[3]

    def out_features(self) -> int:
        return self._need_packed()[4]

    def parameters(self):
        return []

    # ------------------------------------------------------------------ forward
    def forward(self, session, x):
        if self._packed is not None:
            storage, layout, bias, in_f, out_f = self._packed
            dt = session.tensor_dtype(x)
            w = session.tensor_tape.leaf(storage.dequantized(layout).to(device=session.device, dtype=dt.to_torch()), False)
            y = session.tensor_matmul(x, session.tensor_transpose(w, dim0=0, dim1=1))
            if bias is None:
                return y
            b = session.tensor_tape.leaf(torch.tensor(bias, dtype=dt.to_torch(), device=session.device), False)
            return session.tensor_add(y, b)
        xt = session.tensor(x).detach().float()
        obs = MinMaxObserver()
        obs.observe(xt)
        qp = obs.calculate_qparams()
        xq = quantize_per_tensor(xt, qp)
        acc = (xq.float() - qp.zero_point) @ (self.wq.float() - self.wq_params.zero_point).t()
        y = acc * (qp.scale * self.wq_params.scale)
        if self.bias is not None:
            y = y + self.bias
        return session.tensor_tape.leaf(y.to(session.tensor(x).dtype), False)
