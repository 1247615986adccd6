"""nn utilities: packed sequences, weight / spectral norm, quantisation helpers.

Reference: ft-nn/src/lib.rs - PackedSequence + pack/pad utils :19022-19401, weight_norm /
spectral_norm :19457-19601, QParams / MinMaxObserver / QuantizedLinear :20024-20530.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

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


class QuantizedLinear(Module):
    """int8 weight (per-tensor affine), dynamic per-call activation quantisation, fp32 accumulate."""

    def __init__(self, session, linear: Linear):
        super().__init__()
        w = session.tensor(linear.weight).detach().float()
        obs = MinMaxObserver()
        obs.observe(w)
        self.wq_params = obs.calculate_qparams()
        self.wq = quantize_per_tensor(w, self.wq_params)
        self.bias = None if linear.bias is None else session.tensor(linear.bias).detach().float()

    def forward(self, session, x):
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
