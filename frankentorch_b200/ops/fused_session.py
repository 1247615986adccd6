"""GPU-resident fused operator surface: one object whose methods each launch one sm_100a kernel on tensors
that stay on the device, under the names the reference gives them.

Reference: ft-kernel-metal/src/fused.rs - ``matmul_bias`` :676, ``matmul_bias_w16`` :704 (weight resident at
half width), ``layernorm`` :789, ``gelu`` :816, ``add`` :829, ``softmax`` :842, ``mha`` :857; ft-kernel-metal/src/lib.rs
- ``sgemm`` :284 (host slices in, host slice out), ``is_available`` :196.

The reference keeps activations f32 and converts GEMM operands to f16 per tile; here activations are bf16 end to
end and every GEMM runs on the tcgen05 kernel with an f32 accumulator in tensor memory.  A weight is uploaded
once, transposed to the ``[N, K]`` layout that kernel reads (``GpuWeight``), which is this build's form of the
reference's resident f16 weight.  There is no host fallback inside these methods: without a CUDA device or
without the kernel library they raise, and ``sgemm`` reports ``Unavailable`` so that its caller can pick a host
kernel, as the reference's does.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class FusedUnavailable(RuntimeError):
    """No CUDA device (or no kernel library): the caller falls back to a host kernel."""


class FusedKernelError(ValueError):
    """Operand shapes do not fit the operation."""


def is_available() -> bool:
    if not torch.cuda.is_available():
        return False
    try:
        from . import _lib
        _lib.load()
        return True
    except Exception:
        return False


@dataclass
class GpuWeight:
    """A ``[K, N]`` weight kept on the device as bf16 ``[N, K]`` (unit stride along K), uploaded once."""
    data: torch.Tensor          # [N, K] bf16
    rows: int                   # K
    cols: int                   # N

    @staticmethod
    def upload(w: torch.Tensor, device="cuda:0") -> "GpuWeight":
        if w.dim() != 2:
            raise FusedKernelError(f"a weight is 2-D, got shape {tuple(w.shape)}")
        return GpuWeight(w.t().contiguous().to(device, torch.bfloat16), int(w.shape[0]), int(w.shape[1]))


class FusedSession:
    """Fused device operators on ``[rows, cols]`` bf16 tensors."""

    def __init__(self, device="cuda:0"):
        if not is_available():
            raise FusedUnavailable("no CUDA device or kernel library")
        from . import kernels
        self.K = kernels
        self.device = torch.device(device)

    # -- transfers
    def upload(self, x: torch.Tensor) -> torch.Tensor:
        return x.to(self.device, torch.bfloat16, non_blocking=True).contiguous()

    def weight(self, w: torch.Tensor) -> GpuWeight:
        return GpuWeight.upload(w, self.device)

    def download(self, x: torch.Tensor) -> torch.Tensor:
        return x.to("cpu", torch.float32)

    # -- operators
    def _check_mm(self, a: torch.Tensor, k: int, n: int, bias: Optional[torch.Tensor]) -> None:
        if a.dim() != 2 or a.shape[1] != k:
            raise FusedKernelError(f"matmul_bias: a is {tuple(a.shape)}, the weight is [{k}, {n}]")
        if bias is not None and tuple(bias.shape) != (n,):
            raise FusedKernelError(f"matmul_bias: bias is {tuple(bias.shape)}, expected ({n},)")

    def matmul_bias(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``a [M, K] @ w [K, N] + bias``; ``w`` is a plain device tensor (transposed here, per call)."""
        if w.dim() != 2:
            raise FusedKernelError(f"matmul_bias: w is {tuple(w.shape)}")
        self._check_mm(a, int(w.shape[0]), int(w.shape[1]), bias)
        return self.K.gemm(a, w.t().contiguous(), bias=bias)

    def matmul_bias_w16(self, a: torch.Tensor, w: GpuWeight, bias: Optional[torch.Tensor] = None,
                        gelu: bool = False, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The same over a resident weight: no per-call layout work.  ``gelu`` and ``resid`` fold the activation
        and the residual add into the GEMM epilogue (the reference launches them as separate kernels)."""
        self._check_mm(a, w.rows, w.cols, bias)
        if resid is not None and tuple(resid.shape) != (a.shape[0], w.cols):
            raise FusedKernelError(f"matmul_bias_w16: resid is {tuple(resid.shape)}")
        return self.K.gemm(a, w.data, bias=bias, resid=resid, epi=self.K.EPI_GELU_TANH if gelu else self.K.EPI_NONE)

    def layernorm(self, x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        if x.dim() != 2 or tuple(gamma.shape) != (x.shape[1],) or tuple(beta.shape) != (x.shape[1],):
            raise FusedKernelError("layernorm: gamma and beta have one entry per column of x")
        return self.K.layernorm_fwd(x, gamma, beta, eps)[0]

    def gelu(self, x: torch.Tensor) -> torch.Tensor:
        return self.K.gelu_fwd(x, tanh_form=True)

    def add(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        if a.shape != b.shape:
            raise FusedKernelError(f"add: {tuple(a.shape)} vs {tuple(b.shape)}")
        return self.K.add(a, b)

    def softmax(self, x: torch.Tensor) -> torch.Tensor:
        """Row-wise softmax of a 2-D tensor."""
        if x.dim() != 2:
            raise FusedKernelError("softmax: x is 2-D")
        return self.K.softmax_rows(x)

    def mha(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_heads: int) -> torch.Tensor:
        """Multi-head self-attention over per-token ``[seq, d_model]`` projections, heads concatenated:
        ``concat_h softmax(q_h k_h^T / sqrt(head_dim)) v_h``.  One flash-attention launch; the score matrix is
        never written to memory."""
        if q.dim() != 2 or q.shape != k.shape or q.shape != v.shape:
            raise FusedKernelError("mha: q, k, v are [seq, d_model] of one shape")
        seq, d = int(q.shape[0]), int(q.shape[1])
        if n_heads <= 0 or d % n_heads:
            raise FusedKernelError(f"mha: d_model {d} is not divisible by {n_heads} heads")
        hd = d // n_heads
        view = lambda t: t.contiguous().view(1, seq, n_heads, hd)   # noqa: E731
        out, _ = self.K.attention_fwd(view(q), view(k), view(v), causal=False)
        return out.view(seq, d)

    def finish(self) -> None:
        """Wait for the queued kernels and raise if one of them reported a bounded-wait timeout."""
        torch.cuda.synchronize(self.device)
        self.K.check_status()


def sgemm(a, b, m: int, k: int, n: int, device="cuda:0") -> torch.Tensor:
    """``c [m, n] = a [m, k] @ b [k, n]`` for host arrays (flat or shaped), result on the host as f32.  Operands
    are rounded to bf16 on upload; the accumulator is f32.  Raises ``FusedUnavailable`` without a device."""
    a = torch.as_tensor(a, dtype=torch.float32).reshape(-1)
    b = torch.as_tensor(b, dtype=torch.float32).reshape(-1)
    if a.numel() != m * k or b.numel() != k * n:
        raise FusedKernelError(f"shape mismatch: a={a.numel()} (want {m * k}), b={b.numel()} (want {k * n})")
    if not is_available():
        raise FusedUnavailable("no CUDA device or kernel library")
    s = FusedSession(device)
    out = s.K.gemm(s.upload(a.view(m, k)), GpuWeight.upload(b.view(k, n), s.device).data, out_dtype=torch.float32)
    s.finish()
    return out.to("cpu")
