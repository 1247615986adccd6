"""Python launchers for the sm_100a kernels (``torch.Tensor`` in, ``torch.Tensor`` out).

Every function enqueues on the current CUDA stream and returns immediately; none
of them falls back to a PyTorch implementation.  ``check_status()`` reads the
device status word that the kernels' bounded waits report into.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import FtkAttnDesc, FtkGemmDesc

EPI_NONE, EPI_GELU_TANH, EPI_GELU_ERF, EPI_RELU = 0, 1, 2, 3
EPI_MUL_DGELU_TANH, EPI_MUL_DGELU_ERF, EPI_MUL_DRELU = 4, 5, 6

_STATUS_NAMES = {
    1: "WAIT_FULL (TMA data never landed)", 2: "WAIT_EMPTY (stage never released)",
    3: "WAIT_TMEM_FULL (accumulator never completed)", 4: "WAIT_TMEM_EMPTY (accumulator never drained)",
    5: "WAIT_PEER (peer flag never arrived)", 6: "WAIT_SOFTMAX (probabilities never arrived)",
    7: "BAD_ARG (misaligned shared memory or invalid argument)",
    8: "WAIT_WARPS (a warp barrier was abandoned after an abort elsewhere in the CTA)",
    9: "BAD_INDEX (an index read from a tensor, e.g. a token id, was out of range; the access was skipped)",
}

# launch counter: how many of this package's kernels launchers were called (bench reporting)
_launches = 0


class KernelError(RuntimeError):
    """A launcher rejected its arguments or a kernel reported a failed bounded wait."""


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# optional launch trace: while a list is installed, every launcher call appends its name (GEMMs with the tile
# the planner picked); the training engine uses it to put the kernels of a step on the evidence ledger
_TRACE: Optional[list] = None


def trace_begin() -> None:
    global _TRACE
    _TRACE = []


def trace_take() -> list:
    """The launcher calls since the last take (or since ``trace_begin``); empties the trace."""
    global _TRACE
    if _TRACE is None:
        return []
    out, _TRACE = _TRACE, []
    return out


def trace_end() -> list:
    global _TRACE
    out, _TRACE = (_TRACE or []), None
    return out


def _chk(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if _TRACE is not None:
        _TRACE.append(what)
    if rc != 0:
        raise KernelError(f"{what}: launcher returned {rc}")


def check_status(reset: bool = True) -> None:
    """Synchronise and raise if any kernel recorded a protocol failure."""
    v = _lib.load().ftk_read_status(1 if reset else 0)
    if v != 0:
        code, cta = v & 0xFF, v >> 8
        raise KernelError(f"device status {v}: {_STATUS_NAMES.get(code, 'unknown')} (CTA {cta})")


def _bf16(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA bf16 tensor, got {t.dtype} on {t.device}")


# --------------------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
         aux: Optional[torch.Tensor] = None, epi: int = EPI_NONE, alpha: float = 1.0,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, force_bn: int = 0, max_ctas: int = 0, split_k: int = 0,
         reduce_stream: Optional[int] = None, seg_counts: Optional[torch.Tensor] = None,
         seg_rows: int = 0) -> torch.Tensor:
    """``D = epi(alpha * A @ B^T + bias) (+ resid) (+ D)`` on the tcgen05 GEMM.

    ``a`` is ``[M, K]`` (``a_mn=False``) or ``[K, M]`` (``a_mn=True``); ``b`` is
    ``[N, K]`` or ``[K, N]`` likewise.  Both must be bf16 with unit inner stride.
    ``reduce_stream`` (a raw stream handle) moves a split-K reduction off the launching stream;
    the caller joins that stream before reading the output or launching the next split-K GEMM.
    ``seg_counts`` (int32, device) with ``seg_rows``: the rows are segments of ``seg_rows`` rows of which
    only the first ``seg_counts[s]`` are in use; 128-row tiles without a used row are skipped and
    their output rows are left as they were (expert batches with capacity padding).
    """
    _bf16(a, "a"), _bf16(b, "b")
    if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
        raise KernelError("gemm operands must be 2-D with unit inner stride")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise KernelError(f"gemm K mismatch: {K} vs {Kb}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise KernelError("gemm output must be [M, N] with unit inner stride")
    g = FtkGemmDesc()
    g.M, g.N, g.K, g.L0, g.L1 = M, N, K, 1, 1
    g.a_mn, g.b_mn = int(a_mn), int(b_mn)
    g.A, g.lda = a.data_ptr(), a.stride(0)
    g.B, g.ldb = b.data_ptr(), b.stride(0)
    g.D, g.ldd = out.data_ptr(), out.stride(0)
    g.bias = _ptr(bias)
    if resid is not None:
        _bf16(resid, "resid")
        g.resid, g.ldr = resid.data_ptr(), resid.stride(0)
    if aux is not None:
        _bf16(aux, "aux")
        if aux.stride(0) != out.stride(0):
            raise KernelError("aux must share the row stride of the output")
        g.aux = aux.data_ptr()
    g.alpha, g.epi = float(alpha), int(epi)
    g.out_fp32 = 1 if out.dtype == torch.float32 else 0
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm output must be bf16 or fp32")
    g.accumulate, g.force_bn, g.max_ctas = int(accumulate), int(force_bn), int(max_ctas)
    g.split_k = int(split_k)
    g.reduce_stream = reduce_stream
    if seg_counts is not None:
        if seg_counts.dtype != torch.int32 or not seg_counts.is_cuda or seg_rows <= 0:
            raise KernelError("seg_counts must be a CUDA int32 tensor and seg_rows positive")
        if a_mn or seg_counts.numel() < -(-M // seg_rows):
            raise KernelError("seg_counts needs one entry per segment of rows of a row-major A operand")
        g.seg_counts, g.seg_rows = seg_counts.data_ptr(), int(seg_rows)
    lib = _lib.load()
    dev_key = a.device.index if a.device.index is not None else torch.cuda.current_device()
    if split_k != 1 and bias is None and resid is None and aux is None and epi == EPI_NONE:
        ws = _gemm_workspace(a.device)
        g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel() * 4
        busy = _WS_BUSY.get(dev_key)
        if busy is not None or reduce_stream is not None:
            bn, sp = C.c_int(0), C.c_int(1)
            lib.ftk_gemm_plan(C.byref(g), C.byref(bn), C.byref(sp))
            if sp.value > 1:
                if busy is not None:
                    # a reduction on another stream still reads the split-K workspace this GEMM will write
                    torch.cuda.current_stream(a.device).wait_event(busy)
                    _WS_BUSY.pop(dev_key, None)
            else:
                g.reduce_stream = reduce_stream = None
    what = "ftk_gemm_bf16"
    if _TRACE is not None:          # name the tile the planner picks for this problem
        bn, sp = C.c_int(0), C.c_int(1)
        if lib.ftk_gemm_plan(C.byref(g), C.byref(bn), C.byref(sp)) == 0:
            what = ("ftk::gemm2_bf16_sm100<256x256,cta_group2,splitK=%d>" % sp.value) if bn.value == 512 else \
                ("ftk::gemm_bf16_sm100<128x%d,splitK=%d>" % (bn.value, sp.value))
    _chk(lib.ftk_gemm_bf16(C.byref(g), _stream()), what)
    if reduce_stream is not None and g.workspace:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.ExternalStream(reduce_stream, device=a.device))
        _WS_BUSY[dev_key] = ev
    return out


def gemm_grouped(problems, *, a_mn: bool = True, b_mn: bool = True, max_ctas: int = 0) -> None:
    """Several products with one reduction length in one launch: ``problems`` is a sequence of
    ``(a, b, out, accumulate)`` with ``out`` fp32 ``[M_p, N_p]`` (``+=`` when ``accumulate``); operands as in
    :func:`gemm` (the default layouts are those of a weight gradient, ``dW = dy^T x`` with ``a = dy [K, M]``,
    ``b = x [K, N]``).  At most eight problems; every output element is reduced over K by one CTA, in order."""
    n = len(problems)
    if not 1 <= n <= 8:
        raise KernelError("gemm_grouped takes 1 to 8 problems")
    arr = (FtkGemmDesc * n)()
    Kd = None
    for g, (a, b, out, accumulate) in zip(arr, problems):
        _bf16(a, "a"), _bf16(b, "b")
        if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
            raise KernelError("gemm operands must be 2-D with unit inner stride")
        M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
        N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
        if K != Kb or (Kd is not None and K != Kd):
            raise KernelError("gemm_grouped: all problems share one reduction length")
        Kd = K
        if out.dtype != torch.float32 or out.shape != (M, N) or out.stride(1) != 1:
            raise KernelError("gemm_grouped outputs are fp32 [M, N] with unit inner stride")
        g.M, g.N, g.K, g.L0, g.L1 = M, N, K, 1, 1
        g.a_mn, g.b_mn = int(a_mn), int(b_mn)
        g.A, g.lda = a.data_ptr(), a.stride(0)
        g.B, g.ldb = b.data_ptr(), b.stride(0)
        g.D, g.ldd = out.data_ptr(), out.stride(0)
        g.alpha, g.out_fp32, g.accumulate, g.max_ctas = 1.0, 1, int(bool(accumulate)), int(max_ctas)
    _chk(_lib.load().ftk_gemm_group_bf16(arr, n, _stream()),
         "ftk::gemm_group_bf16_sm100<128x192,problems=%d>" % n)


_WORKSPACES = {}
GEMM_WORKSPACE_BYTES = 64 << 20
# per device: event recorded behind a split-K reduction that runs on a stream other than its GEMM's;
# the next split-K GEMM waits for it, and whoever joins that stream calls workspace_idle()
_WS_BUSY = {}


def workspace_idle(device) -> None:
    """The caller has joined the stream that ran split-K reductions: the workspace is free again."""
    key = device.index if getattr(device, "index", None) is not None else torch.cuda.current_device()
    _WS_BUSY.pop(key, None)


def _gemm_workspace(device) -> torch.Tensor:
    """Per-device fp32 scratch for split-K partial tiles (allocated once, outside any capture)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.empty(GEMM_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        _WORKSPACES[key] = ws
    return ws


def gemm_batched(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, M: int, N: int, K: int,
                 L0: int, L1: int, a_strides: Tuple[int, int, int], b_strides: Tuple[int, int, int],
                 d_strides: Tuple[int, int, int], a_mn: bool = False, b_mn: bool = False,
                 alpha: float = 1.0, a_offset: int = 0, b_offset: int = 0, d_offset: int = 0) -> torch.Tensor:
    """Strided-batched GEMM over ``L0*L1`` problems; strides are (row, l0, l1) in elements."""
    _bf16(a, "a"), _bf16(b, "b")
    g = FtkGemmDesc()
    g.M, g.N, g.K, g.L0, g.L1 = M, N, K, L0, L1
    g.a_mn, g.b_mn = int(a_mn), int(b_mn)
    es = a.element_size()
    g.A, (g.lda, g.a_s0, g.a_s1) = a.data_ptr() + a_offset * es, a_strides
    g.B, (g.ldb, g.b_s0, g.b_s1) = b.data_ptr() + b_offset * es, b_strides
    g.D, (g.ldd, g.d_s0, g.d_s1) = out.data_ptr() + d_offset * out.element_size(), d_strides
    g.alpha = float(alpha)
    g.out_fp32 = 1 if out.dtype == torch.float32 else 0
    _chk(_lib.load().ftk_gemm_bf16(C.byref(g), _stream()), "ftk_gemm_bf16(batched)")
    return out


def linear_fwd(x, w, bias=None, *, epi=EPI_NONE, resid=None, aux=None, out=None, seg_counts=None, seg_rows=0):
    """``y = epi(x @ w^T + bias) (+ resid)`` with ``w`` stored ``[out, in]``."""
    return gemm(x, w, bias=bias, epi=epi, resid=resid, aux=aux, out=out, seg_counts=seg_counts, seg_rows=seg_rows)


def linear_dgrad(dy, w, *, epi=EPI_NONE, resid=None, out=None, seg_counts=None, seg_rows=0):
    """``dx = dy @ w`` (``w`` is ``[out, in]``; consumed as an MN-major operand)."""
    return gemm(dy, w, b_mn=True, epi=epi, resid=resid, out=out, seg_counts=seg_counts, seg_rows=seg_rows)


def linear_wgrad(dy, x, *, out=None, accumulate=False, reduce_stream=None):
    """``dw[out, in] (+)= dy^T @ x`` in fp32; both operands are consumed MN-major."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, out_dtype=torch.float32, accumulate=accumulate,
                reduce_stream=reduce_stream)


# --------------------------------------------------------------------------------------- attention
def _attn_desc(q, k, v, o, lse, causal, scale):
    # q/k/v/o: views of shape [B, S, H, hd] (any strides with unit inner stride)
    B, S, H, hd = q.shape
    d = FtkAttnDesc()
    d.B, d.H, d.S, d.hd, d.causal = B, H, S, hd, int(causal)
    d.scale = float(scale if scale is not None else 1.0 / math.sqrt(hd))
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
        _bf16(t, name)
        if t.shape != q.shape or t.stride(3) != 1:
            raise KernelError(f"attention operand {name} must be [B,S,H,hd] with unit inner stride")
        setattr(d, name, t.data_ptr())
        setattr(d, name + "_bs", t.stride(0))
        setattr(d, name + "_ss", t.stride(1))
        setattr(d, name + "_hs", t.stride(2))
    d.lse = lse.data_ptr()
    return d


def attention_fwd(q, k, v, *, causal=True, scale=None, out=None):
    """Flash attention forward.  q/k/v: ``[B, S, H, hd]`` bf16 views.  Returns ``(o, lse)``."""
    B, S, H, hd = q.shape
    if out is None:
        out = torch.empty((B, S, H, hd), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    d = _attn_desc(q, k, v, out, lse, causal, scale)
    _chk(_lib.load().ftk_attn_fwd(C.byref(d), _stream()), "ftk_attn_fwd")
    return out, lse


def attention_bwd(q, k, v, o, lse, d_o, *, causal=True, scale=None, dq=None, dk=None, dv=None):
    """Flash attention backward; returns ``(dq, dk, dv)`` laid out like q/k/v."""
    B, S, H, hd = q.shape
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    for name, t, ref in (("dq", dq, q), ("dk", dk, k), ("dv", dv, v), ("d_o", d_o, o)):
        if t.stride() != ref.stride():
            raise KernelError(f"{name} must share the strides of its primal")
    delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    d = _attn_desc(q, k, v, o, lse, causal, scale)
    d.d_o, d.delta = d_o.data_ptr(), delta.data_ptr()
    d.dq, d.dk, d.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    _chk(_lib.load().ftk_attn_bwd(C.byref(d), _stream()), "ftk_attn_bwd")
    return dq, dk, dv


# --------------------------------------------------------------------------------------- norms
def layernorm_fwd(x, gamma, beta, eps=1e-5, resid=None, out=None):
    """Returns ``(y, mean, rstd, x_sum)``; ``x_sum`` is ``x + resid`` when ``resid`` is given."""
    rows, cols = x.shape
    y = torch.empty_like(x) if out is None else out
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    xs = torch.empty_like(x) if resid is not None else None
    _chk(_lib.load().ftk_layernorm_fwd(x.data_ptr(), _ptr(resid), _ptr(xs), gamma.data_ptr(),
                                       _ptr(beta), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                       rows, cols, float(eps), _stream()), "ftk_layernorm_fwd")
    return y, mean, rstd, (xs if resid is not None else x)


def layernorm_bwd(dy, x, gamma, mean, rstd, *, dx_add=None, dgamma=None, dbeta=None, accumulate=False,
                  out=None):
    rows, cols = x.shape
    lib = _lib.load()
    dx = torch.empty_like(x) if out is None else out
    if dgamma is None:
        dgamma = torch.empty(cols, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(cols, dtype=torch.float32, device=x.device)
        accumulate = False
    nblk = lib.ftk_layernorm_bwd_blocks(rows)
    partial = torch.empty(2 * nblk * cols, dtype=torch.float32, device=x.device)
    _chk(lib.ftk_layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                               rstd.data_ptr(), _ptr(dx_add), dx.data_ptr(), dgamma.data_ptr(),
                               dbeta.data_ptr(), partial.data_ptr(), rows, cols, int(accumulate),
                               _stream()), "ftk_layernorm_bwd")
    return dx, dgamma, dbeta


def rmsnorm_fwd(x, gamma, eps=1e-6):
    rows, cols = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _chk(_lib.load().ftk_rmsnorm_fwd(x.data_ptr(), gamma.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                                     rows, cols, float(eps), _stream()), "ftk_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy, x, gamma, rstd, *, dgamma=None, accumulate=False):
    rows, cols = x.shape
    lib = _lib.load()
    dx = torch.empty_like(x)
    if dgamma is None:
        dgamma = torch.empty(cols, dtype=torch.float32, device=x.device)
        accumulate = False
    nblk = lib.ftk_layernorm_bwd_blocks(rows)
    partial = torch.empty(nblk * cols, dtype=torch.float32, device=x.device)
    _chk(lib.ftk_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), rstd.data_ptr(),
                             dx.data_ptr(), dgamma.data_ptr(), partial.data_ptr(), rows, cols,
                             int(accumulate), _stream()), "ftk_rmsnorm_bwd")
    return dx, dgamma


def softmax_rows(x):
    rows, cols = x.shape
    y = torch.empty_like(x)
    _chk(_lib.load().ftk_softmax_rows(x.data_ptr(), y.data_ptr(), rows, cols,
                                      int(x.dtype == torch.bfloat16), _stream()), "ftk_softmax_rows")
    return y


def softmax_causal(x, scale=1.0):
    L, S, S2 = x.shape
    y = torch.empty_like(x)
    _chk(_lib.load().ftk_softmax_causal_bf16(x.data_ptr(), y.data_ptr(), L, S, float(scale), _stream()),
         "ftk_softmax_causal_bf16")
    return y


def softmax_bwd(y, dy, scale=1.0):
    cols = y.shape[-1]
    rows = y.numel() // cols
    dx = torch.empty_like(y)
    _chk(_lib.load().ftk_softmax_bwd_bf16(y.data_ptr(), dy.data_ptr(), dx.data_ptr(), rows, cols,
                                          float(scale), _stream()), "ftk_softmax_bwd_bf16")
    return dx


# --------------------------------------------------------------------------------------- loss
def cross_entropy_fwd_bwd(logits, targets, vocab, grad_scale, *, want_grad=True, inplace=True):
    """Per-row losses (fp32) and, optionally, ``dlogits = (softmax - onehot) * grad_scale``.

    ``logits`` is ``[rows, ld]`` bf16 with ``ld >= vocab`` (padding columns ignored).
    With ``inplace`` the gradient overwrites ``logits``.
    """
    rows, ld = logits.shape
    losses = torch.empty(rows, dtype=torch.float32, device=logits.device)
    dl = None
    if want_grad:
        dl = logits if inplace else torch.empty_like(logits)
    _chk(_lib.load().ftk_cross_entropy_fwd_bwd(logits.data_ptr(), targets.data_ptr(), losses.data_ptr(),
                                               _ptr(dl), rows, vocab, ld, float(grad_scale), _stream()),
         "ftk_cross_entropy_fwd_bwd")
    return losses, dl


def reduce_mean(x, scale=None, out=None):
    n = x.numel()
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    _chk(_lib.load().ftk_reduce_mean_f32(x.data_ptr(), out.data_ptr(), n,
                                         float(1.0 / n if scale is None else scale), _stream()),
         "ftk_reduce_mean_f32")
    return out


def sumsq(x, out=None, accumulate=False):
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    partial = torch.empty(1024, dtype=torch.float32, device=x.device)
    _chk(_lib.load().ftk_sumsq_f32(x.data_ptr(), out.data_ptr(), partial.data_ptr(), x.numel(),
                                   int(accumulate), _stream()), "ftk_sumsq_f32")
    return out


# --------------------------------------------------------------------------------------- elementwise
def gelu_fwd(x, tanh_form=True):
    y = torch.empty_like(x)
    _chk(_lib.load().ftk_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), int(tanh_form), _stream()), "ftk_gelu_fwd")
    return y


def gelu_bwd(x, dy, tanh_form=True):
    dx = torch.empty_like(x)
    _chk(_lib.load().ftk_gelu_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), int(tanh_form), _stream()),
         "ftk_gelu_bwd")
    return dx


def add(a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    _chk(_lib.load().ftk_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "ftk_add_bf16")
    return out


def cast_f32_to_bf16(x, out=None):
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if out is None else out
    _chk(_lib.load().ftk_cast_f32_to_bf16(x.data_ptr(), out.data_ptr(), x.numel(), _stream()), "ftk_cast_f32_to_bf16")
    return out


def cast_bf16_to_f32(x, out=None, accumulate=False):
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device) if out is None else out
    _chk(_lib.load().ftk_cast_bf16_to_f32(x.data_ptr(), out.data_ptr(), x.numel(), int(accumulate), _stream()),
         "ftk_cast_bf16_to_f32")
    return out


def dropout(x, p, seed, offset=0):
    y = torch.empty_like(x)
    _chk(_lib.load().ftk_dropout_bf16(x.data_ptr(), y.data_ptr(), x.numel(), float(p), int(seed), int(offset), _stream()),
         "ftk_dropout_bf16")
    return y


def colsum(x, out=None, accumulate=False):
    """fp32 column sums of a bf16 ``[rows, cols]`` matrix (bias gradient), fixed order."""
    rows, cols = x.shape
    lib = _lib.load()
    if out is None:
        out = torch.empty(cols, dtype=torch.float32, device=x.device)
        accumulate = False
    partial = torch.empty(lib.ftk_colsum_blocks(rows) * cols, dtype=torch.float32, device=x.device)
    _chk(lib.ftk_colsum_bf16(x.data_ptr(), out.data_ptr(), partial.data_ptr(), rows, cols, x.stride(0),
                             int(accumulate), _stream()), "ftk_colsum_bf16")
    return out


# --------------------------------------------------------------------------------------- embedding
def embedding_fwd(ids, wte, wpe, S):
    rows = ids.numel()
    d = wte.shape[1]
    out = torch.empty((rows, d), dtype=torch.bfloat16, device=wte.device)
    _chk(_lib.load().ftk_embedding_fwd(ids.data_ptr(), wte.data_ptr(), _ptr(wpe), out.data_ptr(), rows, S, d,
                                       wte.shape[0], _stream()), "ftk_embedding_fwd")
    return out


def embedding_bwd(ids, dout, dwte, dwpe, S, *, sorted_form: bool = False):
    """Deterministic scatter-add of ``dout`` rows into fp32 ``dwte`` / ``dwpe`` (both ``+=``).

    Every table row is summed by one CTA in ascending position order, so the result does not depend on
    scheduling.  The default form needs no sort: the CTA of a token's first occurrence scans the later positions
    for the same token.  ``sorted_form`` (and tables wider than 1024 columns) groups the rows with a stable sort
    first; both forms give the same bits.
    """
    rows, d = dout.shape
    flat = ids.reshape(-1)
    vocab = dwte.shape[0] if dwte is not None else 0
    if not sorted_form and d <= 1024 and flat.dtype == torch.int64 and flat.is_contiguous():
        _chk(_lib.load().ftk_embedding_bwd_scan(flat.data_ptr(), dout.data_ptr(), _ptr(dwte), _ptr(dwpe), rows, S, d,
                                                vocab, _stream()), "ftk_embedding_bwd_scan")
        return
    sorted_ids, order = torch.sort(flat, stable=True)
    order32 = order.to(torch.int32)
    _chk(_lib.load().ftk_embedding_bwd(sorted_ids.data_ptr(), order32.data_ptr(), dout.data_ptr(),
                                       _ptr(dwte), _ptr(dwpe), rows, S, d, vocab, _stream()), "ftk_embedding_bwd")


# --------------------------------------------------------------------------------------- optimizer
def adamw(master, shadow, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    _chk(_lib.load().ftk_adamw(master.data_ptr(), _ptr(shadow), grad.data_ptr(), m.data_ptr(), v.data_ptr(),
                               master.numel(), float(lr), float(beta1), float(beta2), float(eps),
                               float(weight_decay), float(bc1), float(bc2), float(grad_scale), _stream()),
         "ftk_adamw")


def adamw_tick(step_dev, hyper_dev, beta1, beta2):
    """Advance the device-resident step counter and bias corrections (graph replayable)."""
    _chk(_lib.load().ftk_adamw_tick(step_dev.data_ptr(), hyper_dev.data_ptr(), float(beta1), float(beta2),
                                    _stream()), "ftk_adamw_tick")


def clip_scale(sumsq_dev, max_norm, hyper_dev, norm_out=None):
    _chk(_lib.load().ftk_clip_scale(sumsq_dev.data_ptr(), float(max_norm), hyper_dev.data_ptr(),
                                    _ptr(norm_out), _stream()), "ftk_clip_scale")


def adamw_dev(master, shadow, grad, m, v, hyper_dev, *, beta1, beta2, eps, weight_decay):
    """AdamW with lr / bias corrections / gradient scale read from device memory."""
    _chk(_lib.load().ftk_adamw_dev(master.data_ptr(), _ptr(shadow), grad.data_ptr(), m.data_ptr(),
                                   v.data_ptr(), master.numel(), hyper_dev.data_ptr(), float(beta1),
                                   float(beta2), float(eps), float(weight_decay), _stream()), "ftk_adamw_dev")


def fill_f32(x, value=0.0):
    _chk(_lib.load().ftk_fill_f32(x.data_ptr(), x.numel(), float(value), _stream()), "ftk_fill_f32")


def timestamp(out: torch.Tensor, index: int = 0, stream: Optional[int] = None) -> None:
    """Store the GPU nanosecond timer into ``out[index]`` (int64) when the stream gets here."""
    _chk(_lib.load().ftk_timestamp(out.data_ptr() + 8 * index, _stream() if stream is None else stream),
         "ftk_timestamp")


# --------------------------------------------------------------------------------------- misc
def present_rgba8(src, width, height, row_bytes, half=False):
    dst = torch.empty((height, width, 4), dtype=torch.float16 if half else torch.float32, device=src.device)
    _chk(_lib.load().ftk_present_rgba8(src.data_ptr(), dst.data_ptr(), width, height, row_bytes, int(half), _stream()),
         "ftk_present_rgba8")
    return dst


def im2col_1d(x, k, stride=1, pad=0):
    t_in, cin = x.shape
    t_out = (t_in + 2 * pad - k) // stride + 1
    y = torch.empty((t_out, cin * k), dtype=torch.float32, device=x.device)
    _chk(_lib.load().ftk_im2col_1d(x.data_ptr(), y.data_ptr(), t_in, cin, k, stride, pad, t_out, _stream()),
         "ftk_im2col_1d")
    return y
