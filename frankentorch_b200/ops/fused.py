"""Tape-recording fused operators of the sm_100a backend.

Each function runs the forward kernel(s), appends ONE node to the tape and attaches a
VJP rule that launches the matching backward kernels.  The rule strings are the
reference's (`rule` field of every backward step, ft-autograd/src/lib.rs:11807-15602)
where the op exists there, extended with the fused epilogue in brackets.

Parameter gradients are written in place into the leaf's bound fp32 gradient buffer
(``TensorTape.bind_grad_buffer``) by the wgrad GEMM epilogue (``accumulate`` when the
buffer already holds a contribution), so no temporary dW tensor is materialised.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..autograd.tape import ACCUMULATED, TensorTape
from . import kernels as K

RULE_LINEAR = "d(A@B)/dA=dOut@B^T; d(A@B)/dB=A^T@dOut"


class SideWork:
    """Small memory-bound kernels of a backward rule (bias column sums, split-K reductions) run on a
    second stream next to the rule's GEMMs and are joined before the rule returns.

    Entering makes the side stream wait for everything the main stream holds (the incoming gradient
    is complete); leaving makes the main stream wait for the side stream, and only then tells the
    tape's observer which parameter gradients were written (a data-parallel bucket must not start
    before the split-K reduction that finishes its last gradient).  Nothing about the arithmetic
    changes: the same kernels see the same data.  Works eagerly and under CUDA-graph capture (the
    fork and the join are captured as parallel branches).  ``FT_SIDE_STREAM=0`` keeps everything on
    one stream."""

    _streams = {}
    enabled = os.environ.get("FT_SIDE_STREAM", "1") != "0"

    def __init__(self, tape: TensorTape, device: torch.device):
        self.tape, self.device = tape, device
        self.on = SideWork.enabled and device.type == "cuda"
        self._marks = []
        self._saved_fn = None

    @classmethod
    def stream_for(cls, device: torch.device) -> torch.cuda.Stream:
        key = device.index if device.index is not None else torch.cuda.current_device()
        if key not in cls._streams:
            cls._streams[key] = torch.cuda.Stream(device=device)
        return cls._streams[key]

    def __enter__(self):
        if self.on:
            self.main = torch.cuda.current_stream(self.device)
            self.side = SideWork.stream_for(self.device)
            ev = torch.cuda.Event()
            ev.record(self.main)
            self.side.wait_event(ev)
            self._saved_fn = self.tape.leaf_grad_written_fn
            if self._saved_fn is not None:
                self.tape.leaf_grad_written_fn = self._marks.append      # held back until the join
        return self

    def __exit__(self, *exc):
        if self.on:
            ev = torch.cuda.Event()
            ev.record(self.side)
            self.main.wait_event(ev)
            K.workspace_idle(self.device)
            self.tape.leaf_grad_written_fn = self._saved_fn
            if self._saved_fn is not None and exc[0] is None:
                for nid in self._marks:
                    self._saved_fn(nid)
        return False

    def wgrad(self, dy2d, x2d, out=None, accumulate=False):
        """Weight gradient GEMM on the main stream; its split-K reduction (if any) on the side stream."""
        if not self.on:
            return K.linear_wgrad(dy2d, x2d, out=out, accumulate=accumulate)
        return K.linear_wgrad(dy2d, x2d, out=out, accumulate=accumulate, reduce_stream=self.side.cuda_stream)

    def colsum(self, dy2d, out=None, accumulate=False):
        if not self.on:
            return K.colsum(dy2d, out=out, accumulate=accumulate)
        with torch.cuda.stream(self.side):
            return K.colsum(dy2d, out=out, accumulate=accumulate)


class WgradQueue:
    """Weight gradients of consecutive backward rules, collected and launched together.

    A weight gradient ``dW = dy^T x`` of a transformer block has 24 - 96 output tiles: alone it needs split-K
    and a reduction kernel to occupy 148 SMs.  The four of a block together are two full waves of 128 x 192
    tiles (``K.gemm_grouped``), each output element reduced over the tokens by one CTA in order.  A rule hands
    its weight gradient to the queue instead of launching it; the queue launches when it holds enough tiles
    (or eight problems) and when the backward pass ends (``TensorTape.backward`` calls :meth:`flush`).  The
    operands stay referenced until then; nothing in a backward pass writes them in place.  The observer of
    finished parameter gradients (data-parallel buckets) is told at the launch, not when a rule queued its
    part.  Large products (the LM head) and gradients without a bound buffer keep the direct path.
    ``FT_WGRAD_GROUP=0`` turns the queue off."""

    enabled = os.environ.get("FT_WGRAD_GROUP", "1") != "0"
    FLUSH_TILES = 266          # ~0.9 x two waves of 148
    MAX_TILES_PER_PROBLEM = 200

    def __init__(self, tape: TensorTape):
        self.tape = tape
        self.items = []        # (dy, x, buf, accumulate, leaf id)
        self.tiles = 0
        self.launches = 0

    @staticmethod
    def tiles_of(M: int, N: int) -> int:
        return -(-M // 128) * -(-N // 192)

    def accepts(self, dy2d, x2d) -> bool:
        if not (dy2d.is_cuda and dy2d.dtype == torch.bfloat16 and x2d.dtype == torch.bfloat16):
            return False
        if dy2d.stride(1) != 1 or x2d.stride(1) != 1 or dy2d.stride(0) % 8 or x2d.stride(0) % 8:
            return False
        if dy2d.data_ptr() % 16 or x2d.data_ptr() % 16:
            return False
        return self.tiles_of(dy2d.shape[1], x2d.shape[1]) <= self.MAX_TILES_PER_PROBLEM

    def add(self, dy2d, x2d, buf, accumulate: bool, nid: int) -> None:
        if self.items and (self.items[0][0].shape[0] != dy2d.shape[0] or any(it[4] == nid for it in self.items)):
            self.flush()       # another reduction length, or a second contribution to the same buffer
        self.items.append((dy2d, x2d, buf, accumulate, nid))
        self.tiles += self.tiles_of(dy2d.shape[1], x2d.shape[1])
        if self.tiles >= self.FLUSH_TILES or len(self.items) == 8:
            self.flush()

    def flush(self) -> None:
        if not self.items:
            return
        items, self.items, self.tiles = self.items, [], 0
        K.gemm_grouped([(dy, x, buf, acc) for dy, x, buf, acc, _ in items])
        self.launches += 1
        fn = self.tape.leaf_grad_written_fn
        if fn is not None:
            for it in items:
                fn(it[4])


def enable_grouped_wgrad(tape: TensorTape) -> bool:
    """Give ``tape`` a :class:`WgradQueue` (the fused rules use it when present).  Returns whether it is on."""
    if WgradQueue.enabled and getattr(tape, "wgrad_queue", None) is None:
        tape.wgrad_queue = WgradQueue(tape)
    return getattr(tape, "wgrad_queue", None) is not None


def _wgrad_into(targets, idx, dy2d, x2d, side: Optional["SideWork"] = None):
    """dW (+)= dy^T x, written into the bound gradient buffer when there is one."""
    run = side.wgrad if side is not None else K.linear_wgrad
    tgt = targets.leaf_target(idx)
    queue = getattr(targets._tape, "wgrad_queue", None)
    if tgt is not None and queue is not None and queue.accepts(dy2d, x2d):
        buf, filled = tgt
        nid = targets._node.inputs[idx]
        targets._tape.nodes[nid].grad_buffer_filled = True       # the observer hears of it at the launch
        queue.add(dy2d, x2d, buf, filled, nid)
        return ACCUMULATED
    if tgt is not None:
        buf, filled = tgt
        run(dy2d, x2d, out=buf, accumulate=filled)
        targets.mark_accumulated(idx)
        return ACCUMULATED
    return run(dy2d, x2d)


def _bgrad_into(targets, idx, dy2d, side: Optional["SideWork"] = None):
    run = side.colsum if side is not None else K.colsum
    tgt = targets.leaf_target(idx)
    if tgt is not None:
        buf, filled = tgt
        run(dy2d, out=buf, accumulate=filled)
        targets.mark_accumulated(idx)
        return ACCUMULATED
    return run(dy2d)


def linear(tape: TensorTape, x: int, w: int, b: Optional[int] = None, *, act: Optional[str] = None,
           resid: Optional[int] = None) -> int:
    """``y = act(x @ w^T + b) (+ resid)``; ``w`` is ``[out, in]`` (ft-nn/src/lib.rs:902).

    ``act`` in ``{None, "gelu_tanh", "gelu_erf", "relu"}``.  With an activation the
    pre-activation is kept (bf16) for the backward epilogue ``dU = (dY W2) * act'(U)``.
    """
    xv, wv = tape.value(x), tape.value(w)
    bv = tape.value(b) if b is not None else None
    rv = tape.value(resid) if resid is not None else None
    x2 = xv.reshape(-1, xv.shape[-1])
    epi = {None: K.EPI_NONE, "gelu_tanh": K.EPI_GELU_TANH, "gelu_erf": K.EPI_GELU_ERF, "relu": K.EPI_RELU}[act]
    depi = {None: K.EPI_NONE, "gelu_tanh": K.EPI_MUL_DGELU_TANH, "gelu_erf": K.EPI_MUL_DGELU_ERF,
            "relu": K.EPI_MUL_DRELU}[act]
    aux = torch.empty((x2.shape[0], wv.shape[0]), dtype=torch.bfloat16, device=xv.device) if act else None
    r2 = rv.reshape(-1, rv.shape[-1]) if rv is not None else None
    y = K.linear_fwd(x2, wv, bv, epi=epi, resid=r2, aux=aux)
    y = y.reshape(*xv.shape[:-1], wv.shape[0])
    inputs = [x, w] + ([b] if b is not None else []) + ([resid] if resid is not None else [])
    has_b, has_r = b is not None, resid is not None
    x_needs = tape.nodes[x].requires_grad

    def vjp(gy, targets):
        g2 = gy.reshape(-1, gy.shape[-1])
        if act:
            # dU = dY * act'(U): elementwise on the saved pre-activation
            g2 = K.gelu_bwd(aux, g2, tanh_form=(act == "gelu_tanh")) if act != "relu" else \
                (g2 * (aux > 0)).to(torch.bfloat16)
        out = []
        with SideWork(tape, g2.device) as side:
            db = _bgrad_into(targets, 2, g2, side) if has_b else None      # column sums next to the GEMMs
            dw = _wgrad_into(targets, 1, g2, x2, side)
            dx = K.linear_dgrad(g2, wv).reshape(xv.shape) if x_needs else None
        out.append(dx)
        out.append(dw)
        if has_b:
            out.append(db)
        if has_r:
            out.append(gy)
        return out

    rule = RULE_LINEAR + (f" [+bias{'+' + act if act else ''}{'+residual' if has_r else ''}]")
    return tape.record("linear", inputs, y, vjp, rule)


def mlp_up_down(tape: TensorTape, x: int, w1: int, b1: int, w2: int, b2: int, resid: int, *,
                act: str = "gelu_tanh") -> int:
    """``resid + (act(x w1^T + b1)) w2^T + b2`` as one node.

    Backward fuses ``act'`` into the dgrad epilogue of the second GEMM:
    ``dU = (dY @ w2) * act'(U)`` is one kernel (no separate elementwise pass).
    """
    xv, w1v, b1v, w2v, b2v, rv = (tape.value(i) for i in (x, w1, b1, w2, b2, resid))
    x2 = xv.reshape(-1, xv.shape[-1])
    r2 = rv.reshape(-1, rv.shape[-1])
    epi = {"gelu_tanh": K.EPI_GELU_TANH, "gelu_erf": K.EPI_GELU_ERF, "relu": K.EPI_RELU}[act]
    depi = {"gelu_tanh": K.EPI_MUL_DGELU_TANH, "gelu_erf": K.EPI_MUL_DGELU_ERF, "relu": K.EPI_MUL_DRELU}[act]
    u = torch.empty((x2.shape[0], w1v.shape[0]), dtype=torch.bfloat16, device=xv.device)
    h = K.linear_fwd(x2, w1v, b1v, epi=epi, aux=u)
    y = K.linear_fwd(h, w2v, b2v, resid=r2).reshape(rv.shape)

    def vjp(gy, targets):
        g2 = gy.reshape(-1, gy.shape[-1])
        with SideWork(tape, g2.device) as side:
            db2 = _bgrad_into(targets, 4, g2, side)
            dw2 = _wgrad_into(targets, 3, g2, h, side)
            du = K.linear_dgrad(g2, w2v, epi=depi, resid=u)      # (dY @ w2) * act'(U)
            # du is produced on the main stream: the side stream must see it before it sums its columns
            if side.on:
                ev = torch.cuda.Event()
                ev.record(side.main)
                side.side.wait_event(ev)
            db1 = _bgrad_into(targets, 2, du, side)
            dw1 = _wgrad_into(targets, 1, du, x2, side)
            dx = K.linear_dgrad(du, w1v).reshape(xv.shape)
        return [dx, dw1, db1, dw2, db2, gy]

    return tape.record("mlp", [x, w1, b1, w2, b2, resid], y, vjp,
                       RULE_LINEAR + f" [mlp: up+bias+{act}, down+bias+residual]")


def layernorm(tape: TensorTape, x: int, gamma: int, beta: int, eps: float = 1e-5) -> int:
    """LayerNorm over the last dim (ft-nn/src/lib.rs:2042; kernel math lib.rs:5824/6052)."""
    xv, gv, bv = tape.value(x), tape.value(gamma), tape.value(beta)
    x2 = xv.reshape(-1, xv.shape[-1])
    y, mean, rstd, _ = K.layernorm_fwd(x2, gv, bv, eps)

    def vjp(gy, targets):
        g2 = gy.reshape(-1, gy.shape[-1])
        # fuse the running gradient of x (the residual branch) into the dx kernel
        cur = targets.take_current(0)
        tg, tb = targets.leaf_target(1), targets.leaf_target(2)
        if tg is not None and tb is not None and tg[1] == tb[1]:
            dx, _, _ = K.layernorm_bwd(g2, x2, gv, mean, rstd, dx_add=None if cur is None else cur.reshape(x2.shape),
                                       dgamma=tg[0], dbeta=tb[0], accumulate=tg[1])
            targets.mark_accumulated(1)
            targets.mark_accumulated(2)
            return [dx.reshape(xv.shape), ACCUMULATED, ACCUMULATED]
        dx, dg, db = K.layernorm_bwd(g2, x2, gv, mean, rstd, dx_add=None if cur is None else cur.reshape(x2.shape))
        return [dx.reshape(xv.shape), dg, db]

    return tape.record("layer_norm", [x, gamma, beta], y.reshape(xv.shape), vjp, "d(layer_norm(x))/dx,dgamma,dbeta")


def rmsnorm(tape: TensorTape, x: int, gamma: int, eps: float = 1e-6) -> int:
    """RMSNorm (ft-nn/src/lib.rs:6843; kernel math ft-kernel-cpu/src/lib.rs:6418/6503)."""
    xv, gv = tape.value(x), tape.value(gamma)
    x2 = xv.reshape(-1, xv.shape[-1])
    y, rstd = K.rmsnorm_fwd(x2, gv, eps)

    def vjp(gy, targets):
        g2 = gy.reshape(-1, gy.shape[-1])
        tg = targets.leaf_target(1)
        if tg is not None:
            dx, _ = K.rmsnorm_bwd(g2, x2, gv, rstd, dgamma=tg[0], accumulate=tg[1])
            targets.mark_accumulated(1)
            return [dx.reshape(xv.shape), ACCUMULATED]
        dx, dg = K.rmsnorm_bwd(g2, x2, gv, rstd)
        return [dx.reshape(xv.shape), dg]

    return tape.record("rms_norm", [x, gamma], y.reshape(xv.shape), vjp, "d(rms_norm(x))/dx,dgamma")


def attention_packed(tape: TensorTape, qkv: int, n_heads: int, *, causal: bool = True,
                     scale: Optional[float] = None) -> int:
    """Multi-head attention over packed ``[B, S, 3*d]`` projections -> ``[B, S, d]``.

    Heads are addressed in place through strided TMA maps: no split/permute copies
    (the reference reshapes to [N*H, S, hd], ft-nn/src/lib.rs:5145-5167).
    """
    qv = tape.value(qkv)
    B, S, d3 = qv.shape
    d = d3 // 3
    hd = d // n_heads
    q, k, v = (qv[:, :, i * d:(i + 1) * d].view(B, S, n_heads, hd) for i in range(3))
    o, lse = K.attention_fwd(q, k, v, causal=causal, scale=scale)

    def vjp(go, targets):
        dqkv = torch.empty_like(qv)
        dq, dk, dv = (dqkv[:, :, i * d:(i + 1) * d].view(B, S, n_heads, hd) for i in range(3))
        K.attention_bwd(q, k, v, o, lse, go.reshape(B, S, n_heads, hd), causal=causal, scale=scale,
                        dq=dq, dk=dk, dv=dv)
        return [dqkv]

    return tape.record("sdpa", [qkv], o.view(B, S, d), vjp, "d(sdpa(q,k,v))/dq,dk,dv [flash, recompute P]")


def embedding(tape: TensorTape, ids: torch.Tensor, wte: int, wpe: Optional[int], S: int) -> int:
    """Token (+ position) embedding; backward is a deterministic sorted scatter-add."""
    wv = tape.value(wte)
    pv = tape.value(wpe) if wpe is not None else None
    B = ids.numel() // S
    out = K.embedding_fwd(ids, wv, pv, S).view(B, S, wv.shape[1])
    inputs = [wte] + ([wpe] if wpe is not None else [])

    def vjp(go, targets):
        g2 = go.reshape(-1, go.shape[-1])
        res = []
        t0 = targets.leaf_target(0)
        t1 = targets.leaf_target(1) if wpe is not None else None
        if t0 is not None and (wpe is None or t1 is not None):
            for t in (t0, t1):
                if t is not None and not t[1]:
                    K.fill_f32(t[0], 0.0)
            K.embedding_bwd(ids, g2, t0[0], t1[0] if t1 is not None else None, S)
            targets.mark_accumulated(0)
            res.append(ACCUMULATED)
            if wpe is not None:
                targets.mark_accumulated(1)
                res.append(ACCUMULATED)
            return res
        dwte = torch.zeros(wv.shape, dtype=torch.float32, device=wv.device)
        dwpe = torch.zeros(pv.shape, dtype=torch.float32, device=wv.device) if pv is not None else None
        K.embedding_bwd(ids, g2, dwte, dwpe, S)
        return [dwte] + ([dwpe] if wpe is not None else [])

    return tape.record("embedding", inputs, out, vjp, "d(index_select(x))/dx=scatter_add_grad")


def lm_head_cross_entropy(tape: TensorTape, x: int, w: int, targets_ids: torch.Tensor, vocab: int) -> int:
    """``mean(cross_entropy(x @ w^T, targets))`` with the softmax gradient formed in place.

    The logits ``[rows, padded_vocab]`` are produced by the GEMM, the loss kernel overwrites
    them with ``(softmax - onehot)/rows`` (ft-kernel-cpu/src/lib.rs:6649/6679), and backward
    only scales by the incoming scalar and runs the two GEMMs.
    """
    xv, wv = tape.value(x), tape.value(w)
    x2 = xv.reshape(-1, xv.shape[-1])
    rows = x2.shape[0]
    logits = K.linear_fwd(x2, wv)
    losses, dlogits = K.cross_entropy_fwd_bwd(logits, targets_ids.reshape(-1), vocab, 1.0 / rows, inplace=True)
    loss = K.reduce_mean(losses)

    def vjp(g, targets):
        # g is the scalar seed (ones for a plain backward); dlogits already carries 1/rows
        dl = dlogits
        if not (g.numel() == 1 and g.dtype == torch.float32 and getattr(g, "_ft_unit_seed", False)):
            dl = (dlogits.float() * g.reshape(()).float()).to(torch.bfloat16)
        with SideWork(tape, dl.device) as side:
            dw = _wgrad_into(targets, 1, dl, x2, side)
            dx = K.linear_dgrad(dl, wv).reshape(xv.shape)
        return [dx, dw]

    return tape.record("lm_head_ce", [x, w], loss.reshape(()), vjp,
                       RULE_LINEAR + " [+softmax-cross-entropy, mean]")


# ----------------------------------------------------------------------------------------------
# Single operators of the session surface (one kernel forward, one or two backward).  The composite
# rules above are what the GPT models use; these give every hot session operator an sm_100a route.
def matmul(tape: TensorTape, a: int, b: int) -> int:
    """``a[M,K] @ b[K,N]`` (ft-autograd MatMul arm, ft-autograd/src/lib.rs:11953)."""
    av, bv = tape.value(a), tape.value(b)
    y = K.gemm(av, bv, b_mn=True)
    a_needs, b_needs = tape.nodes[a].requires_grad, tape.nodes[b].requires_grad

    def vjp(g, targets):
        g = g.contiguous()          # an expanded gradient (from a sum) has zero strides
        da = K.gemm(g, bv) if a_needs else None                         # dOut @ B^T
        db = K.gemm(av, g, a_mn=True, b_mn=True) if b_needs else None   # A^T @ dOut
        return [da, db]

    return tape.record("matmul", [a, b], y, vjp, RULE_LINEAR)


def bmm(tape: TensorTape, a: int, b: int) -> int:
    """Batched ``a[L,M,K] @ b[L,K,N]`` on the strided-batched GEMM."""
    av, bv = tape.value(a), tape.value(b)
    L, M, Kd = av.shape
    N = bv.shape[2]

    def run(x, y, m, n, k, x_mn, y_mn):
        out = torch.empty((L, m, n), dtype=torch.bfloat16, device=x.device)
        K.gemm_batched(x, y, out, M=m, N=n, K=k, L0=L, L1=1, a_strides=(x.stride(1), x.stride(0), 0),
                       b_strides=(y.stride(1), y.stride(0), 0), d_strides=(n, m * n, 0), a_mn=x_mn, b_mn=y_mn)
        return out
    y = run(av, bv, M, N, Kd, False, True)

    def vjp(g, targets):
        g = g.contiguous()
        da = run(g, bv, M, Kd, N, False, False)      # dOut @ B^T  (B given as [K, N] = [n_out, k] row-major)
        db = run(av, g, Kd, N, M, True, True)        # A^T @ dOut
        return [da, db]

    return tape.record("bmm", [a, b], y, vjp, "d(bmm(A,B))/dA=dOut@B^T; d(bmm(A,B))/dB=A^T@dOut (batched)")


def gelu(tape: TensorTape, x: int, *, tanh_form: bool = False) -> int:
    xv = tape.value(x)
    y = K.gelu_fwd(xv, tanh_form=tanh_form)

    def vjp(g, targets):
        return [K.gelu_bwd(xv, g.contiguous(), tanh_form=tanh_form)]

    return tape.record("gelu_tanh" if tanh_form else "gelu", [x], y, vjp, "d(gelu(x))/dx")


def softmax_lastdim(tape: TensorTape, x: int) -> int:
    """Row softmax over the last dimension (ft-kernel-cpu/src/lib.rs:18350; guards of fused.rs:321)."""
    xv = tape.value(x)
    y = K.softmax_rows(xv.reshape(-1, xv.shape[-1])).reshape(xv.shape)

    def vjp(g, targets):
        return [K.softmax_bwd(y, g.contiguous()).reshape(xv.shape)]

    return tape.record("softmax", [x], y, vjp, "d(softmax(x))/dx_i=s_i*(grad_i-sum(grad*s))")


def add_same_shape(tape: TensorTape, a: int, b: int) -> int:
    y = K.add(tape.value(a), tape.value(b))
    return tape.record("add", [a, b], y, lambda g, targets: [g, g], "d(a+b)/da=1; d(a+b)/db=1")


def embedding_lookup(tape: TensorTape, w: int, ids: torch.Tensor) -> int:
    """``w[ids]`` for an id tensor of any shape; backward is the deterministic sorted scatter-add."""
    wv = tape.value(w)
    flat = ids.reshape(-1).to(torch.int64)
    out = K.embedding_fwd(flat, wv, None, flat.numel()).view(*ids.shape, wv.shape[1])

    def vjp(go, targets):
        dw = torch.zeros(wv.shape, dtype=torch.float32, device=wv.device)
        K.embedding_bwd(flat, go.reshape(-1, go.shape[-1]).contiguous(), dw, None, flat.numel())
        return [dw]

    return tape.record("embedding", [w], out, vjp, "d(index_select(x))/dx=scatter_add_grad")


def sdpa(tape: TensorTape, q: int, k: int, v: int, *, causal: bool, scale: Optional[float] = None) -> int:
    """Flash attention on ``[..., S, hd]`` operands (``[N*H, S, hd]`` or ``[N, H, S, hd]``,
    ft-nn/src/lib.rs:5145-5184); the kernels read them as ``[B, S, H, hd]`` views, no copies."""
    qv, kv, vv = tape.value(q), tape.value(k), tape.value(v)

    def as_bshd(t):
        if t.dim() == 3:
            return t.unsqueeze(2)                 # [L, S, 1, hd]
        return t.transpose(1, 2)                  # [N, H, S, hd] -> [N, S, H, hd] view
    q4, k4, v4 = as_bshd(qv), as_bshd(kv), as_bshd(vv)
    o_store = torch.empty_like(qv)
    o, lse = K.attention_fwd(q4, k4, v4, causal=causal, scale=scale, out=as_bshd(o_store))

    def vjp(go, targets):
        go_c = go.contiguous()
        dq, dk, dv = torch.empty_like(qv), torch.empty_like(kv), torch.empty_like(vv)
        K.attention_bwd(q4, k4, v4, o, lse, as_bshd(go_c), causal=causal, scale=scale,
                        dq=as_bshd(dq), dk=as_bshd(dk), dv=as_bshd(dv))
        return [dq, dk, dv]

    return tape.record("sdpa", [q, k, v], o_store, vjp, "d(sdpa(q,k,v))/dq,dk,dv [flash, recompute P]")


def cross_entropy_mean(tape: TensorTape, logits: int, targets_ids: torch.Tensor) -> int:
    """``mean(cross_entropy(logits, targets))``; the logits node keeps its value (the gradient is
    written to a second buffer), ft-kernel-cpu/src/lib.rs:6649/6679."""
    lv = tape.value(logits)
    rows, vocab = lv.shape
    losses, dlogits = K.cross_entropy_fwd_bwd(lv, targets_ids.reshape(-1).to(torch.int64), vocab, 1.0 / rows,
                                              inplace=False)
    loss = K.reduce_mean(losses)

    def vjp(g, targets):
        if g.numel() == 1 and getattr(g, "_ft_unit_seed", False):
            return [dlogits]
        return [(dlogits.float() * g.reshape(()).float()).to(torch.bfloat16)]

    return tape.record("cross_entropy", [logits], loss.reshape(()), vjp,
                       "d(cross_entropy)/dlogits=g*(softmax-onehot)")


def dropout(tape: TensorTape, x: int, p: float, seed: int, offset: int = 0) -> int:
    """Philox dropout: the mask is a function of (seed, offset, element index), so backward
    regenerates it by running the same kernel on the incoming gradient (ft-nn/src/lib.rs:2357-2373)."""
    xv = tape.value(x)
    y = K.dropout(xv, p, seed, offset)

    def vjp(g, targets):
        return [K.dropout(g.contiguous(), p, seed, offset)]

    return tape.record("dropout", [x], y, vjp, "d(dropout(x))/dx=mask/(1-p)")
