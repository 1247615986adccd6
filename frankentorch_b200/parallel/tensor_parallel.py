"""Tensor parallelism with sequence parallelism around it (Megatron-style blocks), built on the
collective-fused GEMMs of :mod:`frankentorch_b200.parallel.fused_gemm`.

Between blocks every rank holds a contiguous slice of the token rows (``[M / world, d]``:
whole sequences of the global batch), so LayerNorm, residual adds, embedding and the LM head
work on local rows only.  Inside a block

* the column-parallel Linear (QKV, fc1) consumes ``all-gather(rows)`` - one kernel,
  all-gather -> GEMM, with bias / GELU in the epilogue;
* the row-parallel Linear (attention output, fc2) produces partial sums that are
  reduce-scattered back to row slices - one kernel, GEMM -> reduce-scatter, with bias and the
  residual added by the owner after the ordered sum.

Backward mirrors it: the gradient of a row-parallel Linear's input is
``all-gather(dY) @ W`` (gather fused again; the GELU derivative rides in that epilogue), the
gradient of a column-parallel Linear's input is ``reduce-scatter(dU @ W)``.

The reference has neither tensor nor sequence parallelism (no column / row-parallel Linear in
ft-nn); the Linear math is ft-nn/src/lib.rs:1076-1100, ft-kernel-cpu/src/lib.rs:17162-17302.

Gradient scaling: each rank's loss is the mean over its own rows and the job's loss is the mean
of those.  Replicated parameters (LayerNorm, embeddings, the biases added after a
reduce-scatter) receive per-rank partial gradients that are *averaged* across ranks; sharded
weights see the gathered upstream gradients of all ranks, i.e. ``world`` times the gradient of
the job loss, and are scaled by ``1 / world`` in their optimizer step.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..autograd.tape import ACCUMULATED, TensorTape
from ..ops import kernels as K
from ..ops.fused import RULE_LINEAR, _bgrad_into, _wgrad_into
from .fused_gemm import FusedCollectives, SymmTensor


class TPContext:
    """Fused-collective state of one tensor-parallel group plus two alternating row-slice buffers."""

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, *, rows_per_rank: int,
                 d_model: int, comm_ctas: int = 0):
        self.group, self.device = group, device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        self.ms, self.d = rows_per_rank, d_model
        self.m = rows_per_rank * self.world
        self.fc = FusedCollectives(group, device, max_gather_bytes=max(self.m * d_model * 2, 1 << 20),
                                   max_inbox_elems=self.m * d_model, comm_ctas=comm_ctas)
        self._shards = [SymmTensor.alloc((rows_per_rank, d_model), torch.bfloat16, group, device) for _ in range(2)]
        self._which = 0

    def begin_step(self) -> None:
        self.fc.begin_step()
        self._which = 0

    def stage(self, rows: torch.Tensor) -> SymmTensor:
        """Copy a ``[M / world, d]`` slice into the next peer-visible buffer (they alternate: a rank
        is never more than one collective ahead of its slowest peer)."""
        s = self._shards[self._which]
        self._which ^= 1
        s.t.copy_(rows.reshape(self.ms, self.d))
        return s


def tp_attention(tape: TensorTape, x: int, wqkv: int, bqkv: int, wproj: int, bproj: int, resid: int,
                 ctx: TPContext, *, heads_local: int, seq_len: int, causal: bool = True) -> int:
    """``resid + reduce_scatter(attn(all_gather(x) Wqkv^T + b) Wproj^T) + bproj`` on row slices.

    ``wqkv`` is this rank's ``[3 * d / world, d]`` block (its heads' q rows, then k, then v),
    ``wproj`` its ``[d, d / world]`` column block.
    """
    xv, wq, bq, wp, bp, rv = (tape.value(i) for i in (x, wqkv, bqkv, wproj, bproj, resid))
    ms, d, m = ctx.ms, ctx.d, ctx.m
    dl = wp.shape[1]
    hd = dl // heads_local
    x_full = torch.empty((m, d), dtype=torch.bfloat16, device=xv.device)
    qkv = ctx.fc.allgather_a_gemm(ctx.stage(xv), wq, x_full, bias=bq)
    B = m // seq_len
    q, k, v = (qkv[:, i * dl:(i + 1) * dl].view(B, seq_len, heads_local, hd) for i in range(3))
    o, lse = K.attention_fwd(q, k, v, causal=causal)
    a2 = o.view(m, dl)
    y = torch.empty((ms, d), dtype=torch.bfloat16, device=xv.device)
    ctx.fc.gemm_reduce_scatter(a2, wp, y, bias=bp, resid=rv.reshape(ms, d))

    def vjp(gy, targets):
        g2 = gy.reshape(ms, d)
        g_full = torch.empty((m, d), dtype=torch.bfloat16, device=g2.device)
        da = ctx.fc.allgather_a_gemm(ctx.stage(g2), wp, g_full, b_mn=True)        # [m, dl] = dY @ Wproj
        dwp = _wgrad_into(targets, 3, g_full, a2)
        dbp = _bgrad_into(targets, 4, g2)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = (dqkv[:, i * dl:(i + 1) * dl].view(B, seq_len, heads_local, hd) for i in range(3))
        K.attention_bwd(q, k, v, o, lse, da.view(B, seq_len, heads_local, hd), causal=causal, dq=dq, dk=dk, dv=dv)
        dwq = _wgrad_into(targets, 1, dqkv, x_full)
        dbq = _bgrad_into(targets, 2, dqkv)
        dx = torch.empty((ms, d), dtype=torch.bfloat16, device=g2.device)
        ctx.fc.gemm_reduce_scatter(dqkv, wq, dx, b_mn=True)                      # rows of dQKV @ Wqkv
        return [dx.reshape(xv.shape), dwq, dbq, dwp, dbp, gy]

    return tape.record("tp_attention", [x, wqkv, bqkv, wproj, bproj, resid], y.reshape(rv.shape), vjp,
                       RULE_LINEAR + " [allgather->qkv, flash sdpa, proj->reduce-scatter+bias+residual]")


def tp_mlp(tape: TensorTape, x: int, w1: int, b1: int, w2: int, b2: int, resid: int, ctx: TPContext, *,
           act: str = "gelu_tanh") -> int:
    """``resid + reduce_scatter(act(all_gather(x) W1^T + b1) W2^T) + b2`` on row slices.

    ``w1`` is this rank's ``[ff / world, d]`` row block, ``w2`` its ``[d, ff / world]`` column block.
    """
    xv, w1v, b1v, w2v, b2v, rv = (tape.value(i) for i in (x, w1, b1, w2, b2, resid))
    ms, d, m = ctx.ms, ctx.d, ctx.m
    ffl = w1v.shape[0]
    epi = {"gelu_tanh": K.EPI_GELU_TANH, "gelu_erf": K.EPI_GELU_ERF, "relu": K.EPI_RELU}[act]
    depi = {"gelu_tanh": K.EPI_MUL_DGELU_TANH, "gelu_erf": K.EPI_MUL_DGELU_ERF, "relu": K.EPI_MUL_DRELU}[act]
    x_full = torch.empty((m, d), dtype=torch.bfloat16, device=xv.device)
    u = torch.empty((m, ffl), dtype=torch.bfloat16, device=xv.device)
    h = ctx.fc.allgather_a_gemm(ctx.stage(xv), w1v, x_full, bias=b1v, epi=epi, aux=u)
    y = torch.empty((ms, d), dtype=torch.bfloat16, device=xv.device)
    ctx.fc.gemm_reduce_scatter(h, w2v, y, bias=b2v, resid=rv.reshape(ms, d))

    def vjp(gy, targets):
        g2 = gy.reshape(ms, d)
        g_full = torch.empty((m, d), dtype=torch.bfloat16, device=g2.device)
        # dU = (all_gather(dY) @ W2) * act'(U): gather, GEMM and activation derivative in one kernel
        du = ctx.fc.allgather_a_gemm(ctx.stage(g2), w2v, g_full, b_mn=True, epi=depi, resid=u)
        dw2 = _wgrad_into(targets, 3, g_full, h)
        db2 = _bgrad_into(targets, 4, g2)
        dw1 = _wgrad_into(targets, 1, du, x_full)
        db1 = _bgrad_into(targets, 2, du)
        dx = torch.empty((ms, d), dtype=torch.bfloat16, device=g2.device)
        ctx.fc.gemm_reduce_scatter(du, w1v, dx, b_mn=True)
        return [dx.reshape(xv.shape), dw1, db1, dw2, db2, gy]

    return tape.record("tp_mlp", [x, w1, b1, w2, b2, resid], y.reshape(rv.shape), vjp,
                       RULE_LINEAR + f" [allgather->fc1+bias+{act}, fc2->reduce-scatter+bias+residual]")
