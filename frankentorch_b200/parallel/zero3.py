"""ZeRO-3 style parameter sharding with the collectives fused into the GEMMs that need them.

Every 2-D weight ``[out, in]`` of a block is split by output rows over the ranks; a rank keeps
only its ``[out / world, in]`` shard (bf16 compute copy in peer-visible memory, fp32 master,
moments and gradient shard locally).

* forward  ``y = x W^T``  : all-gather of the weight shards fused into the GEMM
  (``FusedCollectives.allgather_b_gemm``); tiles of the own shard start at once, the rest as
  their rows arrive;
* backward ``dx = dy W``  : the same gather again, the weight now being sharded along the
  reduction dimension;
* backward ``dW = dy^T x``: a GEMM whose epilogue reduce-scatters the result by rows, so each
  rank ends up with the job-mean gradient of its shard only
  (``FusedCollectives.gemm_reduce_scatter`` with ``alpha = 1 / world``), accumulated in fp32.

Ordering between ranks: the optimizer updates a shard after the data-parallel step of the
replicated parameters, whose start barrier guarantees that every rank has finished its backward
(no rank still reads the old shard); forward gathers use the ready handshake, which a rank
posts from its own gather kernel, i.e. after its optimizer step in stream order.

The reference has no sharded training (FEATURE_PARITY.md:176); Linear math is
ft-nn/src/lib.rs:1076-1100, optimizer state layout ft-optim/src/lib.rs:800-814.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..autograd.tape import ACCUMULATED, TensorTape
from ..ops import kernels as K
from ..ops.fused import RULE_LINEAR, _bgrad_into
from .fused_gemm import FusedCollectives, SymmTensor


class Zero3Context:
    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, *, max_weight_elems: int,
                 comm_ctas: int = 0):
        self.group, self.device = group, device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        self.fc = FusedCollectives(group, device, max_gather_bytes=max(2 * max_weight_elems, 1 << 20),
                                   max_inbox_elems=max_weight_elems, comm_ctas=comm_ctas)
        self.shards: Dict[int, SymmTensor] = {}          # tape leaf id -> peer-visible weight shard
        self._scratch: Dict[Tuple[int, int], torch.Tensor] = {}

    def register(self, leaf: int, shard: SymmTensor) -> None:
        self.shards[leaf] = shard

    def scratch(self, rows: int, cols: int) -> torch.Tensor:
        """Full-size staging buffer for a gathered weight; one per shape, reused by every layer."""
        t = self._scratch.get((rows, cols))
        if t is None:
            t = torch.empty((rows, cols), dtype=torch.bfloat16, device=self.device)
            self._scratch[(rows, cols)] = t
        return t

    def begin_step(self) -> None:
        self.fc.begin_step()


def zero3_linear(tape: TensorTape, x: int, w: int, b: Optional[int], z: Zero3Context, *,
                 act: Optional[str] = None, resid: Optional[int] = None) -> int:
    """``y = act(x @ allgather(w)^T + b) (+ resid)`` with ``w`` this rank's ``[out / world, in]`` shard."""
    xv = tape.value(x)
    bv = tape.value(b) if b is not None else None
    rv = tape.value(resid) if resid is not None else None
    shard = z.shards[w]
    rows_s, cols = shard.t.shape
    out_f = rows_s * z.world
    x2 = xv.reshape(-1, cols)
    epi = {None: K.EPI_NONE, "gelu_tanh": K.EPI_GELU_TANH, "gelu_erf": K.EPI_GELU_ERF, "relu": K.EPI_RELU}[act]
    aux = torch.empty((x2.shape[0], out_f), dtype=torch.bfloat16, device=xv.device) if act else None
    r2 = rv.reshape(-1, out_f) if rv is not None else None
    w_full = z.scratch(out_f, cols)
    y = z.fc.allgather_b_gemm(x2, shard, w_full, bias=bv, epi=epi, resid=r2, aux=aux, handshake=True)
    y = y.reshape(*xv.shape[:-1], out_f)
    inputs = [x, w] + ([b] if b is not None else []) + ([resid] if resid is not None else [])
    has_b, has_r = b is not None, resid is not None
    x_needs = tape.nodes[x].requires_grad

    def vjp(gy, targets):
        g2 = gy.reshape(-1, out_f)
        if act:
            g2 = K.gelu_bwd(aux, g2, tanh_form=(act == "gelu_tanh")) if act != "relu" else \
                (g2 * (aux > 0)).to(torch.bfloat16)
        # dW shard = rows[rank] of mean over ranks of dy^T x, straight into the fp32 gradient shard
        tgt = targets.leaf_target(1)
        if tgt is None:
            raise K.KernelError("a sharded weight needs a bound gradient buffer")
        buf, filled = tgt
        z.fc.gemm_reduce_scatter(g2, x2, buf, a_mn=True, b_mn=True, accumulate=filled, alpha=1.0 / z.world)
        targets.mark_accumulated(1)
        out = [None, ACCUMULATED]
        if has_b:
            out.append(_bgrad_into(targets, 2, g2))
        if x_needs:
            out[0] = z.fc.allgather_b_gemm(g2, shard, w_full, dgrad=True).reshape(xv.shape)
        if has_r:
            out.append(gy)
        return out

    rule = RULE_LINEAR + f" [allgather(W)->gemm{'+bias' if has_b else ''}{'+' + act if act else ''}" \
                         f"{'+residual' if has_r else ''}; dW: gemm->reduce-scatter]"
    return tape.record("zero3_linear", inputs, y, vjp, rule)
