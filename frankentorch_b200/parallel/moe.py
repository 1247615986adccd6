"""Expert-parallel mixture-of-experts feed-forward layer (top-2 softmax router).

The reference has no MoE module (a grep for ``moe`` / ``expert`` / ``router`` finds none); the
layer is assembled from primitives it does have - top-k (ft-kernel-cpu/src/lib.rs:22808), row
softmax (:18350), Linear (ft-nn/src/lib.rs:1076) and scatter/gather - with these choices:

* router: ``softmax(x Wr^T)`` over ``E`` experts, top-2 (ties to the lower index), gates
  renormalised over the chosen pair;
* capacity: every rank may send at most ``ceil(capacity_factor * tokens * 2 / E)`` rows to each
  expert; slots are assigned in (token, k) order, later entries are dropped (deterministic);
* expert ``e`` lives on rank ``e // (E / world)``; the dispatch and combine all-to-alls are the
  permuting peer-memory kernels of ``csrc/moe_sm100.cu`` (rows go straight from the token
  buffer into the expert's receive buffer and back), the expert MLPs are the tcgen05 GEMMs with
  bias+GELU / bias epilogues;
* combine adds ``k = 0`` then ``k = 1`` (then the residual) - a fixed order.

Backward mirrors forward: the scaled output gradient is dispatched with the same slots, the
expert MLP backward runs on the receive buffers (unused rows are exact zeros, so weight and bias
gradients need no masking), its input gradient is combined back, and the gate gradient is the
dot of the output gradient with the rows kept from the forward combine.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional

import torch
import torch.distributed as dist

from ..autograd.tape import ACCUMULATED, TensorTape
from ..ops import _lib
from ..ops import kernels as K
from ..ops._lib import FtkMoeDesc
from .fused_gemm import SymmTensor
from .symm import SymmetricBuffer

ROUTER_ROWS = 128      # router weight is stored [128, d]; rows >= E are zero (one GEMM tile)


class MoEBuffers:
    """Receive / output buffers of one MoE layer, peer-visible: ``[E_local, world, C, d]`` each."""

    def __init__(self, ep: "ExpertParallel"):
        shape = (ep.e_local, ep.world, ep.capacity, ep.d)
        n = ep.e_local * ep.world * ep.capacity * ep.d * 2
        cnt_bytes = 256 * ((ep.e_local * ep.world * 4 + 255) // 256)
        self.buf = SymmetricBuffer(4 * n + cnt_bytes, ep.group, ep.device)
        self.recv_x = SymmTensor(self.buf, shape, torch.bfloat16, 0)
        self.y = SymmTensor(self.buf, shape, torch.bfloat16, n)
        self.recv_dy = SymmTensor(self.buf, shape, torch.bfloat16, 2 * n)
        self.dxe = SymmTensor(self.buf, shape, torch.bfloat16, 3 * n)
        self.counts = SymmTensor(self.buf, (ep.e_local * ep.world,), torch.int32, 4 * n)
        self._ep = ep
        self._act = {}

    def activations(self, ff: int):
        """Pre-activation, activation and their gradient, ``[E_local, world * C, ff]`` each, allocated
        once and zero-filled: the ragged GEMMs never write the rows of skipped tiles, and what they
        leave there must stay finite (the weight gradients multiply those rows by exact zeros)."""
        if ff not in self._act:
            ep = self._ep
            shape = (ep.e_local, ep.world * ep.capacity, ff)
            self._act[ff] = tuple(torch.zeros(shape, dtype=torch.bfloat16, device=ep.device) for _ in range(3))
        return self._act[ff]


class ExpertParallel:
    """Protocol state shared by every MoE layer of a model: epoch word and flag arrays."""

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, *, tokens: int, d_model: int,
                 n_experts: int = 8, capacity_factor: float = 1.25):
        self.group, self.device = group, device
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not divide over {self.world} ranks")
        self.E, self.e_local = n_experts, n_experts // self.world
        self.T, self.d = tokens, d_model
        cap = math.ceil(capacity_factor * tokens * 2 / n_experts)
        self.capacity = (cap + 7) // 8 * 8
        self.lib = _lib.load()
        self.local = torch.zeros(64, dtype=torch.int32, device=device)     # [0] epoch, [1] ticket
        self.flags = SymmetricBuffer(256, group, device)                    # arrive[0:8], ready[16:24]
        self.flags.bytes.zero_()
        torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=group)

    def new_layer_buffers(self) -> MoEBuffers:
        return MoEBuffers(self)

    # ------------------------------------------------------------------ kernel wrappers
    def _desc(self, idx, slot, counts) -> FtkMoeDesc:
        m = FtkMoeDesc()
        m.T, m.d, m.E, m.capacity, m.rank, m.world = self.T, self.d, self.E, self.capacity, self.rank, self.world
        m.idx, m.slot, m.counts = idx.data_ptr(), slot.data_ptr(), counts.data_ptr()
        m.ticket = self.local[1:2].data_ptr()
        m.epoch = self.local[0:1].data_ptr()
        return m

    def _tick(self) -> None:
        K._chk(self.lib.ftk_tick_i32(self.local.data_ptr(), K._stream()), "ftk_tick_i32")

    def _ptrs(self, addrs: List[int]):
        arr = (C.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = addrs[r]
        return arr

    def route(self, logits: torch.Tensor):
        """``logits`` fp32 ``[T, ld]`` -> probs ``[T, E]``, idx ``[T, 2]``, gate ``[T, 2]``, slot, counts."""
        T, dev = self.T, self.device
        probs = torch.empty((T, self.E), dtype=torch.float32, device=dev)
        idx = torch.empty((T, 2), dtype=torch.int32, device=dev)
        gate = torch.empty((T, 2), dtype=torch.float32, device=dev)
        slot = torch.empty((T, 2), dtype=torch.int32, device=dev)
        counts = torch.empty((self.E,), dtype=torch.int32, device=dev)
        s = K._stream()
        K._chk(self.lib.ftk_moe_route(logits.data_ptr(), probs.data_ptr(), idx.data_ptr(), gate.data_ptr(),
                                      T, self.E, logits.stride(0), s), "ftk_moe_route")
        K._chk(self.lib.ftk_moe_slots(idx.data_ptr(), slot.data_ptr(), counts.data_ptr(), T, self.E,
                                      self.capacity, s), "ftk_moe_slots")
        return probs, idx, gate, slot, counts

    def dispatch(self, x2: torch.Tensor, idx, slot, counts, dst: SymmTensor, bufs: MoEBuffers,
                 scale: Optional[torch.Tensor] = None) -> None:
        m = self._desc(idx, slot, counts)
        self._tick()
        K._chk(self.lib.ftk_moe_dispatch(
            C.byref(m), x2.data_ptr(), None if scale is None else scale.data_ptr(),
            self._ptrs(dst.peer_ptrs), self._ptrs(bufs.counts.peer_ptrs), self._ptrs(self.flags.peer_ptrs),
            K._stream()), "ftk_moe_dispatch")

    def combine(self, src: SymmTensor, idx, slot, counts, gate: Optional[torch.Tensor], *,
                resid: Optional[torch.Tensor] = None, keep_rows: bool = False):
        m = self._desc(idx, slot, counts)
        out = torch.empty((self.T, self.d), dtype=torch.bfloat16, device=self.device)
        rows = torch.empty((self.T, 2, self.d), dtype=torch.bfloat16, device=self.device) if keep_rows else None
        self._tick()
        K._chk(self.lib.ftk_moe_combine(
            C.byref(m), self._ptrs(src.peer_ptrs), self._ptrs([p + 64 for p in self.flags.peer_ptrs]),
            None if gate is None else gate.data_ptr(), out.data_ptr(),
            None if resid is None else resid.data_ptr(), None if rows is None else rows.data_ptr(),
            K._stream()), "ftk_moe_combine")
        return out, rows


def moe_ffn(tape: TensorTape, x: int, wr: int, w1: int, b1: int, w2: int, b2: int, ep: ExpertParallel,
            bufs: MoEBuffers, *, resid: Optional[int] = None, act: str = "gelu_tanh") -> int:
    """``(resid +) sum_k gate_k * Expert_{e_k}(x)`` as one tape node.

    ``wr`` is the router weight ``[128, d]`` (rows >= E zero); ``w1 [E_local, ff, d]``,
    ``b1 [E_local, ff]``, ``w2 [E_local, d, ff]``, ``b2 [E_local, d]`` are this rank's experts.
    """
    xv, wrv, w1v, b1v, w2v, b2v = (tape.value(i) for i in (x, wr, w1, b1, w2, b2))
    rv = tape.value(resid) if resid is not None else None
    T, d, el_n = ep.T, ep.d, ep.e_local
    x2 = xv.reshape(T, d)
    epi = {"gelu_tanh": K.EPI_GELU_TANH, "gelu_erf": K.EPI_GELU_ERF, "relu": K.EPI_RELU}[act]
    depi = {"gelu_tanh": K.EPI_MUL_DGELU_TANH, "gelu_erf": K.EPI_MUL_DGELU_ERF, "relu": K.EPI_MUL_DRELU}[act]
    logits = K.gemm(x2, wrv, out_dtype=torch.float32, split_k=1)
    probs, idx, gate, slot, counts = ep.route(logits)
    ep.dispatch(x2, idx, slot, counts, bufs.recv_x, bufs)
    rows_e = ep.world * ep.capacity
    X = bufs.recv_x.t.view(el_n, rows_e, d)
    Y = bufs.y.t.view(el_n, rows_e, d)
    ff = w1v.shape[1]
    # Rows of an expert's batch: `world` segments of `capacity` slots, of which the first
    # recv_counts[e][src] hold tokens.  The GEMMs skip every 128-row tile that holds none (their outputs
    # are never read: combine only fetches slots below the count), so the capacity padding costs nothing.
    # The activation buffers live with the layer, start zeroed and only ever hold finite values in
    # skipped rows, which the weight gradients multiply by the zero rows of the dispatched gradient.
    u, h, du_all = bufs.activations(ff)
    seg = bufs.counts.t.view(el_n, ep.world)
    cap = ep.capacity
    for e in range(el_n):
        K.linear_fwd(X[e], w1v[e], b1v[e], epi=epi, aux=u[e], out=h[e], seg_counts=seg[e], seg_rows=cap)
        K.linear_fwd(h[e], w2v[e], b2v[e], out=Y[e], seg_counts=seg[e], seg_rows=cap)
    out, rows = ep.combine(bufs.y, idx, slot, counts, gate,
                           resid=None if rv is None else rv.reshape(T, d), keep_rows=True)

    def into(targets, i, e, fn):
        """Run ``fn(out=, accumulate=)`` on slice ``e`` of leaf ``i``'s gradient buffer."""
        tgt = targets.leaf_target(i)
        if tgt is None:
            return None
        buf, filled = tgt
        fn(out=buf[e], accumulate=filled)
        return ACCUMULATED

    def vjp(gy, targets):
        g2 = gy.reshape(T, d)
        d_gate = torch.empty((T, 2), dtype=torch.float32, device=g2.device)
        K._chk(ep.lib.ftk_moe_gate_grad(g2.data_ptr(), rows.data_ptr(), d_gate.data_ptr(), T, d, K._stream()),
               "ftk_moe_gate_grad")
        ep.dispatch(g2, idx, slot, counts, bufs.recv_dy, bufs, scale=gate)
        DY = bufs.recv_dy.t.view(el_n, rows_e, d)
        DX = bufs.dxe.t.view(el_n, rows_e, d)
        res = {1: None, 2: None, 3: None, 4: None}
        loose = {i: [] for i in (2, 3, 4, 5)}
        for e in range(el_n):
            r = into(targets, 4, e, lambda out, accumulate: K.linear_wgrad(DY[e], h[e], out=out, accumulate=accumulate))
            if r is None:
                loose[4].append(K.linear_wgrad(DY[e], h[e]))
            r = into(targets, 5, e, lambda out, accumulate: K.colsum(DY[e], out=out, accumulate=accumulate))
            if r is None:
                loose[5].append(K.colsum(DY[e]))
            du = du_all[e]
            K.linear_dgrad(DY[e], w2v[e], epi=depi, resid=u[e], out=du, seg_counts=seg[e], seg_rows=cap)
            r = into(targets, 2, e, lambda out, accumulate: K.linear_wgrad(du, X[e], out=out, accumulate=accumulate))
            if r is None:
                loose[2].append(K.linear_wgrad(du, X[e]))
            r = into(targets, 3, e, lambda out, accumulate: K.colsum(du, out=out, accumulate=accumulate))
            if r is None:
                loose[3].append(K.colsum(du))
            K.linear_dgrad(du, w1v[e], out=DX[e], seg_counts=seg[e], seg_rows=cap)
        grads = {}
        for i in (2, 3, 4, 5):
            if loose[i]:
                grads[i] = torch.stack(loose[i])
            else:
                targets.mark_accumulated(i)
                grads[i] = ACCUMULATED
        dx_tok, _ = ep.combine(bufs.dxe, idx, slot, counts, None)
        d_logits = torch.empty((T, ROUTER_ROWS), dtype=torch.bfloat16, device=g2.device)
        K._chk(ep.lib.ftk_moe_route_bwd(probs.data_ptr(), idx.data_ptr(), d_gate.data_ptr(), d_logits.data_ptr(),
                                        T, ep.E, ROUTER_ROWS, K._stream()), "ftk_moe_route_bwd")
        tgt = targets.leaf_target(1)
        if tgt is not None:
            K.linear_wgrad(d_logits, x2, out=tgt[0], accumulate=tgt[1])
            targets.mark_accumulated(1)
            dwr = ACCUMULATED
        else:
            dwr = K.linear_wgrad(d_logits, x2)
        dx = K.add(dx_tok, K.linear_dgrad(d_logits, wrv)).reshape(xv.shape)
        outg = [dx, dwr, grads[2], grads[3], grads[4], grads[5]]
        if resid is not None:
            outg.append(gy)
        return outg

    inputs = [x, wr, w1, b1, w2, b2] + ([resid] if resid is not None else [])
    shape = rv.shape if rv is not None else xv.shape
    return tape.record("moe_ffn", inputs, out.reshape(shape), vjp,
                       "d(moe)/dx: dispatch(g*gate) -> expert mlp bwd -> combine; d(gate)=<g,y_k>; router softmax/top2")


def moe_ffn_reference(x, wr, w1, b1, w2, b2, capacity: int, *, rank_tokens: Optional[List[torch.Tensor]] = None):
    """Plain PyTorch fp32 forward of the same layer for one rank's tokens (all experts given).

    ``w1 [E, ff, d]`` etc. hold every expert.  Capacity is per (source rank, expert), so a rank's
    result depends only on its own tokens.
    """
    xf = x.float()
    E = w1.shape[0]
    p = torch.softmax(xf @ wr.float()[:E].t(), dim=-1)
    top = torch.topk(p, 2, dim=-1)
    idx, pv = top.indices, top.values
    gate = pv / pv.sum(-1, keepdim=True)
    T = xf.shape[0]
    flat = idx.reshape(-1)
    keep = torch.zeros(2 * T, dtype=torch.bool)
    fc = flat.cpu()
    seen = [0] * E
    for j in range(2 * T):
        e = int(fc[j])
        keep[j] = seen[e] < capacity
        seen[e] += 1
    keep = keep.to(x.device).reshape(T, 2)
    out = torch.zeros_like(xf)
    for k in range(2):
        for e in range(E):
            sel = (idx[:, k] == e) & keep[:, k]
            if sel.any():
                xe = xf[sel].to(torch.bfloat16).float()
                hh = torch.nn.functional.gelu(xe @ w1[e].float().t() + b1[e].float(), approximate="tanh")
                ye = hh.to(torch.bfloat16).float() @ w2[e].float().t() + b2[e].float()
                out[sel] += gate[sel, k:k + 1] * ye.to(torch.bfloat16).float()
    return out, idx, gate, keep
