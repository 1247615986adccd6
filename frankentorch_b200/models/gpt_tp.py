"""Tensor-parallel (+ sequence-parallel) GPT: the decoder of :mod:`frankentorch_b200.models.gpt`
with every block's Linear layers split over the ranks of one NVLink domain.

Per rank: a slice of the global batch's token rows (whole sequences).  Embedding, LayerNorm,
residuals and the LM head + cross-entropy act on local rows; the attention and MLP blocks are
the collective-fused ops of :mod:`frankentorch_b200.parallel.tensor_parallel`.

Two parameter arenas:

* ``arena`` (replicated, peer-visible): embeddings, LayerNorm parameters and the biases that are
  added after a reduce-scatter.  Their per-rank gradients are averaged by the fused
  reduce-scatter + sharded AdamW + all-gather step of ``FusedDataParallel``.
* ``local_arenas[0]`` (this rank's weight shards): QKV / fc1 row blocks with their biases and
  attention-output / fc2 column blocks, updated by the plain fused AdamW with gradients scaled
  by ``1 / world`` (``local_grad_scale``).

The reference has no model parallelism; module composition follows ft-nn (Linear lib.rs:902,
LayerNorm :2042, MultiheadAttention :4685).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..autograd.tape import TensorTape
from ..ops import fused as F
from ..parallel.tensor_parallel import TPContext, tp_attention, tp_mlp
from .gpt import GPTConfig, ParamArena


class TensorParallelGPT:
    def __init__(self, cfg: GPTConfig, tape: TensorTape, device, *, group: Optional[dist.ProcessGroup],
                 micro_batch: int, seq_len: int, seed: int = 1234, comm_ctas: int = 0):
        self.cfg, self.tape, self.device = cfg, tape, torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        W = self.world
        d, ff, Vp = cfg.d_model, cfg.d_ff, cfg.padded_vocab
        if cfg.n_head % W or ff % W or d % W:
            raise ValueError(f"heads={cfg.n_head}, d_ff={ff}, d_model={d} must divide by the {W} ranks")
        self.dl, self.ffl, self.heads_local = d // W, ff // W, cfg.n_head // W
        self.seq_len = seq_len
        rows = micro_batch * seq_len
        if rows % 128:
            raise ValueError("tokens per rank must be a multiple of 128")
        self.ctx = TPContext(group, self.device, rows_per_rank=rows, d_model=d, comm_ctas=comm_ctas)
        rep: List[Tuple[str, Tuple[int, ...]]] = [("wte.weight", (Vp, d)), ("wpe.weight", (cfg.max_seq, d))]
        loc: List[Tuple[str, Tuple[int, ...]]] = []
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            rep += [(p + "ln1.weight", (d,)), (p + "ln1.bias", (d,)), (p + "attn.out_proj.bias", (d,)),
                    (p + "ln2.weight", (d,)), (p + "ln2.bias", (d,)), (p + "mlp.fc2.bias", (d,))]
            loc += [(p + "attn.qkv_proj.weight", (3 * self.dl, d)), (p + "attn.qkv_proj.bias", (3 * self.dl,)),
                    (p + "attn.out_proj.weight", (d, self.dl)),
                    (p + "mlp.fc1.weight", (self.ffl, d)), (p + "mlp.fc1.bias", (self.ffl,)),
                    (p + "mlp.fc2.weight", (d, self.ffl))]
        rep += [("ln_f.weight", (d,)), ("ln_f.bias", (d,))]
        self.arena = ParamArena(rep, self.device, group=group if W > 1 else None, pad_multiple=1024 * W)
        self.local_arena = ParamArena(loc, self.device)
        self.local_arenas = [self.local_arena]
        self.local_grad_scale = 1.0 / W
        self._init_weights(seed)
        self.leaf: Dict[str, int] = {}
        for arena in (self.arena, self.local_arena):
            for name, _ in arena.specs:
                nid = tape.leaf(arena.view(arena.params, name), requires_grad=True, name=name)
                tape.bind_grad_buffer(nid, arena.view(arena.grads, name))
                self.leaf[name] = nid
        self.param_boundary = len(tape)
        from ..ops.fused import enable_grouped_wgrad
        enable_grouped_wgrad(tape)       # a block's weight gradients are launched together

    # ------------------------------------------------------------------ initialisation
    def _init_weights(self, seed: int) -> None:
        """Random init on the device; every rank draws the same replicated values and its own shards."""
        cfg = self.cfg
        proj_std = 0.02 / math.sqrt(2 * cfg.n_layer)
        for ai, arena in enumerate((self.arena, self.local_arena)):
            for pi, (name, shape) in enumerate(arena.specs):
                dst = arena.view(arena.master, name)
                if name.endswith(".bias"):
                    dst.zero_()
                elif ".ln" in name or name.startswith("ln_f"):
                    dst.fill_(1.0)
                else:
                    std = proj_std if ("out_proj.weight" in name or "fc2.weight" in name) else 0.02
                    g = torch.Generator(device=self.device)
                    g.manual_seed(seed * 1000003 + pi * 131 + (self.rank + 1 if ai == 1 else 0))
                    dst.copy_(torch.randn(shape, generator=g, device=self.device, dtype=torch.float32) * std)
                    if name == "wte.weight":
                        dst[cfg.vocab_size:] = 0.0
            arena.sync_shadow()

    def load_full_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """Take this rank's slices of an unsharded GPT ``state_dict`` (q / k / v rows of its heads,
        matching columns of the output projection, its fc1 rows / fc2 columns)."""
        cfg, r, dl, ffl, d = self.cfg, self.rank, self.dl, self.ffl, self.cfg.d_model
        for name, shape in self.arena.specs:
            t = sd[name].float()
            dst = self.arena.view(self.arena.master, name)
            if name == "wte.weight":
                dst[: cfg.vocab_size].copy_(t)
            else:
                dst.copy_(t)
        for name, shape in self.local_arena.specs:
            t = sd[name].float()
            if name.endswith("qkv_proj.weight"):
                t = torch.cat([t[i * d + r * dl: i * d + (r + 1) * dl] for i in range(3)])
            elif name.endswith("qkv_proj.bias"):
                t = torch.cat([t[i * d + r * dl: i * d + (r + 1) * dl] for i in range(3)])
            elif name.endswith("out_proj.weight"):
                t = t[:, r * dl:(r + 1) * dl]
            elif name.endswith("fc1.weight") or name.endswith("fc1.bias"):
                t = t[r * ffl:(r + 1) * ffl]
            elif name.endswith("fc2.weight"):
                t = t[:, r * ffl:(r + 1) * ffl]
            self.local_arena.view(self.local_arena.master, name).copy_(t.contiguous())
        self.arena.sync_shadow()
        self.local_arena.sync_shadow()

    def param_count(self) -> int:
        return self.cfg.param_count()

    # ------------------------------------------------------------------ step protocol
    def begin_step(self) -> None:
        self.ctx.begin_step()

    def reset_grads(self) -> None:
        for nid in self.leaf.values():
            self.tape.zero_accumulated_gradient(nid)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> int:
        """``ids`` / ``targets``: this rank's ``[micro_batch, seq]`` sequences; returns the local mean loss."""
        cfg, tape, P = self.cfg, self.tape, self.leaf
        B, S = ids.shape
        x = F.embedding(tape, ids, P["wte.weight"], P["wpe.weight"], S)
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            h = F.layernorm(tape, x, P[p + "ln1.weight"], P[p + "ln1.bias"], cfg.ln_eps)
            x = tp_attention(tape, h, P[p + "attn.qkv_proj.weight"], P[p + "attn.qkv_proj.bias"],
                             P[p + "attn.out_proj.weight"], P[p + "attn.out_proj.bias"], x, self.ctx,
                             heads_local=self.heads_local, seq_len=S)
            h = F.layernorm(tape, x, P[p + "ln2.weight"], P[p + "ln2.bias"], cfg.ln_eps)
            x = tp_mlp(tape, h, P[p + "mlp.fc1.weight"], P[p + "mlp.fc1.bias"], P[p + "mlp.fc2.weight"],
                       P[p + "mlp.fc2.bias"], x, self.ctx, act=cfg.act)
        h = F.layernorm(tape, x, P["ln_f.weight"], P["ln_f.bias"], cfg.ln_eps)
        return F.lm_head_cross_entropy(tape, h, P["wte.weight"], targets, cfg.vocab_size)
