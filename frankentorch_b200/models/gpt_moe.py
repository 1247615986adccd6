"""Mixture-of-experts GPT decoder with expert parallelism.

Every block keeps the dense attention sub-layer of :mod:`frankentorch_b200.models.gpt` and
replaces the MLP by the top-2 routed expert layer of :mod:`frankentorch_b200.parallel.moe`
(8 experts of FFN width ``d_ff`` by default, capacity factor 1.25).  Experts are spread over the
ranks; tokens travel to their experts and back through the peer-memory dispatch / combine
kernels.

Parameters: ``arena`` holds what every rank replicates (embeddings, LayerNorm, attention
weights, router weights) and is reduced across ranks like a data-parallel model;
``local_arenas[0]`` holds this rank's experts.  An expert receives the upstream gradients of all
ranks' tokens, i.e. ``world`` times the gradient of the job loss (the mean of the ranks' local
mean losses), hence ``local_grad_scale = 1 / world``.

The reference has no MoE layer; the dense parts follow ft-nn (MultiheadAttention lib.rs:4685,
LayerNorm :2042, Linear :902).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..autograd.tape import TensorTape
from ..ops import fused as F
from ..parallel.moe import ROUTER_ROWS, ExpertParallel, moe_ffn
from .gpt import GPTConfig, ParamArena


@dataclass
class MoEConfig:
    n_experts: int = 8
    capacity_factor: float = 1.25

    @staticmethod
    def gpt_preset(name: str) -> GPTConfig:
        presets = {
            "moe-12l": dict(n_layer=12, d_model=1024, n_head=16, d_ff=4096, max_seq=2048),
            "moe-tiny": dict(n_layer=2, d_model=128, n_head=2, d_ff=256, max_seq=128, vocab_size=1000),
        }
        return GPTConfig(name=name, **presets[name])


class MoEGPT:
    def __init__(self, cfg: GPTConfig, moe: MoEConfig, tape: TensorTape, device, *,
                 group: Optional[dist.ProcessGroup], micro_batch: int, seq_len: int, seed: int = 1234):
        self.cfg, self.moe, self.tape, self.device = cfg, moe, tape, torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        W = self.world
        d, ff, Vp = cfg.d_model, cfg.d_ff, cfg.padded_vocab
        self.ep = ExpertParallel(group, self.device, tokens=micro_batch * seq_len, d_model=d,
                                 n_experts=moe.n_experts, capacity_factor=moe.capacity_factor)
        el = self.ep.e_local
        self.bufs = [self.ep.new_layer_buffers() for _ in range(cfg.n_layer)]
        rep: List[Tuple[str, Tuple[int, ...]]] = [("wte.weight", (Vp, d)), ("wpe.weight", (cfg.max_seq, d))]
        loc: List[Tuple[str, Tuple[int, ...]]] = []
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            rep += [(p + "ln1.weight", (d,)), (p + "ln1.bias", (d,)),
                    (p + "attn.qkv_proj.weight", (3 * d, d)), (p + "attn.qkv_proj.bias", (3 * d,)),
                    (p + "attn.out_proj.weight", (d, d)), (p + "attn.out_proj.bias", (d,)),
                    (p + "ln2.weight", (d,)), (p + "ln2.bias", (d,)),
                    (p + "moe.router.weight", (ROUTER_ROWS, d))]
            loc += [(p + "moe.experts.w1", (el, ff, d)), (p + "moe.experts.b1", (el, ff)),
                    (p + "moe.experts.w2", (el, d, ff)), (p + "moe.experts.b2", (el, d))]
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

    def _init_weights(self, seed: int) -> None:
        cfg = self.cfg
        proj_std = 0.02 / math.sqrt(2 * cfg.n_layer)
        for ai, arena in enumerate((self.arena, self.local_arena)):
            for pi, (name, shape) in enumerate(arena.specs):
                dst = arena.view(arena.master, name)
                if name.endswith(".bias") or name.endswith(".b1") or name.endswith(".b2"):
                    dst.zero_()
                elif ".ln" in name or name.startswith("ln_f"):
                    dst.fill_(1.0)
                else:
                    std = proj_std if (name.endswith("out_proj.weight") or name.endswith(".w2")) else 0.02
                    g = torch.Generator(device=self.device)
                    g.manual_seed(seed * 1000003 + pi * 131 + (self.rank + 1 if ai == 1 else 0))
                    dst.copy_(torch.randn(shape, generator=g, device=self.device, dtype=torch.float32) * std)
                    if name == "wte.weight":
                        dst[cfg.vocab_size:] = 0.0
                    if name.endswith("router.weight"):
                        dst[self.moe.n_experts:] = 0.0      # only the first E rows are experts
            arena.sync_shadow()

    def param_count(self) -> int:
        """Parameters of the whole model (all experts of all ranks)."""
        cfg, E = self.cfg, self.moe.n_experts
        d, ff = cfg.d_model, cfg.d_ff
        per_layer = 4 * d + 3 * d * d + 3 * d + d * d + d + E * d + E * (2 * d * ff + ff + d)
        return cfg.vocab_size * d + cfg.max_seq * d + cfg.n_layer * per_layer + 2 * d

    def reset_grads(self) -> None:
        for nid in self.leaf.values():
            self.tape.zero_accumulated_gradient(nid)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> int:
        cfg, tape, P = self.cfg, self.tape, self.leaf
        B, S = ids.shape
        x = F.embedding(tape, ids, P["wte.weight"], P["wpe.weight"], S)
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            h = F.layernorm(tape, x, P[p + "ln1.weight"], P[p + "ln1.bias"], cfg.ln_eps)
            qkv = F.linear(tape, h, P[p + "attn.qkv_proj.weight"], P[p + "attn.qkv_proj.bias"])
            a = F.attention_packed(tape, qkv, cfg.n_head, causal=True)
            x = F.linear(tape, a, P[p + "attn.out_proj.weight"], P[p + "attn.out_proj.bias"], resid=x)
            h = F.layernorm(tape, x, P[p + "ln2.weight"], P[p + "ln2.bias"], cfg.ln_eps)
            x = moe_ffn(tape, h, P[p + "moe.router.weight"], P[p + "moe.experts.w1"], P[p + "moe.experts.b1"],
                        P[p + "moe.experts.w2"], P[p + "moe.experts.b2"], self.ep, self.bufs[l],
                        resid=x, act=cfg.act)
        h = F.layernorm(tape, x, P["ln_f.weight"], P["ln_f.bias"], cfg.ln_eps)
        return F.lm_head_cross_entropy(tape, h, P["wte.weight"], targets, cfg.vocab_size)
