"""GPT decoder with ZeRO-3 style sharding of the block weights.

The four weight matrices of every block (QKV, attention output, fc1, fc2) are split by output
rows over the ranks (``local_arenas[0]``: bf16 shards in peer-visible memory plus fp32 master /
moments / gradient shards); they are gathered inside the GEMMs that consume them and their
gradients leave the weight-gradient GEMMs already reduce-scattered
(:mod:`frankentorch_b200.parallel.zero3`).  Embeddings, LayerNorm parameters and biases stay
replicated in ``arena`` and go through the fused reduce-scatter + sharded AdamW + all-gather
step of ``FusedDataParallel`` (optimizer state sharded, parameters replicated).

Data parallel semantics: every rank trains on its own micro-batch; the job loss is the mean of
the ranks' losses.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..autograd.tape import TensorTape
from ..ops import fused as F
from ..parallel.fused_gemm import SymmTensor
from ..parallel.zero3 import Zero3Context, zero3_linear
from .gpt import GPTConfig, ParamArena


class Zero3GPT:
    def __init__(self, cfg: GPTConfig, tape: TensorTape, device, *, group: Optional[dist.ProcessGroup],
                 seed: int = 1234, comm_ctas: int = 0):
        self.cfg, self.tape, self.device = cfg, tape, torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        W = self.world
        d, ff, Vp = cfg.d_model, cfg.d_ff, cfg.padded_vocab
        if (d // W) % 128 or (ff // W) % 128 or d % W or ff % W:
            raise ValueError(f"d_model={d} and d_ff={ff} must split into multiples of 128 rows over {W} ranks")
        rep: List[Tuple[str, Tuple[int, ...]]] = [("wte.weight", (Vp, d)), ("wpe.weight", (cfg.max_seq, d))]
        shd: List[Tuple[str, Tuple[int, ...]]] = []
        self.full_shapes: Dict[str, Tuple[int, int]] = {}
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            rep += [(p + "ln1.weight", (d,)), (p + "ln1.bias", (d,)), (p + "attn.qkv_proj.bias", (3 * d,)),
                    (p + "attn.out_proj.bias", (d,)), (p + "ln2.weight", (d,)), (p + "ln2.bias", (d,)),
                    (p + "mlp.fc1.bias", (ff,)), (p + "mlp.fc2.bias", (d,))]
            for name, (o, i) in ((p + "attn.qkv_proj.weight", (3 * d, d)), (p + "attn.out_proj.weight", (d, d)),
                                 (p + "mlp.fc1.weight", (ff, d)), (p + "mlp.fc2.weight", (d, ff))):
                shd.append((name, (o // W, i)))
                self.full_shapes[name] = (o, i)
        rep += [("ln_f.weight", (d,)), ("ln_f.bias", (d,))]
        self.arena = ParamArena(rep, self.device, group=group if W > 1 else None, pad_multiple=1024 * W)
        # the shard arena is always peer-visible: its bf16 copy is what the other ranks gather from
        self.shard_arena = ParamArena(shd, self.device, group=group, pad_multiple=1024) if W > 1 else \
            ParamArena(shd, self.device)
        self.local_arenas = [self.shard_arena]
        self.local_grad_scale = 1.0          # the reduce-scatter already forms the mean over ranks
        self.z = Zero3Context(group, self.device, max_weight_elems=max(3 * d * d, ff * d), comm_ctas=comm_ctas)
        self._init_weights(seed)
        self.leaf: Dict[str, int] = {}
        for arena in (self.arena, self.shard_arena):
            for name, _ in arena.specs:
                nid = tape.leaf(arena.view(arena.params, name), requires_grad=True, name=name)
                tape.bind_grad_buffer(nid, arena.view(arena.grads, name))
                self.leaf[name] = nid
        for name, shape in shd:
            off, _ = self.shard_arena.offsets[name]
            if W > 1:
                st = SymmTensor(self.shard_arena.params_buf, shape, torch.bfloat16, byte_offset=off * 2)
            else:
                st = _LocalShard(self.shard_arena.view(self.shard_arena.params, name))
            self.z.register(self.leaf[name], st)
        self.param_boundary = len(tape)

    def _init_weights(self, seed: int) -> None:
        cfg = self.cfg
        proj_std = 0.02 / math.sqrt(2 * cfg.n_layer)
        for ai, arena in enumerate((self.arena, self.shard_arena)):
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
        """Replicated entries whole, block weights by this rank's output-row range."""
        cfg = self.cfg
        for name, _ in self.arena.specs:
            dst = self.arena.view(self.arena.master, name)
            if name == "wte.weight":
                dst[: cfg.vocab_size].copy_(sd[name].float())
            else:
                dst.copy_(sd[name].float())
        for name, shape in self.shard_arena.specs:
            rows = shape[0]
            self.shard_arena.view(self.shard_arena.master, name).copy_(
                sd[name].float()[self.rank * rows:(self.rank + 1) * rows])
        self.arena.sync_shadow()
        self.shard_arena.sync_shadow()

    def param_count(self) -> int:
        return self.cfg.param_count()

    def begin_step(self) -> None:
        self.z.begin_step()

    def reset_grads(self) -> None:
        for nid in self.leaf.values():
            self.tape.zero_accumulated_gradient(nid)

    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> int:
        cfg, tape, P, z = self.cfg, self.tape, self.leaf, self.z
        B, S = ids.shape
        x = F.embedding(tape, ids, P["wte.weight"], P["wpe.weight"], S)
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            h = F.layernorm(tape, x, P[p + "ln1.weight"], P[p + "ln1.bias"], cfg.ln_eps)
            qkv = zero3_linear(tape, h, P[p + "attn.qkv_proj.weight"], P[p + "attn.qkv_proj.bias"], z)
            a = F.attention_packed(tape, qkv, cfg.n_head, causal=True)
            x = zero3_linear(tape, a, P[p + "attn.out_proj.weight"], P[p + "attn.out_proj.bias"], z, resid=x)
            h = F.layernorm(tape, x, P[p + "ln2.weight"], P[p + "ln2.bias"], cfg.ln_eps)
            u = zero3_linear(tape, h, P[p + "mlp.fc1.weight"], P[p + "mlp.fc1.bias"], z, act=cfg.act)
            x = zero3_linear(tape, u, P[p + "mlp.fc2.weight"], P[p + "mlp.fc2.bias"], z, resid=x)
        h = F.layernorm(tape, x, P["ln_f.weight"], P["ln_f.bias"], cfg.ln_eps)
        return F.lm_head_cross_entropy(tape, h, P["wte.weight"], targets, cfg.vocab_size)


class _LocalShard:
    """Single-rank stand-in for a :class:`SymmTensor` (the only 'peer' is this process)."""

    def __init__(self, t: torch.Tensor):
        self.t = t
        self.peer_ptrs = [t.data_ptr()]
