"""Decoder-only GPT (GPT-2 family) on the DAC tape with the sm_100a fused operators.

The reference ships the parts (Embedding ft-nn/src/lib.rs:2873, LayerNorm :2042,
Linear :902, MultiheadAttention :4685 + SDPA :5178, GELU :1927, cross-entropy, AdamW)
but no decoder LM; this module composes them as a pre-LN GPT-2 block stack with a
weight-tied LM head.  State-dict keys are dotted module paths in sorted order, like
`module_state_dict` (ft-nn/src/lib.rs:651).

All parameters live in one flat arena (bf16 compute copy, fp32 master, fp32 gradient,
AdamW moments) so the optimizer, gradient clipping and the multi-GPU reduce-scatter
each run as one kernel over contiguous memory.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..autograd.tape import TensorTape
from ..ops import fused as F


@dataclass
class GPTConfig:
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    d_ff: int = 3072
    vocab_size: int = 50257
    max_seq: int = 1024
    act: str = "gelu_tanh"          # GPT-2 checkpoints use the tanh form
    ln_eps: float = 1e-5
    tie_lm_head: bool = True
    name: str = "gpt2-small"

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 127) // 128 * 128

    @staticmethod
    def preset(name: str) -> "GPTConfig":
        presets = {
            "gpt2-small": dict(n_layer=12, d_model=768, n_head=12, d_ff=3072, max_seq=1024),
            "gpt2-medium": dict(n_layer=24, d_model=1024, n_head=16, d_ff=4096, max_seq=2048),
            "gpt-1.3b": dict(n_layer=24, d_model=2048, n_head=16, d_ff=8192, max_seq=2048),
            "gpt-tiny": dict(n_layer=2, d_model=128, n_head=2, d_ff=512, max_seq=128, vocab_size=1000),
        }
        if name not in presets:
            raise KeyError(f"unknown GPT preset {name!r}; have {sorted(presets)}")
        return GPTConfig(name=name, **presets[name])

    def param_count(self) -> int:
        d, L = self.d_model, self.n_layer
        per_layer = 4 * d + 3 * d * d + 3 * d + d * d + d + d * self.d_ff + self.d_ff + self.d_ff * d + d
        return self.vocab_size * d + self.max_seq * d + L * per_layer + 2 * d


class ParamArena:
    """Flat parameter storage: bf16 compute copy + fp32 master/grad/moments, 256-byte aligned slots.

    With a process ``group`` the gradient and parameter arenas are allocated in peer-visible
    (symmetric) memory so the multi-GPU kernels can read / write them over NVLink, and the total
    length is padded so it splits into equal float4-aligned shards.
    """

    ALIGN = 128  # elements

    def __init__(self, specs: List[Tuple[str, Tuple[int, ...]]], device, *, group=None, pad_multiple: int = 1024,
                 peer_visible: bool = False, multicast_params: bool = False):
        self.specs = specs
        self.offsets: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
        off = 0
        for name, shape in specs:
            n = int(math.prod(shape))
            self.offsets[name] = (off, tuple(shape))
            off += (n + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        off = (off + pad_multiple - 1) // pad_multiple * pad_multiple
        self.numel = off
        self.symmetric = group is not None or peer_visible   # (a one-rank job can use the peer kernels too)
        if self.symmetric:
            from ..parallel.symm import SymmetricBuffer
            self.params_buf = (self._multicast_params(off * 2, group, device) if multicast_params else None) or \
                SymmetricBuffer(off * 2, group, device)
            self.grads_buf = SymmetricBuffer(off * 4, group, device)
            self.params = self.params_buf.tensor(torch.bfloat16, off)
            self.grads = self.grads_buf.tensor(torch.float32, off)
        else:
            self.params = torch.zeros(off, dtype=torch.bfloat16, device=device)
            self.grads = torch.zeros(off, dtype=torch.float32, device=device)
        # arena offsets where a data-parallel gradient bucket must end (see parallel/data_parallel.py)
        self.bucket_cuts: List[int] = []
        self.master = torch.zeros(off, dtype=torch.float32, device=device)
        self.m = torch.zeros(off, dtype=torch.float32, device=device)
        self.v = torch.zeros(off, dtype=torch.float32, device=device)

    @staticmethod
    def _multicast_params(nbytes: int, group, device):
        """The parameter arena as a multicast (NVLS) buffer when ``FT_DP_NVLS`` asks for it (``1``, or ``auto`` =
        jobs of eight or more ranks) and the system offers a multicast address; None otherwise.  The
        data-parallel update then broadcasts the new bf16 parameters with one multimem store per value.
        Off by default: on 2 and 4 GPUs the step time was the same with either form (12.75 / 12.72 and
        12.76 / 12.72 ms), the egress saving only matters with more peers."""
        import os
        want = os.environ.get("FT_DP_NVLS", "0")
        if group is None or want == "0":
            return None
        import torch.distributed as dist
        world = dist.get_world_size(group)
        if world < 2 or (want == "auto" and world < 8) or torch.device(device).type != "cuda":
            return None
        try:
            from ..parallel.nvls import MulticastBuffer
            buf = MulticastBuffer(nbytes, group, device)
        except Exception:       # no symmetric-memory support in this build / on this system: peer stores
            buf = None
        # every rank takes the same path: one that could not bind the object sends all back to peer stores
        ok = torch.tensor([1 if (buf is not None and buf.has_multicast) else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        return buf if int(ok) == 1 else None

    def slot_end(self, name: str) -> int:
        """One past the last arena element of the (128-aligned) slot of parameter ``name``."""
        off, shape = self.offsets[name]
        n = int(math.prod(shape))
        return off + (n + self.ALIGN - 1) // self.ALIGN * self.ALIGN

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        off, shape = self.offsets[name]
        return flat[off: off + int(math.prod(shape))].view(shape)

    def sync_shadow(self) -> None:
        self.params.copy_(self.master)

    def drop_full_optimizer_state(self) -> None:
        """Called by a sharded optimizer that now owns its slice of master / m / v."""
        self.master = self.m = self.v = None


class GPT:
    """GPT-2 style decoder; ``forward`` records the step on a :class:`TensorTape`."""

    def __init__(self, cfg: GPTConfig, tape: TensorTape, device="cuda", seed: int = 1234, *, group=None,
                 peer_visible: bool = False):
        self.cfg = cfg
        self.tape = tape
        self.device = torch.device(device)
        d, ff, Vp = cfg.d_model, cfg.d_ff, cfg.padded_vocab
        specs: List[Tuple[str, Tuple[int, ...]]] = [("wte.weight", (Vp, d)), ("wpe.weight", (cfg.max_seq, d))]
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            specs += [
                (p + "ln1.weight", (d,)), (p + "ln1.bias", (d,)),
                (p + "attn.qkv_proj.weight", (3 * d, d)), (p + "attn.qkv_proj.bias", (3 * d,)),
                (p + "attn.out_proj.weight", (d, d)), (p + "attn.out_proj.bias", (d,)),
                (p + "ln2.weight", (d,)), (p + "ln2.bias", (d,)),
                (p + "mlp.fc1.weight", (ff, d)), (p + "mlp.fc1.bias", (ff,)),
                (p + "mlp.fc2.weight", (d, ff)), (p + "mlp.fc2.bias", (d,)),
            ]
        specs += [("ln_f.weight", (d,)), ("ln_f.bias", (d,))]
        if not cfg.tie_lm_head:
            specs.append(("lm_head.weight", (Vp, d)))
        world = 1
        if group is not None:
            import torch.distributed as dist
            world = dist.get_world_size(group)
        self.arena = ParamArena(specs, self.device, group=group, pad_multiple=1024 * world,
                                peer_visible=peer_visible, multicast_params=True)
        # the embeddings' gradients are complete only when the backward pass ends (the token table is
        # also the LM head): they form one bucket of their own
        self.arena.bucket_cuts.append(self.arena.slot_end("wpe.weight"))
        # the weight gradients of a block are launched together (two full waves, no split-K)
        from ..ops.fused import enable_grouped_wgrad
        enable_grouped_wgrad(tape)
        self._init_weights(seed)
        # parameters are the lowest-index leaves of the tape; the per-step graph is truncated above
        self.leaf: Dict[str, int] = {}
        for name, _ in specs:
            nid = tape.leaf(self.arena.view(self.arena.params, name), requires_grad=True, name=name)
            tape.bind_grad_buffer(nid, self.arena.view(self.arena.grads, name))
            self.leaf[name] = nid
        self.param_boundary = len(tape)
        # set by the training engine: called with a parameter name before the forward pass reads that
        # parameter (and everything before it in the arena), see FusedDataParallel.gate_param
        self.param_gate = None

    def _init_weights(self, seed: int) -> None:
        cfg, a = self.cfg, self.arena
        g = torch.Generator(device="cpu").manual_seed(seed)
        proj_std = 0.02 / math.sqrt(2 * cfg.n_layer)
        for name, shape in a.specs:
            dst = a.view(a.master, name)
            if name.endswith(".bias"):
                dst.zero_()
            elif ".ln" in name or name.startswith("ln_f"):
                dst.fill_(1.0)
            else:
                std = proj_std if (name.endswith("out_proj.weight") or name.endswith("fc2.weight")) else 0.02
                w = torch.randn(shape, generator=g, dtype=torch.float32) * std
                if name in ("wte.weight", "lm_head.weight"):
                    w[cfg.vocab_size:] = 0.0   # padding rows
                dst.copy_(w)
        a.sync_shadow()

    # ------------------------------------------------------------------ module-style accessors
    def named_parameters(self) -> List[Tuple[str, torch.Tensor]]:
        return [(n, self.arena.view(self.arena.master, n)) for n, _ in self.arena.specs]

    def parameters(self) -> List[int]:
        return [self.leaf[n] for n, _ in self.arena.specs]

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """fp32 master weights keyed by dotted module path, in sorted key order."""
        sd = {}
        for name, shape in self.arena.specs:
            t = self.arena.view(self.arena.master, name)
            if name in ("wte.weight", "lm_head.weight"):
                t = t[: self.cfg.vocab_size]
            sd[name] = t.detach().clone()
        return dict(sorted(sd.items()))

    def load_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True):
        own = {n: s for n, s in self.arena.specs}
        missing = [k for k in own if k not in sd]
        unexpected = [k for k in sd if k not in own]
        if strict and (missing or unexpected):
            raise KeyError(f"load_state_dict(strict): missing={missing} unexpected={unexpected}")
        # validate every shape before mutating anything (all-or-nothing, ft-nn/src/lib.rs:700-731)
        for k, t in sd.items():
            if k not in own:
                continue
            want = list(own[k])
            if k in ("wte.weight", "lm_head.weight"):
                want[0] = self.cfg.vocab_size
            if list(t.shape) != want:
                raise ValueError(f"shape mismatch for {k}: {tuple(t.shape)} vs {tuple(want)}")
        for k, t in sd.items():
            if k not in own:
                continue
            dst = self.arena.view(self.arena.master, k)
            if k in ("wte.weight", "lm_head.weight"):
                dst = dst[: self.cfg.vocab_size]
            dst.copy_(t.to(dst.device, torch.float32))
        self.arena.sync_shadow()
        return {"missing_keys": missing, "unexpected_keys": unexpected}

    # ------------------------------------------------------------------ forward
    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> int:
        """Record one training forward; returns the tape id of the scalar mean loss."""
        cfg, tape, P = self.cfg, self.tape, self.leaf
        B, S = ids.shape
        gate = self.param_gate
        if gate is not None:
            gate("wpe.weight")
        x = F.embedding(tape, ids, P["wte.weight"], P["wpe.weight"], S)
        for l in range(cfg.n_layer):
            p = f"blocks.{l}."
            if gate is not None:
                gate(p + "mlp.fc2.bias")
            h = F.layernorm(tape, x, P[p + "ln1.weight"], P[p + "ln1.bias"], cfg.ln_eps)
            qkv = F.linear(tape, h, P[p + "attn.qkv_proj.weight"], P[p + "attn.qkv_proj.bias"])
            a = F.attention_packed(tape, qkv, cfg.n_head, causal=True)
            x = F.linear(tape, a, P[p + "attn.out_proj.weight"], P[p + "attn.out_proj.bias"], resid=x)
            h = F.layernorm(tape, x, P[p + "ln2.weight"], P[p + "ln2.bias"], cfg.ln_eps)
            x = F.mlp_up_down(tape, h, P[p + "mlp.fc1.weight"], P[p + "mlp.fc1.bias"],
                              P[p + "mlp.fc2.weight"], P[p + "mlp.fc2.bias"], x, act=cfg.act)
        if gate is not None:
            gate("ln_f.bias")
        h = F.layernorm(tape, x, P["ln_f.weight"], P["ln_f.bias"], cfg.ln_eps)
        head = P["wte.weight"] if cfg.tie_lm_head else P["lm_head.weight"]
        return F.lm_head_cross_entropy(tape, h, head, targets, cfg.vocab_size)

    def reset_grads(self) -> None:
        """Mark every gradient slot empty: the first contribution of the next backward overwrites."""
        for nid in self.leaf.values():
            self.tape.zero_accumulated_gradient(nid)
