#!/usr/bin/env python
"""Stock PyTorch arm of the headline benchmark: the same GPT-2 training step written with
``torch.nn`` modules, cuBLAS GEMMs, ``F.scaled_dot_product_attention`` (flash), bf16 autocast
with fp32 master weights, fused ``torch.optim.AdamW``, gradient clipping, and
``DistributedDataParallel`` (NCCL all-reduce) or ``FullyShardedDataParallel`` on more than one
GPU; ``--parallel tp`` is a Megatron-style tensor + sequence parallel GPT (NCCL all-gather /
reduce-scatter around column- and row-parallel ``nn.Linear``), ``--parallel ep`` a top-2
mixture-of-experts GPT with ``all_to_all_single`` dispatch / combine and ``torch.bmm`` experts.  Nothing of this repository's kernels or engine is on this path.  ``bench.py`` imports
:class:`TorchArm` to sample this arm interleaved with its own in one invocation.

    python benchmarks/torch_baseline.py --model gpt2-small --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29501 benchmarks/torch_baseline.py --model gpt2-small

Prints one JSON line with the same metric as ``bench.py`` (train tokens/sec, whole job, device
timed with CUDA events, max over ranks).
"""
import argparse
import json
import math
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

PRESETS = {
    "gpt2-small": dict(n_layer=12, d=768, h=12, ff=3072, mb=8, seq=1024),
    "gpt2-medium": dict(n_layer=24, d=1024, h=16, ff=4096, mb=4, seq=2048),
    "gpt-1.3b": dict(n_layer=24, d=2048, h=16, ff=8192, mb=4, seq=2048),
    "gpt-tiny": dict(n_layer=2, d=128, h=2, ff=512, mb=4, seq=128),
    "moe-12l": dict(n_layer=12, d=1024, h=16, ff=4096, mb=4, seq=2048, experts=8, capacity_factor=1.25),
    "moe-tiny": dict(n_layer=2, d=128, h=2, ff=256, mb=4, seq=128, experts=8, capacity_factor=1.25, vocab=1000),
}
VOCAB = 50257


class Block(nn.Module):
    def __init__(self, d, h, ff):
        super().__init__()
        self.h = h
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, ff), nn.Linear(ff, d)

    def forward(self, x):
        B, S, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.h, d // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, d)
        x = x + self.proj(a)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class GPT(nn.Module):
    def __init__(self, n_layer, d, h, ff, seq, vocab=VOCAB):
        super().__init__()
        self.vp = (vocab + 127) // 128 * 128
        self.wte, self.wpe = nn.Embedding(self.vp, d), nn.Embedding(seq, d)
        self.blocks = nn.ModuleList(Block(d, h, ff) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d)
        for n, p in self.named_parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02 / math.sqrt(2 * n_layer) if ("proj" in n or "fc2" in n) else 0.02)

    def forward(self, ids, targets):
        pos = torch.arange(ids.shape[1], device=ids.device)
        x = self.wte(ids) + self.wpe(pos)
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.view(-1))


# ---------------------------------------------------------------- tensor + sequence parallel (Megatron style)
class _GatherRows(torch.autograd.Function):
    """all-gather along dim 0 in forward, reduce-scatter of the gradient in backward (NCCL)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * w,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] // w,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ScatterRows(torch.autograd.Function):
    """reduce-scatter along dim 0 in forward, all-gather of the gradient in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = torch.empty((x.shape[0] // w,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] * w,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class TPBlock(nn.Module):
    """Column-parallel QKV / fc1, row-parallel proj / fc2, LayerNorm and residuals on sequence shards."""

    def __init__(self, d, h, ff, world, group, mb, seq):
        super().__init__()
        self.hl, self.hd, self.world, self.group, self.mb, self.seq = h // world, d // h, world, group, mb, seq
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d // world), nn.Linear(d // world, d, bias=False)
        self.fc1, self.fc2 = nn.Linear(d, ff // world), nn.Linear(ff // world, d, bias=False)
        self.proj_b, self.fc2_b = nn.Parameter(torch.zeros(d)), nn.Parameter(torch.zeros(d))

    def forward(self, x):                                   # x: [B*S/W, d], rows sharded over the ranks
        g = self.group
        a = _GatherRows.apply(self.ln1(x), g)               # [B*S, d]
        q, k, v = self.qkv(a).view(self.mb, self.seq, 3, self.hl, self.hd).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(self.mb * self.seq, -1)
        x = x + _ScatterRows.apply(self.proj(o), g) + self.proj_b
        a = _GatherRows.apply(self.ln2(x), g)
        u = F.gelu(self.fc1(a), approximate="tanh")
        return x + _ScatterRows.apply(self.fc2(u), g) + self.fc2_b


class TPGPT(nn.Module):
    def __init__(self, n_layer, d, h, ff, seq, world, group, mb, vocab=VOCAB):
        super().__init__()
        self.vp = (vocab + 127) // 128 * 128
        self.world, self.group, self.rank = world, group, dist.get_rank(group)
        self.wte, self.wpe = nn.Embedding(self.vp, d), nn.Embedding(seq, d)
        self.blocks = nn.ModuleList(TPBlock(d, h, ff, world, group, mb, seq) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d)
        for n, p in self.named_parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02 / math.sqrt(2 * n_layer) if ("proj" in n or "fc2" in n) else 0.02)

    def forward(self, ids, targets):
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device)
        x = (self.wte(ids) + self.wpe(pos)).view(B * S, -1)
        rows = B * S // self.world
        x = x[self.rank * rows:(self.rank + 1) * rows]      # sequence parallel: this rank's rows
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        t = targets.reshape(-1)[self.rank * rows:(self.rank + 1) * rows]
        return F.cross_entropy(logits.float(), t) / self.world      # summed over the ranks = the job's mean loss

    def sharded(self, name: str) -> bool:
        return any(k in name for k in ("qkv.", "proj.weight", "fc1.", "fc2.weight"))


# ---------------------------------------------------------------- expert parallel mixture of experts
class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g.contiguous(), group=ctx.group)
        return out, None


class MoEBlock(nn.Module):
    """Attention block + top-2 mixture of experts with fixed capacity: scatter into per-expert slots,
    ``all_to_all_single`` to the experts' ranks, batched expert MLPs (``torch.bmm``), all-to-all back, gather."""

    def __init__(self, d, h, ff, experts, cap, world, group):
        super().__init__()
        self.h, self.E, self.cap, self.world, self.group = h, experts, cap, world, group
        el = experts // world
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.router = nn.Linear(d, experts, bias=False)
        self.w1, self.b1 = nn.Parameter(torch.empty(el, d, ff)), nn.Parameter(torch.zeros(el, 1, ff))
        self.w2, self.b2 = nn.Parameter(torch.empty(el, ff, d)), nn.Parameter(torch.zeros(el, 1, d))

    def forward(self, x):
        B, S, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.h, d // self.h).permute(2, 0, 3, 1, 4)
        x = x + self.proj(F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, d))
        t = self.ln2(x).view(B * S, d)
        probs = F.softmax(self.router(t).float(), dim=-1)
        gate, idx = probs.topk(2, dim=-1)                                   # [T, 2]
        gate = (gate / gate.sum(-1, keepdim=True)).to(t.dtype)
        flat = idx.reshape(-1)                                              # assignment a = 2 t + k
        onehot = F.one_hot(flat, self.E)
        slot = (onehot.cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1)   # position inside the expert's buffer
        keep = slot < self.cap
        dest = torch.where(keep, flat * self.cap + slot, torch.full_like(flat, self.E * self.cap))
        send = torch.zeros(self.E * self.cap + 1, d, dtype=t.dtype, device=t.device)
        send = send.index_copy(0, dest, t.repeat_interleave(2, dim=0))[:-1]
        el = self.E // self.world
        if self.world > 1:
            recv = _AllToAll.apply(send, self.group)                        # [W, el, cap, d] by source rank
        else:
            recv = send
        xe = recv.view(self.world, el, self.cap, d).transpose(0, 1).reshape(el, self.world * self.cap, d)
        ye = torch.bmm(F.gelu(torch.bmm(xe, self.w1.to(xe.dtype)) + self.b1.to(xe.dtype), approximate="tanh"),
                       self.w2.to(xe.dtype)) + self.b2.to(xe.dtype)
        back = ye.view(el, self.world, self.cap, d).transpose(0, 1).reshape(self.E * self.cap, d)
        if self.world > 1:
            back = _AllToAll.apply(back, self.group)
        back = torch.cat([back, back.new_zeros(1, d)])
        y2 = back.index_select(0, dest).view(B * S, 2, d)                   # dropped assignments read the zero row
        return x + (y2 * gate.unsqueeze(-1)).sum(1).view(B, S, d)


class MoEGPT(nn.Module):
    def __init__(self, n_layer, d, h, ff, seq, experts, cap, world, group, vocab=VOCAB):
        super().__init__()
        self.vp = (vocab + 127) // 128 * 128
        self.wte, self.wpe = nn.Embedding(self.vp, d), nn.Embedding(seq, d)
        self.blocks = nn.ModuleList(MoEBlock(d, h, ff, experts, cap, world, group) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d)
        for n, p in self.named_parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02 / math.sqrt(2 * n_layer) if ("proj" in n or "w2" in n) else 0.02)

    def forward(self, ids, targets):
        pos = torch.arange(ids.shape[1], device=ids.device)
        x = self.wte(ids) + self.wpe(pos)
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.view(-1))

    def sharded(self, name: str) -> bool:
        return any(name.endswith(k) for k in (".w1", ".b1", ".w2", ".b2"))


class TorchArm:
    """The stock-PyTorch training step as an object, so a harness can interleave it with another arm.

    ``parallel``: ``"ddp"`` (DistributedDataParallel, NCCL all-reduce) or ``"fsdp"``
    (FullyShardedDataParallel, full sharding per transformer block, bf16 compute parameters, fp32
    reduce).  With one rank both are the plain module.  The arm reports its own version
    (``version_line``) and the region it times (``timed_steps_line``)."""

    TIMED_STEPS = ("forward", "backward", "clip", "optimizer")

    def __init__(self, model_name: str, dev, world: int = 1, rank: int = 0, parallel: str = "ddp",
                 micro_batch: int = 0, seq_len: int = 0):
        c = dict(PRESETS[model_name])
        if micro_batch:
            c["mb"] = micro_batch
        if seq_len:
            c["seq"] = seq_len
        self.cfg, self.dev, self.world, self.parallel = c, dev, world, parallel
        torch.manual_seed(1234)
        self.manual_sync = False
        group = dist.group.WORLD if world > 1 else None
        vocab = c.get("vocab", VOCAB)
        if parallel == "tp" and world > 1:
            # the job's batch is micro_batch x world sequences (the same on every rank; each rank owns the rows
            # of micro_batch sequences between the blocks' collectives), as in this repository's TP + SP model
            model = TPGPT(c["n_layer"], c["d"], c["h"], c["ff"], c["seq"], world, group, c["mb"] * world, vocab).to(dev)
            self.manual_sync, self.grad_div = True, 1.0          # the loss is already divided by the world size
        elif parallel == "ep":
            tokens = c["mb"] * c["seq"]
            cap = (int(math.ceil(c["capacity_factor"] * tokens * 2 / c["experts"])) + 127) // 128 * 128
            model = MoEGPT(c["n_layer"], c["d"], c["h"], c["ff"], c["seq"], c["experts"], cap, world, group, vocab).to(dev)
            self.manual_sync, self.grad_div = world > 1, float(world)
        else:
            model = GPT(c["n_layer"], c["d"], c["h"], c["ff"], c["seq"], vocab).to(dev)
        self.model = model
        self.fsdp = False
        if self.manual_sync:
            self.wrapped = model
            self.rep = [p for n, p in model.named_parameters() if not model.sharded(n)]
            self.shd = [p for n, p in model.named_parameters() if model.sharded(n)]
        elif world > 1 and parallel == "fsdp":
            import functools

            from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
            from torch.distributed.fsdp import MixedPrecision, ShardingStrategy
            from torch.distributed.fsdp.wrap import transformer_auto_wrap_policy
            self.wrapped = FSDP(model, sharding_strategy=ShardingStrategy.FULL_SHARD, use_orig_params=True,
                                auto_wrap_policy=functools.partial(transformer_auto_wrap_policy,
                                                                   transformer_layer_cls={Block}),
                                mixed_precision=MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                                               buffer_dtype=torch.bfloat16),
                                device_id=dev)
            self.fsdp = True
        elif world > 1 and parallel == "ddp":
            self.wrapped = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index])
        else:
            self.wrapped = model
        self.opt = torch.optim.AdamW(self.wrapped.parameters(), lr=3e-4, weight_decay=0.01, fused=True)
        g = torch.Generator().manual_seed(1000 + (0 if parallel == "tp" else rank))    # tensor parallel: one batch
        n_seq = c["mb"] * (world if (parallel == "tp" and world > 1) else 1)
        tok = torch.randint(0, vocab, (n_seq, c["seq"] + 1), generator=g).to(dev)
        self.ids, self.tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        self.loss = None

    @property
    def impl(self) -> str:
        par = {"ddp": "DDP/NCCL", "fsdp": "FSDP full-shard/NCCL",
               "tp": "Megatron-style tensor + sequence parallel, NCCL all-gather / reduce-scatter",
               "ep": "expert parallel, NCCL all_to_all_single + torch.bmm experts"}[self.parallel] \
            if (self.world > 1 or self.parallel == "ep") else "single GPU"
        return f"stock pytorch (nn.Module, cuBLAS, SDPA, autocast bf16, fused AdamW, {par})"

    @staticmethod
    def version_line() -> str:
        return "PT_TORCH_VERSION %s" % torch.__version__

    @classmethod
    def timed_steps_line(cls) -> str:
        return "PT_TIMED_STEPS " + ",".join(cls.TIMED_STEPS)

    def step(self):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.wrapped(self.ids, self.tgt)
        loss.backward()
        if self.manual_sync:
            self._sync_and_clip(1.0)
        elif self.fsdp:
            self.wrapped.clip_grad_norm_(1.0)
        else:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.loss = loss
        return loss

    def _sync_and_clip(self, max_norm: float) -> None:
        """Replicated parameters: one flat all-reduce of their gradients; clip by the norm over ALL parameters
        (replicated ones counted once, sharded ones summed over the ranks)."""
        grads = [p.grad for p in self.rep if p.grad is not None]
        flat = torch._utils._flatten_dense_tensors(grads)
        dist.all_reduce(flat)
        for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
            g.copy_(f)
        every = [p.grad for p in self.rep + self.shd if p.grad is not None]
        if self.grad_div != 1.0:
            torch._foreach_div_(every, self.grad_div)
        sq = torch.stack([torch.stack([g.float().pow(2).sum() for g in grads]).sum(),
                          torch.stack([p.grad.float().pow(2).sum() for p in self.shd if p.grad is not None]).sum()])
        local = sq[1:2].clone()
        dist.all_reduce(local)
        norm = (sq[0] + local[0]).sqrt()
        torch._foreach_mul_(every, torch.clamp(max_norm / (norm + 1e-6), max=1.0))

    def timed_block(self, steps: int) -> float:
        """Device time (ms, CUDA events on the launching stream) of ``steps`` optimizer steps."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            self.step()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    def release(self) -> None:
        self.wrapped = self.model = self.opt = None
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-small", choices=sorted(PRESETS))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--parallel", default="ddp", choices=["ddp", "fsdp", "tp", "ep"])
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    arm = TorchArm(args.model, dev, world, rank, args.parallel)
    c = arm.cfg
    for _ in range(max(args.warmup, 3)):
        arm.step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([arm.timed_block(args.steps)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    toks = c["mb"] * c["seq"] * world * args.steps
    if rank == 0:
        print(arm.version_line())
        print(arm.timed_steps_line())
        print(json.dumps({"impl": arm.impl,
                          "metric": "train tokens/sec (box, max over ranks)", "value": toks / (ms / 1e3),
                          "ms_per_step": ms / args.steps, "n_gpus": world, "steps": args.steps,
                          "config": {"model": args.model, "micro_batch_per_gpu": c["mb"], "seq_len": c["seq"]},
                          "final_loss": float(arm.loss)}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
