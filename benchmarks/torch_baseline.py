#!/usr/bin/env python
"""Stock PyTorch arm of the headline benchmark: the same GPT-2 training step written with
``torch.nn`` modules, cuBLAS GEMMs, ``F.scaled_dot_product_attention`` (flash), bf16 autocast
with fp32 master weights, fused ``torch.optim.AdamW``, gradient clipping, and
``DistributedDataParallel`` (NCCL all-reduce) or ``FullyShardedDataParallel`` on more than one
GPU.  Nothing of this repository's kernels or engine is on this path.  ``bench.py`` imports
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
        model = GPT(c["n_layer"], c["d"], c["h"], c["ff"], c["seq"]).to(dev)
        self.model = model
        self.fsdp = False
        if world > 1 and parallel == "fsdp":
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
        elif world > 1:
            self.wrapped = nn.parallel.DistributedDataParallel(model, device_ids=[dev.index])
        else:
            self.wrapped = model
        self.opt = torch.optim.AdamW(self.wrapped.parameters(), lr=3e-4, weight_decay=0.01, fused=True)
        g = torch.Generator().manual_seed(1000 + rank)
        tok = torch.randint(0, VOCAB, (c["mb"], c["seq"] + 1), generator=g).to(dev)
        self.ids, self.tgt = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        self.loss = None

    @property
    def impl(self) -> str:
        par = {"ddp": "DDP/NCCL", "fsdp": "FSDP full-shard/NCCL"}[self.parallel] if self.world > 1 else "single GPU"
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
        if self.fsdp:
            self.wrapped.clip_grad_norm_(1.0)
        else:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.loss = loss
        return loss

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
    ap.add_argument("--parallel", default="ddp", choices=["ddp", "fsdp"])
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
