#!/usr/bin/env python
"""Encoder-stack inference: the GPU-resident ``EncoderGpu`` against the same stack in stock PyTorch.

    python benchmarks/encoder_bench.py --seq 1500 --d 1280 --heads 20 --layers 32

The default is the shape the reference quotes for its Metal encoder ("turbo": seq 1500, d 1280,
32 layers; crates/ft-kernel-metal/src/fused.rs:1149-1160).  Times are CUDA events around a whole
forward on resident activations (upload and download excluded), after warm-up; the stock arm runs
the same math with bf16 ``torch.nn.functional`` ops (cuBLAS + flash SDPA).
"""
import argparse
import json
import pathlib
import sys

import torch

sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))

from frankentorch_b200.models.encoder import EncoderGpu, EncoderLayerWeights, LN_EPS


def torch_stack(layers, x, heads):
    S, d = x.shape
    hd = d // heads
    F = torch.nn.functional
    for l in layers:
        n1 = F.layer_norm(x, (d,), l["ln1_g"], l["ln1_b"], LN_EPS)
        qkv = F.linear(n1, l["w_qkv"], l["b_qkv"]).view(S, 3, heads, hd).permute(1, 2, 0, 3)
        a = F.scaled_dot_product_attention(qkv[0][None], qkv[1][None], qkv[2][None])[0].transpose(0, 1).reshape(S, d)
        x1 = x + F.linear(a, l["wo"], l["bo"])
        n2 = F.layer_norm(x1, (d,), l["ln2_g"], l["ln2_b"], LN_EPS)
        x = x1 + F.linear(F.gelu(F.linear(n2, l["w1"], l["b1"]), approximate="tanh"), l["w2"], l["b2"])
    return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=1500)
    ap.add_argument("--d", type=int, default=1280)
    ap.add_argument("--heads", type=int, default=20)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--chunk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    g = torch.Generator().manual_seed(0)
    layers = [EncoderLayerWeights.random(args.d, 4 * args.d, g) for _ in range(args.layers)]
    enc = EncoderGpu(layers, args.heads, chunk=args.chunk)
    x = torch.randn(args.seq, args.d, generator=g).to("cuda", torch.bfloat16)
    tl = [{k: getattr(gl, k) for k in ("ln1_g", "ln1_b", "w_qkv", "b_qkv", "wo", "bo", "ln2_g", "ln2_b", "w1", "b1", "w2", "b2")}
          for gl in enc.layers]

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.iters

    ours = timeit(lambda: enc.forward_stack(x))
    with torch.no_grad():
        theirs = timeit(lambda: torch_stack(tl, x, args.heads))
        err = (enc.forward_stack(x).float() - torch_stack(tl, x, args.heads).float()).abs().max().item()
    flops = args.layers * (2 * args.seq * args.d * (4 * args.d + 8 * args.d) + 4 * args.seq * args.seq * args.d)
    print(json.dumps({"op": f"encoder forward seq {args.seq} d {args.d} heads {args.heads} layers {args.layers}",
                      "ours_ms": ours, "torch_bf16_ms": theirs, "speedup": theirs / ours,
                      "ours_tflops": flops / ours / 1e9, "max_abs_diff_vs_torch_bf16": err,
                      "graph_launches_per_forward": len(enc.chunks()),
                      "kernels_per_layer": enc.launches_per_layer}))


if __name__ == "__main__":
    main()
