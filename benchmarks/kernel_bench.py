#!/usr/bin/env python
"""Micro-benchmarks of single kernels (CUDA-event timing, L2 flushed between iterations).

    python benchmarks/kernel_bench.py gemm --m 8192 --n 2304 --k 768 [--mode fwd|dgrad|wgrad]
    python benchmarks/kernel_bench.py attn --b 8 --s 1024 --h 12 --hd 64 [--bwd]
    python benchmarks/kernel_bench.py sweep            # the shapes of the five training configs

Each line reports the achieved TFLOP/s (or GB/s) and the fraction of the measured peak read from
MEASURED_PEAKS.json at the repository root (fallback 1590 TFLOP/s, 6650 GB/s), next to the same
op in stock PyTorch (cuBLAS / SDPA) timed the same way.  With ``--iters 1 --no-ref`` the script
launches the kernel a minimal number of times, which is the form used under ``ncu``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from frankentorch_b200.ops import kernels as ops  # noqa: E402


def peaks():
    p = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "src": "fallback"}
    try:
        d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        p.update(bf16_tflops=float(d["bf16_tflops"]), hbm_gbs=float(d["hbm_gbs"]), src="measured")
    except Exception:
        pass
    return p


_FLUSH = None


def timeit(fn, iters, warm):
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        _FLUSH.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    return tot / max(iters, 1)


def bf(*shape, scale=0.1):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def bench_gemm(M, N, K, mode, iters, warm, ref=True, force_bn=0):
    pk = peaks()
    x, w, dy = bf(M, K), bf(N, K), bf(M, N)
    fl = 2.0 * M * N * K
    if mode == "fwd":
        ours, theirs = (lambda: ops.gemm(x, w, force_bn=force_bn)), (lambda: x @ w.t())
    elif mode == "dgrad":
        ours, theirs = (lambda: ops.gemm(dy, w, b_mn=True, force_bn=force_bn)), (lambda: dy @ w)
    else:
        out = torch.empty(N, K, dtype=torch.float32, device="cuda")
        ours = lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out=out, force_bn=force_bn)
        theirs = lambda: dy.t() @ x
    t1 = timeit(ours, iters, warm)
    line = f"gemm {mode:5s} M{M} N{N} K{K}: {t1*1e3:8.1f} us {fl/t1/1e9:7.1f} TF/s ({fl/t1/1e9/pk['bf16_tflops']:.2f} of {pk['src']} peak)"
    if ref:
        t2 = timeit(theirs, iters, warm)
        line += f" | cuBLAS {t2*1e3:8.1f} us {fl/t2/1e9:7.1f} TF/s  ratio {t2/t1:.2f}"
    print(line, flush=True)
    ops.check_status()


def bench_attn(B, S, H, hd, bwd, iters, warm, ref=True):
    import torch.nn.functional as F
    pk = peaks()
    d = H * hd
    qkv = bf(B, S, 3 * d, scale=0.5)
    q, k, v = (qkv[:, :, i * d:(i + 1) * d].view(B, S, H, hd) for i in range(3))
    o, lse = ops.attention_fwd(q, k, v)
    fl = 4.0 * B * H * S * S * hd / 2
    if not bwd:
        t1 = timeit(lambda: ops.attention_fwd(q, k, v), iters, warm)
        line = f"attn fwd B{B} S{S} H{H} hd{hd}: {t1*1e3:8.1f} us {fl/t1/1e9:6.1f} TF/s ({fl/t1/1e9/pk['bf16_tflops']:.2f} of {pk['src']} peak)"
        if ref:
            qt, kt, vt = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
            t2 = timeit(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True), iters, warm)
            line += f" | torch SDPA {t2*1e3:8.1f} us  ratio {t2/t1:.2f}"
    else:
        do = bf(B, S, H, hd)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = (dqkv[:, :, i * d:(i + 1) * d].view(B, S, H, hd) for i in range(3))
        t1 = timeit(lambda: ops.attention_bwd(q, k, v, o, lse, do, dq=dq, dk=dk, dv=dv), iters, warm)
        line = f"attn bwd B{B} S{S} H{H} hd{hd}: {t1*1e3:8.1f} us {2.5*fl/t1/1e9:6.1f} TF/s ({2.5*fl/t1/1e9/pk['bf16_tflops']:.2f} of {pk['src']} peak)"
        if ref:
            qt, kt, vt = (t.permute(0, 2, 1, 3).contiguous().requires_grad_(True) for t in (q, k, v))
            ot = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
            dot = do.permute(0, 2, 1, 3).contiguous()
            t2 = timeit(lambda: torch.autograd.grad(ot, (qt, kt, vt), dot, retain_graph=True), iters, warm)
            line += f" | torch SDPA {t2*1e3:8.1f} us  ratio {t2/t1:.2f}"
    print(line, flush=True)
    ops.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "sweep"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--mode", default="fwd", choices=["fwd", "dgrad", "wgrad"])
    ap.add_argument("--force-bn", type=int, default=0)
    ap.add_argument("--b", type=int, default=8)
    ap.add_argument("--s", type=int, default=1024)
    ap.add_argument("--h", type=int, default=12)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-ref", action="store_true")
    a = ap.parse_args()
    if a.what == "gemm":
        bench_gemm(a.m, a.n, a.k, a.mode, a.iters, a.warmup, not a.no_ref, a.force_bn)
    elif a.what == "attn":
        bench_attn(a.b, a.s, a.h, a.hd, a.bwd, a.iters, a.warmup, not a.no_ref)
    else:
        for (N, Kd) in [(2304, 768), (768, 768), (3072, 768), (768, 3072), (50304, 768),
                        (3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096), (8192, 8192)]:
            for mode in ("fwd", "dgrad", "wgrad"):
                bench_gemm(8192, N, Kd, mode, a.iters, a.warmup)
        for (B, S, H, hd) in [(8, 1024, 12, 64), (4, 2048, 16, 64), (4, 2048, 16, 128)]:
            bench_attn(B, S, H, hd, False, a.iters, a.warmup)
            bench_attn(B, S, H, hd, True, a.iters, a.warmup)


if __name__ == "__main__":
    main()
