#!/usr/bin/env python
"""Per-operator benchmark on the reference's own op list, through the public session API.

    python benchmarks/ops_bench.py                 # CPU reference path (f64 session)
    python benchmarks/ops_bench.py --device cuda   # sm_100a backend (bf16, hardened mode)

The list, the sizes and the method (10 warm-ups, 30 runs, p50) are those of the reference's
incumbent generator (scripts/pytorch_baseline.py:12-46 -> benchmarks/pytorch_baseline.json) and of
its own published profile (docs/planning/PROFILING-RESULTS.md:27-63).  One JSON line per
operator: our p50 in microseconds and ``vs_baseline`` = published p50 of the reference / ours
(above 1: faster than the reference's published number; hardware differs, see ``note``), plus the
same ratio against the published single-thread PyTorch CPU figure.
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

# published p50 (us): (reference's PyTorch CPU incumbent, FrankenTorch itself or None)
PUBLISHED = {
    "matmul_64": (9.02, 16.5), "matmul_128": (49.05, 107.7), "matmul_256": (365.15, 810.0),
    "matmul_512": (2908.39, 6191.0), "matmul_1024": (24022.43, 49360.0),
    "bmm_b8_128": (390.33, 1280.0), "bmm_b16_128": (845.18, 2584.0), "bmm_b32_128": (23124.26, 5676.0),
    "sum_1e3": (2.77, None), "sum_1e4": (3.13, None), "sum_1e5": (7.39, None), "sum_1e6": (48.79, None),
    "softmax_32x128": (6.98, None), "softmax_32x512": (20.63, None), "softmax_32x2048": (81.73, None),
    "softmax_32x8192": (292.73, None),
    "relu_1e6": (91.19, 2772.0), "exp_1e6": (1182.49, 2925.0), "add_1e6": (110.34, 908.0),
    "matmul_fwd_bwd_64": (140.21, None), "matmul_fwd_bwd_128": (387.75, None), "matmul_fwd_bwd_256": (1819.59, None),
    "linear_32x512_256": (113.93, 1207.0), "linear_32x512_512": (223.5, 2615.0),
    "linear_32x512_1024": (440.56, 5404.0), "linear_32x512_2048": (885.89, 10382.0),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--runs", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=10)
    a = ap.parse_args()
    import torch

    from frankentorch_b200.session import FrankenTorchSession
    cuda = a.device == "cuda"
    s = FrankenTorchSession("hardened" if cuda else "strict", device=a.device, ledger_dispatch=False)

    def rnd(*shape, rg=False):
        return s.tensor_variable_from_storage(torch.randn(*shape).to(a.device, torch.bfloat16 if cuda else torch.float64), rg)

    def sync():
        if cuda:
            torch.cuda.synchronize()

    def timed(fn):
        boundary = s.autograd_graph_len()
        for _ in range(a.warmup):
            fn()
            s.truncate_autograd_graph(boundary)
        ts = []
        for _ in range(a.runs):
            sync()
            t0 = time.perf_counter()
            fn()
            sync()
            ts.append((time.perf_counter() - t0) * 1e6)
            s.truncate_autograd_graph(boundary)
        return statistics.median(ts)

    cases = {}
    for n in (64, 128, 256, 512, 1024):
        x, y = rnd(n, n), rnd(n, n)
        cases[f"matmul_{n}"] = lambda x=x, y=y: s.tensor_matmul(x, y)
    for b in (8, 16, 32):
        x, y = rnd(b, 128, 128), rnd(b, 128, 128)
        cases[f"bmm_b{b}_128"] = lambda x=x, y=y: s.tensor_bmm(x, y)
    for e in (3, 4, 5, 6):
        x = rnd(10 ** e)
        cases[f"sum_1e{e}"] = lambda x=x: s.tensor_sum(x)
    for c in (128, 512, 2048, 8192):
        x = rnd(32, c)
        cases[f"softmax_32x{c}"] = lambda x=x: s.tensor_softmax(x, dim=-1)
    x6, y6 = rnd(10 ** 6), rnd(10 ** 6)
    cases["relu_1e6"] = lambda: s.tensor_relu(x6)
    cases["exp_1e6"] = lambda: s.tensor_exp(x6)
    cases["add_1e6"] = lambda: s.tensor_add(x6, y6)
    for n in (64, 128, 256):
        x, y = rnd(n, n, rg=True), rnd(n, n, rg=True)

        def fb(x=x, y=y):
            out = s.tensor_sum(s.tensor_matmul(x, y))
            s.tensor_backward(out)
            s.tensor_zero_grads([x, y])
        cases[f"matmul_fwd_bwd_{n}"] = fb
    xin = rnd(32, 512)
    for o in (256, 512, 1024, 2048):
        w, b = rnd(o, 512), rnd(o)
        cases[f"linear_32x512_{o}"] = lambda w=w, b=b: s.tensor_linear(xin, w, b)

    note = ("published figures: x86-64 CPU, one thread (benchmarks/pytorch_baseline.json:2-8, "
            "docs/planning/PROFILING-RESULTS.md:27-63); ours: " +
            (f"one B200 ({torch.cuda.get_device_name(0)}), bf16, host-timed per call with a device synchronisation"
             if cuda else f"this machine's CPU, {torch.get_num_threads()} torch thread(s), f64 session"))
    for name, fn in cases.items():
        us = timed(fn)
        pt, ft = PUBLISHED[name]
        print(json.dumps({"op": name, "device": a.device, "p50_us": round(us, 2), "runs": a.runs,
                          "published_frankentorch_p50_us": ft, "published_pytorch_cpu_p50_us": pt,
                          "vs_baseline": None if ft is None else round(ft / us, 3),
                          "vs_published_pytorch_cpu": round(pt / us, 3), "note": note}), flush=True)
    if cuda:
        from frankentorch_b200.ops import kernels as K
        K.check_status()


if __name__ == "__main__":
    main()
