#!/usr/bin/env python
"""Micro-benchmarks of single kernels (CUDA-event timing, L2 flushed between iterations).

    python benchmarks/kernel_bench.py gemm --m 8192 --n 2304 --k 768 [--mode fwd|dgrad|wgrad]
    python benchmarks/kernel_bench.py attn --b 8 --s 1024 --h 12 --hd 64 [--bwd]
    python benchmarks/kernel_bench.py sweep            # the shapes of the five training configs
    python benchmarks/kernel_bench.py rows --case all  # row / elementwise / optimizer / comm kernels (world = 1)

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


class Clocks:
    """SM clock and throttle reasons sampled with NVML while the cases run (read-only queries)."""

    def __init__(self):
        self.rows, self.stop_flag, self.thread = [], None, None

    def __enter__(self):
        try:
            import threading

            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        self.rows.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), int(reasons(h))))
                    except Exception:
                        pass
                    self.stop_flag.wait(0.02)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *exc):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            if self.rows:
                import statistics
                bits = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}
                seen = 0
                for _, r in self.rows:
                    seen |= r
                out = {"sm_mhz": statistics.median(r[0] for r in self.rows), "sm_max_mhz": self.mx,
                       "reasons": sorted(n for b, n in bits.items() if seen & b), "samples": len(self.rows)}
        print(json.dumps({"clocks": out}), flush=True)
        return False


def _row_cases(rows, cols):
    """name -> (callable, algorithmic bytes moved per call).  Inputs exceed L2 only for the big cases; the
    timing loop flushes L2 between iterations either way."""
    f32 = lambda *sh: torch.randn(*sh, device="cuda")
    x, dy = bf(rows, cols, scale=1.0), bf(rows, cols, scale=1.0)
    g, b = bf(cols, scale=1.0), bf(cols)
    n = rows * cols
    y, mean, rstd, _ = ops.layernorm_fwd(x, g, b)
    yr, rr = ops.rmsnorm_fwd(x, g)
    sm = ops.softmax_rows(x)
    V, d, T = 50304, cols, rows
    ids = torch.randint(0, 50257, (T,), device="cuda")
    wte, wpe = bf(V, d), bf(1024, d)
    dwte, dwpe = torch.zeros(V, d, device="cuda"), torch.zeros(1024, d, device="cuda")
    N = 32 << 20
    master, gr, m, v = f32(N), f32(N), torch.zeros(N, device="cuda"), torch.zeros(N, device="cuda")
    shadow = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    hyper = torch.tensor([1e-3, 0.1, 0.001, 1.0], device="cuda")
    ss, nrm = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    xf = f32(rows, cols)
    logits = bf(rows, V, scale=1.0)
    cases = {
        "cross_entropy": (lambda: ops.cross_entropy_fwd_bwd(logits, ids, 50257, 1.0 / rows, inplace=True), 4 * rows * V),
        "layernorm_fwd": (lambda: ops.layernorm_fwd(x, g, b), 4 * n),
        "layernorm_bwd": (lambda: ops.layernorm_bwd(dy, x, g, mean, rstd, dx_add=dy), 8 * n),
        "rmsnorm_fwd": (lambda: ops.rmsnorm_fwd(x, g), 4 * n),
        "rmsnorm_bwd": (lambda: ops.rmsnorm_bwd(dy, x, g, rr), 6 * n + 4 * n),
        "softmax_rows": (lambda: ops.softmax_rows(x), 4 * n),
        "softmax_bwd": (lambda: ops.softmax_bwd(sm, dy), 6 * n),
        "gelu_fwd": (lambda: ops.gelu_fwd(x), 4 * n),
        "gelu_bwd": (lambda: ops.gelu_bwd(x, dy), 6 * n),
        "add": (lambda: ops.add(x, dy), 6 * n),
        "dropout": (lambda: ops.dropout(x, 0.1, 7), 4 * n),
        "cast_f32_bf16": (lambda: ops.cast_f32_to_bf16(xf), 6 * n),
        "colsum": (lambda: ops.colsum(dy), 2 * n),
        "embedding_fwd": (lambda: ops.embedding_fwd(ids, wte, wpe, 1024), 4 * T * d + 2 * T * d),
        "embedding_bwd": (lambda: ops.embedding_bwd(ids, dy, dwte, dwpe, 1024), 2 * T * d + 8 * T * d),
        "embedding_bwd_sorted": (lambda: ops.embedding_bwd(ids, dy, dwte, dwpe, 1024, sorted_form=True),
                                 2 * T * d + 8 * T * d),
        "embedding_bwd_repeats": (lambda: ops.embedding_bwd(ids % 50, dy, dwte, dwpe, 1024), 2 * T * d + 8 * T * d),
        "adamw_dev": (lambda: ops.adamw_dev(master, shadow, gr, m, v, hyper, beta1=0.9, beta2=0.999, eps=1e-8,
                                            weight_decay=0.01), 30 * N),
        "sumsq": (lambda: ops.sumsq(gr, out=ss), 4 * N),
        "clip_scale": (lambda: ops.clip_scale(ss, 1.0, hyper, nrm), 16),
    }
    return cases


def bench_rows(case, rows, cols, iters, warm):
    pk = peaks()
    cases = _row_cases(rows, cols)
    names = list(cases) if case == "all" else [case]
    for name in names:
        fn, nbytes = cases[name]
        t = timeit(fn, iters, warm)
        gbs = nbytes / t / 1e6
        print(f"{name:14s} rows {rows} cols {cols}: {t*1e3:8.1f} us {gbs:8.1f} GB/s "
              f"({gbs / pk['hbm_gbs']:.2f} of {pk['src']} copy bandwidth)", flush=True)
    ops.check_status()


def bench_dp_world1(n_params, iters, warm):
    """The bucketed data-parallel kernels with this GPU as the only rank (push, reduce, norm, update)."""
    import types

    from frankentorch_b200.models.gpt import ParamArena
    from frankentorch_b200.parallel.data_parallel import FusedDataParallel
    pk = peaks()
    dev = torch.device("cuda", 0)
    arena = ParamArena([("w", (n_params,))], dev, peer_visible=True)
    arena.master.normal_()
    arena.grads.normal_()
    dp = FusedDataParallel(arena, None, dev, bucket_elems=n_params // 4, overlap=False,
                           defer_update=False)
    opt = types.SimpleNamespace(beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, grad_clip=1.0)
    hyper = torch.tensor([1e-3, 0.1, 0.001, 1.0], device="cuda")
    nrm, ss = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")

    def step():
        dp.begin_step()
        dp.reduce_and_update(arena, hyper, opt, ss, nrm, None)
    t = timeit(step, iters, warm)
    nbytes = n_params * (4 + 2 + 2 + 4 + 4 + 24 + 2)       # push r/w, reduce r/w, update r/w master+m+v, params
    print(f"dp_world1 {n_params} params: {t*1e3:8.1f} us {nbytes / t / 1e6:8.1f} GB/s "
          f"({nbytes / t / 1e6 / pk['hbm_gbs']:.2f} of {pk['src']} copy bandwidth)", flush=True)
    ops.check_status()


def bench_group(tokens, d, iters, warm):
    """The four weight gradients of a transformer block (qkv, proj, fc1, fc2) as one grouped launch, against
    the same four as separate GEMMs (split-K where the planner wants it) and against cuBLAS."""
    pk = peaks()
    shapes = ((3 * d, d), (d, d), (4 * d, d), (d, 4 * d))
    dys = [bf(tokens, m) for m, n in shapes]
    xs = [bf(tokens, n) for m, n in shapes]
    outs = [torch.zeros(m, n, device="cuda") for m, n in shapes]
    flops = sum(2.0 * tokens * m * n for m, n in shapes)
    t_g = timeit(lambda: ops.gemm_grouped([(dy, x, o, False) for dy, x, o in zip(dys, xs, outs)]), iters, warm)
    t_s = timeit(lambda: [ops.gemm(dy, x, a_mn=True, b_mn=True, out=o) for dy, x, o in zip(dys, xs, outs)], iters, warm)
    t_c = timeit(lambda: [torch.matmul(dy.t(), x) for dy, x in zip(dys, xs)], iters, warm)
    print(f"grouped wgrad T{tokens} d{d}: {t_g*1e3:8.1f} us {flops/t_g/1e9:7.1f} TF/s ({flops/t_g/1e9/pk['bf16_tflops']:.2f} of "
          f"{pk['src']} peak) | four separate launches {t_s*1e3:8.1f} us | cuBLAS x4 (bf16 out) {t_c*1e3:8.1f} us", flush=True)
    ops.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "sweep", "rows", "dp", "group"])
    ap.add_argument("--case", default="all")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=768)
    ap.add_argument("--params", type=int, default=32 << 20)
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
    with Clocks():
        _dispatch(a)


def _dispatch(a):
    if a.what == "gemm":
        bench_gemm(a.m, a.n, a.k, a.mode, a.iters, a.warmup, not a.no_ref, a.force_bn)
    elif a.what == "attn":
        bench_attn(a.b, a.s, a.h, a.hd, a.bwd, a.iters, a.warmup, not a.no_ref)
    elif a.what == "rows":
        bench_rows(a.case, a.rows, a.cols, a.iters, a.warmup)
    elif a.what == "dp":
        bench_dp_world1(a.params, a.iters, a.warmup)
    elif a.what == "group":
        bench_group(a.m, a.k, a.iters, a.warmup)
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
