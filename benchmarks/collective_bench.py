"""Collective-fused kernels against the library baseline (NCCL collective + cuBLAS GEMM).

Launch one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29700 benchmarks/collective_bench.py [--iters 10]

Shapes are the per-layer collectives of the tensor-parallel 1.3B, ZeRO-3 GPT-2-medium and
expert-parallel configurations.  Times are CUDA events on the launching stream, max over ranks,
with an L2 flush between iterations.  The roofline of a fused op is the slower of
FLOPs / measured GEMM peak and NVLink bytes / 770 GB/s (measured peer copy per direction).
"""
import argparse
import contextlib
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

LINK_GBS = 770.0


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            j = json.load(f)
        return float(j.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 1590.0, "fallback"


def timeit(fn, iters, warm, flush):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t) * 1e3   # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--comm-ctas", type=int, default=0, help="0 = the launcher's default")
    ap.add_argument("--nvls-ctas", type=int, default=148)
    ap.add_argument("--gathers-only", action="store_true", help="only the all-gather -> GEMM rows")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.fused_gemm import FusedCollectives, SymmTensor
    from frankentorch_b200.parallel.moe import ExpertParallel

    from kernel_bench import Clocks
    clk = Clocks() if rank == 0 else contextlib.nullcontext()
    clk.__enter__()
    peak, src = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = dist.group.WORLD
    bf = lambda *s: (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)
    rows = []

    def report(name, t_fused, t_base, flops, wire_bytes):
        roof = max(flops / (peak * 1e12), wire_bytes / (LINK_GBS * 1e9)) * 1e6
        rows.append(dict(op=name, fused_us=round(t_fused, 1), nccl_cublas_us=round(t_base, 1),
                         speedup=round(t_base / t_fused, 2), roofline_us=round(roof, 1),
                         frac_of_roofline=round(roof / t_fused, 3)))

    ms = 8192
    m = ms * world
    fc = FusedCollectives(g, dev, max_inbox_elems=world * ms * 2048, comm_ctas=args.comm_ctas)

    # ---- K12: all-gather(x) -> GEMM (column-parallel fc1 slice of the 1.3B model)
    d, n = 2048, 8192 // 8
    xs = SymmTensor.alloc((ms, d), torch.bfloat16, g, dev)
    xs.t.copy_(bf(ms, d))
    x_full = torch.empty((m, d), dtype=torch.bfloat16, device=dev)
    w = bf(n, d)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    t_f = timeit(lambda: fc.allgather_a_gemm(xs, w, x_full, out=out), args.iters, args.warmup, flush)
    K.check_status()

    def base_ag():
        dist.all_gather_into_tensor(x_full, xs.t)
        torch.matmul(x_full, w.t(), out=out)
    t_b = timeit(base_ag, args.iters, args.warmup, flush)
    report(f"allgather->gemm  x[{ms}x{d}]*{world} @ W[{n}x{d}]", t_f, t_b, 2.0 * m * n * d,
           (world - 1) * ms * d * 2)
    # push form: two alternating symmetric staging buffers, the shards delivered by their owners, through
    # the copy engines (deliveries queued on a second stream) or by copy CTAs inside the GEMM kernel
    stg = fc.staging((m, d))
    turn = [0]

    def push_ag():
        turn[0] ^= 1
        fc.allgather_a_gemm(xs, w, stg[turn[0]], out=out)
    want = torch.matmul(x_full, w.t())
    for transport, label in (("ew", "push, epilogue warps"), ("ce", "push, copy engines"), ("sm", "push, copy CTAs")):
        fc.transport = transport
        t_p = timeit(push_ag, args.iters, args.warmup, flush)
        K.check_status()
        assert torch.equal(stg[turn[0]].t, x_full), "push gather staged other rows than the NCCL all-gather"
        assert float((out.float() - want.float()).abs().max()) <= 2e-2 * float(want.float().abs().max())
        report(f"allgather->gemm ({label})  x[{ms}x{d}]*{world} @ W[{n}x{d}]", t_p, t_b, 2.0 * m * n * d,
               (world - 1) * ms * d * 2)
    del stg

    if not args.gathers_only:
        # ---- K13: GEMM -> reduce-scatter (row-parallel fc2 slice)
        kk, n2 = 8192 // 8, 2048
        a = bf(m, kk)
        w2 = bf(n2, kk)
        shard = torch.empty((ms, n2), dtype=torch.bfloat16, device=dev)
        full = torch.empty((m, n2), dtype=torch.bfloat16, device=dev)
        t_f = timeit(lambda: fc.gemm_reduce_scatter(a, w2, shard), args.iters, args.warmup, flush)
        K.check_status()

        def base_rs():
            torch.matmul(a, w2.t(), out=full)
            dist.reduce_scatter_tensor(shard, full)
        t_b = timeit(base_rs, args.iters, args.warmup, flush)
        report(f"gemm->reduce-scatter  A[{m}x{kk}] @ W[{n2}x{kk}]", t_f, t_b, 2.0 * m * n2 * kk,
               (world - 1) * ms * n2 * 2)

    # ---- K11: all-gather(W shards) -> GEMM (ZeRO-3 qkv projection of GPT-2 medium)
    d3, n3 = 1024, 3072
    ws = SymmTensor.alloc((n3 // world, d3), torch.bfloat16, g, dev)
    ws.t.copy_(bf(n3 // world, d3))
    w_full = torch.empty((n3, d3), dtype=torch.bfloat16, device=dev)
    x3 = bf(8192, d3)
    out3 = torch.empty((8192, n3), dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    t_f = timeit(lambda: fc.allgather_b_gemm(x3, ws, w_full, out=out3), args.iters, args.warmup, flush)
    K.check_status()

    def base_agw():
        dist.all_gather_into_tensor(w_full, ws.t)
        torch.matmul(x3, w_full.t(), out=out3)
    t_b = timeit(base_agw, args.iters, args.warmup, flush)
    report(f"allgather(W)->gemm  x[8192x{d3}] @ W[{n3}x{d3}]", t_f, t_b, 2.0 * 8192 * n3 * d3,
           (world - 1) * (n3 // world) * d3 * 2)
    wstg = fc.staging((n3, d3))

    def push_agw():
        turn[0] ^= 1
        fc.allgather_b_gemm(x3, ws, wstg[turn[0]], out=out3)
    for transport, label in (("ew", "push, epilogue warps"), ("ce", "push, copy engines"), ("sm", "push, copy CTAs")):
        fc.transport = transport
        t_p = timeit(push_agw, args.iters, args.warmup, flush)
        K.check_status()
        assert torch.equal(wstg[turn[0]].t, w_full), "push gather staged other weights than the NCCL all-gather"
        report(f"allgather(W)->gemm ({label})  x[8192x{d3}] @ W[{n3}x{d3}]", t_p, t_b, 2.0 * 8192 * n3 * d3,
               (world - 1) * (n3 // world) * d3 * 2)

    # ---- K14 / K16: MoE dispatch and combine (8 experts, top-2, capacity 1.25, d = 1024)
    T, dm, E = 8192, 1024, 8
    if E % world == 0 and not args.gathers_only:
        ep = ExpertParallel(g, dev, tokens=T, d_model=dm, n_experts=E)
        bufs = ep.new_layer_buffers()
        xt = bf(T, dm)
        logits = torch.randn(T, 128, device=dev)
        probs, idx, gate, slot, counts = ep.route(logits)
        t_f = timeit(lambda: ep.dispatch(xt, idx, slot, counts, bufs.recv_x, bufs), args.iters, args.warmup, flush)
        K.check_status()
        sent = int((slot >= 0).sum())
        remote = sent * (world - 1) / world
        send = torch.empty((world * ep.e_local * ep.capacity, dm), dtype=torch.bfloat16, device=dev)
        recv = torch.empty_like(send)
        order = torch.argsort(idx.reshape(-1), stable=True)

        def base_a2a():
            send[: order.numel()] = xt.repeat_interleave(2, dim=0)[order]      # permute, then exchange
            dist.all_to_all_single(recv, send)
        t_b = timeit(base_a2a, args.iters, args.warmup, flush)
        report(f"moe dispatch  T={T} d={dm} top-2 cap={ep.capacity}", t_f, t_b, 0.0, remote * dm * 2)
        t_f = timeit(lambda: ep.combine(bufs.recv_x, idx, slot, counts, gate), args.iters, args.warmup, flush)
        K.check_status()

        def base_comb():
            dist.all_to_all_single(send, recv)
            y2 = send[: order.numel()][torch.argsort(order)].view(T, 2, dm)
            return (y2 * gate.unsqueeze(-1)).sum(1)
        t_b = timeit(base_comb, args.iters, args.warmup, flush)
        report(f"moe combine  T={T} d={dm}", t_f, t_b, 0.0, remote * dm * 2)

    # ---- NVLS: multimem.st all-gather and multimem.ld_reduce all-reduce against NCCL
    try:
        if args.gathers_only:
            raise RuntimeError('skipped (--gathers-only)')
        from frankentorch_b200.parallel.nvls import MulticastBuffer, NvlsCollectives, NvlsUnavailable
        nel = 8 << 20                                            # 32 MiB of fp32 per rank
        mb = MulticastBuffer(world * nel * 4 + nel * 4, None, dev)
        coll = NvlsCollectives(mb, n_ctas=args.nvls_ctas)
        srcv = torch.randn(nel, device=dev)
        gathered = torch.empty(world * nel, device=dev)
        t_f = timeit(lambda: coll.all_gather(srcv, 0), args.iters, args.warmup, flush)
        t_b = timeit(lambda: dist.all_gather_into_tensor(gathered, srcv), args.iters, args.warmup, flush)
        K.check_status()
        assert torch.equal(mb.tensor(torch.float32, world * nel, 0), gathered)
        report(f"nvls all-gather  {nel * 4 >> 20} MiB per rank (multimem.st)", t_f, t_b, 0.0, (world - 1) * nel * 4)
        red = torch.randn(nel, device=dev)
        off = world * nel * 4
        t_f = timeit(lambda: coll.all_reduce_(off, nel, torch.float32), args.iters, args.warmup, flush)
        t_b = timeit(lambda: dist.all_reduce(red), args.iters, args.warmup, flush)
        K.check_status()
        report(f"nvls all-reduce  {nel * 4 >> 20} MiB fp32 (multimem.ld_reduce + st)", t_f, t_b, 0.0,
               2 * (world - 1) * nel * 4 // world)
    except Exception as e:          # no multicast object on this system: say so, keep the other rows
        if rank == 0:
            print(json.dumps({"nvls": "unavailable", "why": repr(e)[:200]}))

    clk.__exit__(None, None, None)
    if rank == 0:
        print(json.dumps({"world": world, "gemm_peak_tflops": peak, "peak_source": src, "link_gbs": LINK_GBS,
                          "iters": args.iters, "results": rows}, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
