"""Worker for the collective-fused GEMM test (launched by torch.distributed.run, one rank per GPU).

Every rank regenerates all ranks' inputs from seeds, so the fp32 reference of each fused op is
computed locally with plain PyTorch and no communication.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rnd(shape, seed, dev, scale=0.25):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(dev)


def close(got, ref, what, rank, tol=2e-2):
    err = (got.float() - ref).abs().max().item()
    lim = tol * max(1.0, ref.abs().max().item())
    if not err <= lim:
        raise AssertionError(f"rank {rank} {what}: max err {err} > {lim}")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.fused_gemm import FusedCollectives, SymmTensor

    ms, kdim, n = 256, 384, 1024           # rows per rank, reduction, output columns
    m = ms * world
    fc = FusedCollectives(dist.group.WORLD, dev, max_inbox_elems=world * ms * n, comm_ctas=4)
    x_sh = [SymmTensor.alloc((ms, kdim), torch.bfloat16, dist.group.WORLD, dev) for _ in range(2)]
    w_sh = SymmTensor.alloc((n // world, kdim), torch.bfloat16, dist.group.WORLD, dev)
    x_full = torch.empty((m, kdim), dtype=torch.bfloat16, device=dev)
    w_full = torch.empty((n, kdim), dtype=torch.bfloat16, device=dev)
    x_stage = fc.staging((m, kdim))        # push form: peers store into these
    w_stage = fc.staging((n, kdim))

    for it in range(3):                    # several epochs over the same flag arrays
        base = 1000 * it
        # push form: one transport per epoch (epilogue warps of every CTA, copy CTAs, copy engines)
        fc.transport = ("ew", "sm", "ce")[it]
        # ---- all-gather(A) -> GEMM, ranks hold different weights (column-parallel)
        xs = [rnd((ms, kdim), base + r, dev) for r in range(world)]
        w = rnd((n, kdim), base + 100 + rank, dev)
        bias = rnd((n,), base + 150 + rank, dev)
        sh = x_sh[it & 1]
        sh.t.copy_(xs[rank])
        out = fc.allgather_a_gemm(sh, w, x_full, bias=bias)
        K.check_status()
        ref = torch.cat(xs).float() @ w.float().t() + bias.float()
        close(out, ref, f"gather-A epoch {it}", rank)
        assert torch.equal(x_full, torch.cat(xs)), "gathered activations differ"
        # push form of the same op (the owners store their shards into every staging buffer)
        out_p = fc.allgather_a_gemm(sh, w, x_stage[it & 1], bias=bias)
        K.check_status()
        assert torch.equal(out_p, out), "push and pull gathers give different products"
        assert torch.equal(x_stage[it & 1].t, torch.cat(xs)), "pushed activations differ"

        # ---- all-gather(B) -> GEMM forward and dgrad, weight sharded by output rows
        ws = [rnd((n // world, kdim), base + 200 + r, dev) for r in range(world)]
        dist.barrier()                     # peers finished reading the previous weights
        w_sh.t.copy_(ws[rank])
        torch.cuda.synchronize()
        dist.barrier()                     # the weight handshake is the caller's (optimizer step)
        x = rnd((512, kdim), base + 300 + rank, dev)
        out = fc.allgather_b_gemm(x, w_sh, w_full)
        K.check_status()
        wf = torch.cat(ws).float()
        close(out, x.float() @ wf.t(), f"gather-B fwd epoch {it}", rank)
        dy = rnd((512, n), base + 400 + rank, dev)
        out = fc.allgather_b_gemm(dy, w_sh, w_full, dgrad=True)
        K.check_status()
        close(out, dy.float() @ wf, f"gather-B dgrad epoch {it}", rank)
        out_p = fc.allgather_b_gemm(x, w_sh, w_stage[0])
        K.check_status()
        close(out_p, x.float() @ wf.t(), f"gather-B fwd (push) epoch {it}", rank)
        assert torch.equal(w_stage[0].t, torch.cat(ws)), "pushed weights differ"
        out_p = fc.allgather_b_gemm(dy, w_sh, w_stage[1], dgrad=True)
        K.check_status()
        assert torch.equal(out_p, out), "push and pull dgrad differ"

        # ---- GEMM -> reduce-scatter with bias and residual, bf16 and fp32-accumulate outputs
        a_all = [rnd((m, kdim), base + 500 + r, dev) for r in range(world)]
        b_all = [rnd((n, kdim), base + 600 + r, dev) for r in range(world)]
        resid = rnd((ms, n), base + 700 + rank, dev)
        full = sum(a.float() @ b.float().t() for a, b in zip(a_all, b_all))
        ref = full[rank * ms:(rank + 1) * ms] + resid.float()
        out = torch.empty((ms, n), dtype=torch.bfloat16, device=dev)
        fc.gemm_reduce_scatter(a_all[rank], b_all[rank], out, resid=resid)
        K.check_status()
        close(out, ref, f"scatter epoch {it}", rank, tol=3e-2)
        acc = torch.ones((ms, n), dtype=torch.float32, device=dev)
        fc.gemm_reduce_scatter(a_all[rank], b_all[rank], acc, accumulate=True)
        K.check_status()
        close(acc, full[rank * ms:(rank + 1) * ms] + 1.0, f"scatter fp32 epoch {it}", rank, tol=3e-2)
        # reproducible: same inputs, same bits
        out2 = torch.empty_like(out)
        fc.gemm_reduce_scatter(a_all[rank], b_all[rank], out2, resid=resid)
        K.check_status()
        assert torch.equal(out, out2), "reduce-scatter is not bit-reproducible"

    # one copy CTA: its ring of six slots wraps (every slot is reused, phases flip) in both forms
    fc1 = FusedCollectives(dist.group.WORLD, dev, comm_ctas=1)
    fc1.transport = "sm"
    stage1 = fc1.staging((m, kdim))
    for it in range(2):
        xs = [rnd((ms, kdim), 9000 + 10 * it + r, dev) for r in range(world)]
        w = rnd((n, kdim), 9100 + it, dev)
        sh = x_sh[it & 1]
        sh.t.copy_(xs[rank])
        ref = torch.cat(xs).float() @ w.float().t()
        out = fc1.allgather_a_gemm(sh, w, x_full)
        K.check_status()
        close(out, ref, f"gather-A one copy CTA (pull) {it}", rank)
        out = fc1.allgather_a_gemm(sh, w, stage1[it & 1])
        K.check_status()
        close(out, ref, f"gather-A one copy CTA (push) {it}", rank)
        assert torch.equal(stage1[it & 1].t, torch.cat(xs)), "pushed activations differ (one copy CTA)"

    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("COMM_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
