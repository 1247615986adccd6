"""Worker for the multicast (NVLS) collectives test (launched by torch.distributed.run, one rank
per GPU): multimem all-gather against ``dist.all_gather`` (bit-exact), multimem all-reduce in
fp32 and bf16 against an fp32 sum (tolerance), identical on every rank and across two runs."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.nvls import MulticastBuffer, NvlsCollectives
    n = 1 << 20                                   # elements per rank
    buf = MulticastBuffer(world * n * 4 + n * 4, None, dev)
    if not buf.has_multicast:
        if rank == 0:
            print("NVLS_WORKER_SKIP no multicast address on this system")
        dist.barrier()
        dist.destroy_process_group()
        return
    coll = NvlsCollectives(buf)
    g = torch.Generator().manual_seed(100 + rank)
    # all-gather: bit-exact against NCCL
    for it in range(3):
        src = torch.randn(n, generator=g).to(dev)
        got = coll.all_gather(src, 0).clone()
        want = [torch.empty_like(src) for _ in range(world)]
        dist.all_gather(want, src)
        assert torch.equal(got, torch.stack(want)), ("all_gather", it)
    # all-reduce, fp32 and bf16: against an fp32 sum; the same bits on every rank and on a second run
    off = world * n * 4
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        numel = n if dtype == torch.float32 else 2 * n
        x = torch.randn(numel, generator=g).to(dev).to(dtype)
        ref = x.float().clone()
        dist.all_reduce(ref)
        view = buf.tensor(dtype, numel, off)
        runs = []
        for _ in range(2):
            view.copy_(x)
            out = coll.all_reduce_(off, numel, dtype).clone()
            runs.append(out)
        K.check_status()
        err = float((runs[0].float() - ref).abs().max() / ref.abs().max())
        assert err < tol, (str(dtype), err)
        assert torch.equal(runs[0], runs[1]), "all_reduce differs between two runs"
        everyone = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(everyone, runs[0])
        assert all(torch.equal(everyone[0], e) for e in everyone), "ranks disagree on the reduced values"
    # timing (CUDA events, max over ranks), for the log only
    src = torch.randn(n, device=dev)
    for fn, name, nbytes in ((lambda: coll.all_gather(src, 0), "all_gather", n * 4 * world),
                             (lambda: coll.all_reduce_(off, n, torch.float32), "all_reduce_f32", n * 4)):
        for _ in range(5):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier()
        a.record()
        for _ in range(20):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 20], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"nvls {name}: {float(t) * 1e3:.1f} us for {nbytes >> 20} MiB result per rank, world {world}")
    K.check_status()
    dist.barrier()
    if rank == 0:
        print("NVLS_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
