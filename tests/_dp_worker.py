"""Worker for the multi-GPU data-parallel test (launched by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build(dev, group, impl, graph, **dp_kw):
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.data_parallel import FusedDataParallel, NcclDataParallel
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = GPTConfig.preset("gpt-tiny")
    tape = TensorTape(grad_dtype=None)
    tape.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
    model = GPT(cfg, tape, device=dev, seed=3, group=group)
    dp = FusedDataParallel(model.arena, group, dev, **dp_kw) if impl == "fused" else \
        NcclDataParallel(model.arena, group, dev)
    eng = TrainEngine(model, 2, 128, OptimConfig(lr=1e-3, grad_clip=1.0), use_cuda_graph=graph, dp=dp)
    return cfg, model, eng


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from frankentorch_b200.ops import kernels as K
    results = {}
    # several small buckets (started under the backward pass) and, as a cross-check, one big bucket
    # launched after it; bf16 on the wire except for the fp32 run that is held against NCCL tightly
    small = dict(bucket_elems=40_000)
    runs = (("nccl", False, {}), ("fused", False, small), ("fused", True, small),
            ("fused1", True, dict(bucket_elems=1 << 40, overlap=False)),
            ("fused32", True, dict(bucket_elems=40_000, wire="fp32")),
            ("fused_now", True, dict(bucket_elems=40_000, defer_update=False)),
            ("fused_nvls", True, small))
    nvls_used = False
    for impl, graph, kw in runs:
        # the parameter all-gather through NVSwitch multimem stores only in the run that names it
        os.environ["FT_DP_NVLS"] = "1" if impl == "fused_nvls" else "0"
        cfg, model, eng = build(dev, dist.group.WORLD, "fused" if impl.startswith("fused") else impl, graph, **kw)
        g = torch.Generator().manual_seed(100 + rank)          # different data per rank
        losses = []
        tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
        ids, tgt = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
        for _ in range(6):
            losses.append(eng.step(ids, tgt))
        eng.sync_parameters()
        K.check_status()
        if impl.startswith("fused"):
            assert eng.dp.step_ok()
            assert eng.dp.nvls_params == (impl == "fused_nvls" and eng.dp.nvls_params)
            nvls_used = nvls_used or eng.dp.nvls_params
            if impl == "fused":
                assert len(eng.dp.buckets) > 3 and eng.dp.launch_order[0] == len(eng.dp.buckets) - 1
        params = model.arena.params.float().clone()
        # every rank must hold identical parameters after the all-gather
        ref = params.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, params), f"{impl}: rank {rank} parameters differ from rank 0"
        results[(impl, graph)] = (params, losses)
        dist.barrier()
    base = results[("nccl", False)][0]
    for key in (("fused", False), ("fused", True), ("fused1", True), ("fused32", True)):
        diff = (results[key][0] - base).abs().max().item()
        assert diff < 2e-2, f"{key}: params differ from the NCCL path by {diff}"
    # fp32 on the wire differs from the NCCL all-reduce only by summation order
    d32 = (results[("fused32", True)][0] - base).abs().max().item()
    assert d32 <= (results[("fused", True)][0] - base).abs().max().item() + 1e-6, d32
    # eager and graph replays of the fused path are bit-identical (fixed rank-order reduction), and so
    # are the deferred (under the next forward pass) and the immediate update
    assert torch.equal(results[("fused", False)][0], results[("fused", True)][0])
    assert torch.equal(results[("fused_now", True)][0], results[("fused", True)][0])
    assert results[("fused_now", True)][1] == results[("fused", True)][1]
    # the multimem broadcast moves the same bits as the peer stores
    assert torch.equal(results[("fused_nvls", True)][0], results[("fused", True)][0])
    assert results[("fused_nvls", True)][1] == results[("fused", True)][1]
    assert results[("fused", True)][1][-1] < results[("fused", True)][1][0]
    if rank == 0:
        print("DP_WORKER_OK", world, "nvls_params" if nvls_used else "peer_stores_only", results[("fused", True)][1])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
