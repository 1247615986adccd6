"""Worker for the ZeRO-3 GPT test (launched by torch.distributed.run, one rank per GPU).

Each rank also trains an unsharded copy of the same model on the global batch; the mean of the
ranks' local losses must follow the unsharded loss step by step.
"""
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
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.models.gpt_zero3 import Zero3GPT
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.data_parallel import FusedDataParallel
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine

    cfg = GPTConfig(n_layer=2, d_model=256, n_head=4, d_ff=1024, vocab_size=1000, max_seq=128, name="gpt-zero3-test")
    bs, S = 2, 128
    opt = OptimConfig(lr=1e-3, grad_clip=None)

    def new_tape():
        t = TensorTape(grad_dtype=None)
        t.accumulate_fn = lambda a, b: K.add(a, b) if a.dtype == torch.bfloat16 else a + b
        return t

    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab_size, (world * bs, S + 1), generator=g)
    ids_all, tgt_all = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    mine = slice(rank * bs, (rank + 1) * bs)

    ref = GPT(cfg, new_tape(), device=dev, seed=3)
    sd = ref.state_dict()
    ref_eng = TrainEngine(ref, world * bs, S, opt, use_cuda_graph=False)
    ref_losses = [ref_eng.step(ids_all.pin_memory(), tgt_all.pin_memory()) for _ in range(4)]

    for graph in (False, True):
        tp = Zero3GPT(cfg, new_tape(), dev, group=dist.group.WORLD, seed=3, comm_ctas=4)
        tp.load_full_state_dict(sd)
        dp = FusedDataParallel(tp.arena, dist.group.WORLD, dev)
        eng = TrainEngine(tp, bs, S, opt, use_cuda_graph=graph, dp=dp)
        losses = []
        for _ in range(4):
            l = eng.step(ids_all[mine].contiguous().pin_memory(), tgt_all[mine].contiguous().pin_memory())
            t = torch.tensor([l], device=dev)
            dist.all_reduce(t)
            losses.append(float(t) / world)
        K.check_status()
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 3e-2 * max(1.0, abs(b)), f"graph={graph}: zero3 {losses} vs unsharded {ref_losses}"
        assert losses[-1] < losses[0], losses
        if rank == 0:
            print(f"graph={graph} zero3={['%.4f' % x for x in losses]} ref={['%.4f' % x for x in ref_losses]}")
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("ZERO3_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
