"""Worker for the multi-GPU expert-parallel MoE test (launched by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from _moe_check import run
    run(dist.group.WORLD, rank, world, dev)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("MOE_WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
