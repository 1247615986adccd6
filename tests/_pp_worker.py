"""Worker for the pipeline-parallel test on GPUs (launched by torch.distributed.run, 2 ranks):
two stages over NCCL point-to-point transfers, both schedules, against a single-process run,
with the time the transfers overlap the compute reported."""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    # a short timeout: a mis-ordered exchange must end in an error, not in a wait
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.parallel.pipeline import GPipeStage, tape_op
    M, B, d_in, d_h, d_out = 4, 64, 256, 512, 128
    g = torch.Generator().manual_seed(0)
    w1 = (torch.randn(d_h, d_in, generator=g) * 0.05).to(dev)
    w2 = (torch.randn(d_out, d_h, generator=g) * 0.05).to(dev)
    xs = [torch.randn(B, d_in, generator=g).to(dev) for _ in range(M)]
    ts = [torch.randn(B, d_out, generator=g).to(dev) for _ in range(M)]
    # single-process reference (fp32)
    a, b = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    ref_loss = sum((((torch.relu(x @ a.t()) @ b.t()) - t) ** 2).mean() for x, t in zip(xs, ts)) / M
    ref_loss.backward()
    results = {}
    for schedule in ("gpipe", "1f1b"):
        tape = TensorTape(grad_dtype=torch.float32)
        if rank == 0:
            w = tape.leaf(w1.clone(), requires_grad=True)
            stage = GPipeStage(tape, lambda tp, x, m: tape_op(tp, "relu", [tape_op(tp, "linear", [x, w])]),
                               rank=0, world=2)
            kw = dict(micro_inputs=xs, out_shape=(B, d_h))
        else:
            w = tape.leaf(w2.clone(), requires_grad=True)

            def loss_fn(tp, y, t, m):
                dlt = tape_op(tp, "sub", [y, tp.leaf(t, requires_grad=False)])
                return tape_op(tp, "mean", [tape_op(tp, "mul", [dlt, dlt])])
            stage = GPipeStage(tape, lambda tp, x, m: tape_op(tp, "linear", [x, w]), rank=1, world=2, loss_fn=loss_fn)
            kw = dict(targets=ts, in_shape=(B, d_h))
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        loss = stage.step(n_micro=M, dtype=torch.float32, device=dev, schedule=schedule, **kw)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        grad = tape.accumulated_gradient(w)
        want = (a if rank == 0 else b).grad
        err = float((grad - want).abs().max() / want.abs().max())
        assert err < 1e-4, (schedule, rank, err)
        if rank == 1:
            assert abs(loss - float(ref_loss)) < 1e-4 * max(1.0, abs(float(ref_loss))), (loss, float(ref_loss))
        assert stage.max_live <= (M if schedule == "gpipe" else world - rank)
        results[schedule] = (dt, stage.max_live)
        dist.barrier()
    if rank == 0:
        print("PP_WORKER_OK", {k: (round(v[0] * 1e3, 2), v[1]) for k, v in results.items()})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
