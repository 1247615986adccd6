"""GPipe schedule over gloo point-to-point transfers (CPU ranks) against a single-process run."""
import datetime
import multiprocessing as mp
import os

import torch
import torch.distributed as dist


def _weights():
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(16, 8, generator=g, dtype=torch.float64) * 0.3
    w2 = torch.randn(4, 16, generator=g, dtype=torch.float64) * 0.3
    xs = [torch.randn(5, 8, generator=g, dtype=torch.float64) for _ in range(3)]
    ts = [torch.randn(5, 4, generator=g, dtype=torch.float64) for _ in range(3)]
    return w1, w2, xs, ts


def _reference():
    w1, w2, xs, ts = _weights()
    w1 = w1.clone().requires_grad_(True)
    w2 = w2.clone().requires_grad_(True)
    loss = sum((((torch.relu(x @ w1.t()) @ w2.t()) - t) ** 2).mean() for x, t in zip(xs, ts)) / len(xs)
    loss.backward()
    return float(loss), w1.grad, w2.grad


def _rank_main(rank, world, port, q, schedule="gpipe"):
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.parallel.pipeline import GPipeStage, tape_op
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    w1, w2, xs, ts = _weights()
    tape = TensorTape(grad_dtype=torch.float64)
    if rank == 0:
        w = tape.leaf(w1, requires_grad=True)
        stage = GPipeStage(tape, lambda tp, x, m: tape_op(tp, "relu", [tape_op(tp, "linear", [x, w])]),
                           rank=0, world=2)
        stage.step(n_micro=3, micro_inputs=xs, out_shape=(5, 16), schedule=schedule)
        q.put((0, (stage.max_live, stage.last_order), tape.accumulated_gradient(w)))
    else:
        w = tape.leaf(w2, requires_grad=True)

        def loss_fn(tp, y, t, m):
            d = tape_op(tp, "sub", [y, tp.leaf(t, requires_grad=False)])
            return tape_op(tp, "mean", [tape_op(tp, "mul", [d, d])])
        stage = GPipeStage(tape, lambda tp, x, m: tape_op(tp, "linear", [x, w]), rank=1, world=2, loss_fn=loss_fn)
        loss = stage.step(n_micro=3, targets=ts, in_shape=(5, 16), schedule=schedule)
        q.put((1, loss, tape.accumulated_gradient(w)))
    dist.barrier()
    dist.destroy_process_group()


def test_gpipe_two_stages_match_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29850 + os.getpid() % 100
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        r, loss, g = q.get(timeout=120)
        res[r] = (loss, g)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ref_loss, g1, g2 = _reference()
    assert abs(res[1][0] - ref_loss) < 1e-12
    assert torch.allclose(res[0][1], g1, atol=1e-12, rtol=1e-12)
    assert torch.allclose(res[1][1], g2, atol=1e-12, rtol=1e-12)


def test_one_f_one_b_matches_single_process_and_bounds_live_micro_batches():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29950 + os.getpid() % 40
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q, "1f1b")) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        r, info, g = q.get(timeout=120)
        res[r] = (info, g)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    ref_loss, g1, g2 = _reference()
    assert abs(res[1][0] - ref_loss) < 1e-12
    assert torch.allclose(res[0][1], g1, atol=1e-12, rtol=1e-12)
    assert torch.allclose(res[1][1], g2, atol=1e-12, rtol=1e-12)
    max_live, order = res[0][0]
    # stage 0 of 2: one warm-up forward, then forward / backward pairs, then the last backward
    assert order == [("f", 0), ("f", 1), ("b", 0), ("f", 2), ("b", 1), ("b", 2)] and max_live == 2
