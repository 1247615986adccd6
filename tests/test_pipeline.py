"""GPipe schedule over gloo point-to-point transfers (CPU ranks) against a single-process run."""
import datetime
import multiprocessing as mp
import os

import pytest
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


def test_posting_orders_pair_up_for_every_stage_and_schedule():
    """The host-side replay of the per-pair posting orders (what an in-order point-to-point stream
    would execute) finds no two ranks waiting for each other, for both schedules and several shapes;
    and it does flag an order in which both neighbours send first."""
    from frankentorch_b200.parallel import pipeline as P
    for schedule in ("gpipe", "1f1b"):
        for world in (2, 3, 4, 8):
            for M in (1, 2, 3, 4, 8, 16):
                for r in range(world):
                    P.check_pair_orders(r, world, M, schedule)
    # 1F1B steady state: a stage's send of the next activation and its receive of a gradient form one group
    g = P.comm_groups(0, 2, 3, "1f1b")
    assert [("send", 1, "act", 1), ("recv", 1, "grad", 0)] in g
    assert P.comm_groups(1, 2, 3, "1f1b")[1] == [("send", 0, "grad", 0), ("recv", 0, "act", 1)]
    # without grouping, the same schedule has both stages sending first: the replay must refuse it
    real = P.comm_groups

    def ungrouped(rank, world, n_micro, schedule):
        return [[t] for grp in real(rank, world, n_micro, schedule) for t in grp]
    P.comm_groups = ungrouped
    try:
        import pytest
        with pytest.raises(RuntimeError, match="deadlock"):
            P.check_pair_orders(0, 2, 3, "1f1b")
    finally:
        P.comm_groups = real


def test_release_values_frees_a_micro_batch_but_keeps_ids():
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.parallel.pipeline import tape_op
    tape = TensorTape(grad_dtype=torch.float64)
    w = tape.leaf(torch.ones(3, 3, dtype=torch.float64), requires_grad=True)
    lo = len(tape)
    x = tape.leaf(torch.ones(2, 3, dtype=torch.float64), requires_grad=False)
    y = tape_op(tape, "relu", [tape_op(tape, "linear", [x, w])])
    hi = len(tape)
    assert tape.release_values(lo, hi) == 2
    assert tape.value(y) is None and tape.value(w) is not None and tape.value(x) is not None
    assert len(tape) == hi


def test_posting_orders_complete_on_one_in_order_queue_per_rank():
    """Grouped NCCL transfers of a rank share one stream whatever the neighbour: the replay with one queue
    per rank must drain for every schedule, and a hand-made bad order must be refused."""
    from frankentorch_b200.parallel import pipeline as pp
    for world in (2, 3, 4, 5):
        for m in (1, 2, 4, 7):
            for schedule in ("gpipe", "1f1b"):
                pp.check_fifo_orders(world, m, schedule)
    real = pp.comm_groups

    def both_send_first(rank, world, n_micro, schedule):
        return [[("send", 1 - rank, "act", 0)], [("recv", 1 - rank, "act", 0)]]
    pp.comm_groups = both_send_first
    try:
        with pytest.raises(RuntimeError, match="deadlock"):
            pp.check_fifo_orders(2, 1, "gpipe")
    finally:
        pp.comm_groups = real
