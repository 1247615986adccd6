"""Failure detection: heartbeats and typed errors on the host, bounded waits on the device.

Failures are injected on the host only (a rank that raises, exits, or stops publishing); the one
device test lets a bounded wait run out on a flag that nothing sets and reads the status word.
"""
import multiprocessing as mp
import os
import time

import pytest
import torch
import torch.distributed as dist

from frankentorch_b200.parallel.health import (DeviceWaitTimeout, HardenedTrainer, PeerFailure, RankHealth,
                                               device_status_error, gloo_max_agreement)


def test_heartbeat_timeout_and_announced_failure():
    store = dist.HashStore()
    now = [100.0]
    a = RankHealth(store, 0, 2, timeout_s=5.0, clock=lambda: now[0])
    with pytest.raises(PeerFailure, match="never published"):
        a.check_peers()
    b = RankHealth(store, 1, 2, timeout_s=5.0, clock=lambda: now[0])
    a.before_step(1)
    now[0] += 4.0
    b.beat(1)
    a.before_step(2)
    now[0] += 6.0                      # rank 1 silent for more than the timeout
    with pytest.raises(PeerFailure) as e:
        a.before_step(3)
    assert e.value.rank == 1 and "no heartbeat" in e.value.reason
    b.beat(3)
    a.check_peers()
    b.announce_failure("loss is NaN")
    with pytest.raises(PeerFailure, match="announced failure.*loss is NaN"):
        a.check_peers()


def test_status_word_decoding():
    assert device_status_error(0) is None
    err = device_status_error(5 | (17 << 8))
    assert isinstance(err, DeviceWaitTimeout) and err.code == 5 and err.cta == 17 and "another rank" in err.name


class _FakeDP:
    def __init__(self, name, ok=True):
        self.name, self.ok = name, ok

    def step_ok(self):
        return self.ok


class _FakeEngine:
    """The two things the policy needs from an engine: run a step, swap the data-parallel object."""

    def __init__(self, dp):
        self.dp, self.steps, self.device_steps, self.switched = dp, 0, 0, 0

    def step(self, ids, targets, read_loss=True):
        self.steps += 1
        return float(self.steps)

    def step_device(self, read_loss=False):
        self.device_steps += 1
        return -1.0

    def switch_data_parallel(self, factory):
        self.dp = factory()
        self.switched += 1


class _Ledger:
    def __init__(self):
        self.rows = []

    def record(self, kind, summary, detail):
        self.rows.append((kind, summary, detail))


def test_strict_raises_and_hardened_falls_back():
    status = [0]
    strict = HardenedTrainer(_FakeEngine(_FakeDP("fused")), lambda: _FakeDP("nccl"), mode="strict",
                             read_status=lambda: status[0], check_every=2)
    strict.step(None, None)
    strict.step(None, None)
    status[0] = 5 | (3 << 8)
    strict.step(None, None)                       # odd step: not polled
    with pytest.raises(DeviceWaitTimeout):
        strict.step(None, None)

    led = _Ledger()
    status[0] = 0
    eng = _FakeEngine(_FakeDP("fused", ok=False))
    hard = HardenedTrainer(eng, lambda: _FakeDP("nccl"), mode="hardened", read_status=lambda: status[0],
                           check_every=1, ledger=led)
    assert hard.step(None, None) == 1.0 and eng.dp.name == "fused" and not hard.fell_back
    status[0] = 5
    # the failed step updated nothing (step_ok() is False): it is run again on the fallback path
    assert hard.step(None, None) == -1.0
    assert hard.fell_back and eng.dp.name == "nccl" and eng.switched == 1 and eng.device_steps == 1
    assert led.rows and led.rows[0][0] == "durability" and hard.events[0]["code"] == 5
    assert hard.events[0]["last_step_rerun"] is True
    hard.step(None, None)                         # no more polling after the fallback
    assert eng.switched == 1 and eng.device_steps == 1


def _agree_main(rank, world, port, q):
    """gloo ranks: only rank 1's device reports a timeout; both must take the fallback branch."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=__import__("datetime").timedelta(seconds=60))
    eng = _FakeEngine(_FakeDP("fused", ok=True))
    status = [0]
    tr = HardenedTrainer(eng, lambda: _FakeDP("nccl"), mode="hardened", read_status=lambda: status[0],
                         agree=gloo_max_agreement(dist.group.WORLD), check_every=1)
    tr.step(None, None)
    if rank == 1:
        status[0] = 5 | (9 << 8)
    tr.step(None, None)
    q.put((rank, tr.fell_back, eng.dp.name, tr.events[0]["local_status"], tr.events[0]["agreed_status"]))
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_agree_on_the_fallback_over_a_host_group():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29950 + os.getpid() % 40
    procs = [ctx.Process(target=_agree_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        item = q.get(timeout=90)
        res[item[0]] = item
    for p in procs:
        p.join(timeout=30)
        assert not p.is_alive()
    assert res[0][1:] == (True, "nccl", 0, 5 | (9 << 8))
    assert res[1][1:] == (True, "nccl", 5 | (9 << 8), 5 | (9 << 8))


@pytest.mark.gpu
def test_hardened_fallback_through_the_real_engine(cuda_device):
    """World of one on a real GPU: a reported timeout (injected through the status reader, no kernel
    is made to wait) makes the engine leave its captured graph, gather the sharded optimizer state
    back into the arena and continue on the library path; training goes on from the same state."""
    from frankentorch_b200.autograd.tape import TensorTape
    from frankentorch_b200.models.gpt import GPT, GPTConfig
    from frankentorch_b200.ops import kernels as K
    from frankentorch_b200.parallel.data_parallel import FusedDataParallel, NcclDataParallel
    from frankentorch_b200.training.engine import OptimConfig, TrainEngine
    cfg = GPTConfig.preset("gpt-tiny")

    def make(peer):
        tape = TensorTape(grad_dtype=None)
        tape.accumulate_fn = lambda a, b: K.add(a, b) if (a.dtype == torch.bfloat16 and a.is_cuda) else a + b
        model = GPT(cfg, tape, device=cuda_device, seed=3, peer_visible=peer)
        dp = FusedDataParallel(model.arena, None, cuda_device, wire="fp32", bucket_elems=40_000) if peer else None
        return model, TrainEngine(model, 2, 128, OptimConfig(lr=1e-3, grad_clip=None), use_cuda_graph=True, dp=dp)
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g)
    ids, tgt = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    m_ref, e_ref = make(False)
    ref = [e_ref.step(ids, tgt) for _ in range(6)]
    model, eng = make(True)
    status = [0]
    led = _Ledger()
    tr = HardenedTrainer(eng, lambda: NcclDataParallel(model.arena, None, cuda_device), mode="hardened",
                         read_status=lambda: status[0], check_every=1, ledger=led)
    got = [tr.step(ids, tgt) for _ in range(3)]
    status[0] = 5
    got += [tr.step(ids, tgt) for _ in range(3)]
    eng.sync_parameters()
    K.check_status()
    assert tr.fell_back and isinstance(eng.dp, NcclDataParallel) and not eng.use_graph
    assert model.arena.master is not None and model.arena.m is not None
    assert led.rows and tr.events[0]["last_step_rerun"] is False
    assert got == ref, (got, ref)
    assert torch.equal(model.arena.params, m_ref.arena.params)


def _rank_main(rank, world, port, q):
    """gloo ranks: all-reduce for a few steps; rank 2 raises after step 2 and leaves between steps."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    health = RankHealth(store, rank, world, timeout_s=3.0)
    dist.barrier()
    done = 0
    try:
        for step in range(1, 8):
            if rank == 2 and step == 3:
                raise FloatingPointError("injected: loss is NaN")
            # peers learn of a failure on the host, before they enter the next collective
            deadline = time.time() + 2.0
            while time.time() < deadline:
                health.before_step(step)
                others = [s["hb"]["step"] for s in health.peer_states().values() if s["hb"]]
                if all(s >= step for s in others):
                    break
                time.sleep(0.02)
            else:
                health.check_peers()
                raise PeerFailure(-1, "peers did not reach the step")
            t = torch.ones(4) * rank
            dist.all_reduce(t)
            done = step
        q.put((rank, "finished", done))
    except PeerFailure as e:
        q.put((rank, "peer_failure", done, e.rank))
    except FloatingPointError as e:
        health.announce_failure(str(e))
        q.put((rank, "raised", done))
    time.sleep(0.5)       # keep the store alive while the others read it


def test_gloo_ranks_detect_a_failed_peer_between_steps():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29750 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(3):
        item = q.get(timeout=90)
        res[item[0]] = item
    for p in procs:
        p.join(timeout=30)
        assert not p.is_alive()
    assert res[2][1] == "raised" and res[2][2] == 2
    for r in (0, 1):
        assert res[r][1] == "peer_failure" and res[r][3] == 2, res
        assert res[r][2] == 2, "survivors must stop before entering the collective of step 3"


@pytest.mark.gpu
def test_bounded_device_wait_reports_and_context_survives(cuda_device):
    from frankentorch_b200.ops import _lib
    from frankentorch_b200.ops import kernels as K
    lib = _lib.load()
    K.check_status()
    flag = torch.zeros(1, dtype=torch.int32, device=cuda_device)          # nothing ever sets it
    waited = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    budget = 200_000_000                                                   # ~0.1 s of SM cycles
    rc = lib.ftk_wait_probe(flag.data_ptr(), 1, budget, waited.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    with pytest.raises(K.KernelError, match="status"):
        K.check_status()
    assert int(waited) >= budget
    err = device_status_error(5)
    assert isinstance(err, DeviceWaitTimeout)
    # the status word was reset and the context still runs kernels; a satisfied wait is silent
    flag.fill_(1)
    rc = lib.ftk_wait_probe(flag.data_ptr(), 1, budget, waited.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    K.check_status()
    assert int(waited) == 0
    x = torch.ones(1024, device=cuda_device)
    assert float((x * 2).sum()) == 2048.0
