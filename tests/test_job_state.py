"""Scheduler / PRNG / data-loader position survive a save + restore and replay bit for bit (CPU)."""
import pytest
import torch

from frankentorch_b200.data import DataLoader, DataLoaderConfig, TensorDataset
from frankentorch_b200.optim import SGD, CosineAnnealingLR
from frankentorch_b200.session import FrankenTorchSession
from frankentorch_b200.training.checkpoint import load_job_state, restore_job_state, save_job_state


def _job(seed=7):
    s = FrankenTorchSession(seed=seed)
    w = s.tensor_variable([1.0, 2.0], [2], True)
    opt = SGD([w], lr=0.1)
    sched = CosineAnnealingLR(opt, 10)
    ds = TensorDataset({"x": torch.arange(20, dtype=torch.float64).reshape(10, 2), "y": torch.arange(10, dtype=torch.float64)})
    loader = DataLoader(ds, DataLoaderConfig(3).with_shuffle(True))
    loader.seed(99)
    return s, opt, sched, loader


def _advance(s, opt, sched, loader, n):
    trace = []
    for _ in range(n):
        idx = loader.next_indices()
        if idx is None:
            loader.reset()
            idx = loader.next_indices()
        trace.append((tuple(idx), sched.step(opt), s.tensor_values(s.rand([2]))))
    return trace


def test_job_state_round_trip_replays_the_same_stream(tmp_path):
    s, opt, sched, loader = _job()
    _advance(s, opt, sched, loader, 3)
    path = save_job_state(str(tmp_path / "job.json"), scheduler=sched, session=s, loader=loader, step=3, extra={"epoch": 0})
    want = _advance(s, opt, sched, loader, 5)
    s2, opt2, sched2, loader2 = _job(seed=1234)          # different seed: everything comes from the file
    assert load_job_state(path, scheduler=sched2, session=s2, loader=loader2) == 3
    opt2.set_lr(sched2.get_last_lr()[0])
    got = _advance(s2, opt2, sched2, loader2, 5)
    assert got == want


def test_job_state_rejects_foreign_files():
    with pytest.raises(ValueError):
        restore_job_state({"schema": "something-else"})
    s, *_ = _job()
    with pytest.raises(ValueError):
        restore_job_state({"schema": "ft-job-state-v1", "prng": [1, 2, 3]}, session=s)
