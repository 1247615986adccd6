"""Device timing and NVTX ranges.

The reference's observability is structural (dispatch decisions, backward telemetry, stage
profilers inside single kernels such as ``eigh_stage_profile_f64``
crates/ft-kernel-cpu/src/lib.rs:28235 and the SVD nanosecond counters ``:33786-33820``).  On the
GPU the equivalents are CUDA events on the launching stream and NVTX ranges that a timeline tool
can attribute to tape nodes; both live here.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Dict, List, Optional

import torch

from .config import env_flag


@contextlib.contextmanager
def _null_range(_name: str):
    yield


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when a CUDA device is present; a no-op on CPU builds."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def install_tape_ranges(tape, enabled: Optional[bool] = None, range_fn: Optional[Callable] = None) -> bool:
    """Wrap every backward rule of ``tape`` in a range named ``bwd:<rule>#<node>``.

    ``enabled`` defaults to the ``FT_NVTX`` switch.  Under CUDA graph capture the ranges are seen
    once, at capture time, which is where the tape runs.  Returns whether ranges are on.
    """
    on = bool(env_flag("FT_NVTX")) if enabled is None else bool(enabled)
    tape.range_fn = (range_fn or nvtx_range) if on else None
    return on


class StageProfile:
    """Named stages timed with CUDA events (device time) or ``perf_counter`` (CPU tensors).

        prof = StageProfile()
        with prof.stage("forward"): ...
        with prof.stage("backward"): ...
        prof.summary()   # {"forward": {"n": 1, "ms": ...}, ...}
    """

    def __init__(self, device: Optional[torch.device] = None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._open: List = []
        self._events: Dict[str, List] = {}
        self._cpu: Dict[str, List[float]] = {}

    @contextlib.contextmanager
    def stage(self, name: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            with nvtx_range(name):
                yield
            b.record()
            self._events.setdefault(name, []).append((a, b))
        else:
            import time
            t0 = time.perf_counter()
            yield
            self._cpu.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)

    def summary(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        if self.cuda:
            torch.cuda.synchronize()
            for k, evs in self._events.items():
                ms = [a.elapsed_time(b) for a, b in evs]
                out[k] = {"n": len(ms), "ms": sum(ms), "ms_max": max(ms)}
        for k, ms in self._cpu.items():
            out[k] = {"n": len(ms), "ms": sum(ms), "ms_max": max(ms)}
        return out
