"""Bounded recycling pool for large host buffers (reference: ft-core/src/buffer_pool.rs).

On the GPU the PyTorch caching allocator plays this role (see ``device_stats``); this pool
covers host-side f64 staging buffers with the reference's limits: only buffers of at least
256 KiB are parked, at most 64 of them, at most 512 MiB in total, and a parked buffer is handed
out only if it is no more than 4x larger than the request (:47-60).  ``take_zeroed`` /
``take_filled`` / ``recycle`` / ``stats`` mirror :206-329.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import List

import torch

MIN_POOLED_BYTES = 256 * 1024
MAX_PARKED = 64
MAX_PARKED_BYTES = 512 * 1024 * 1024
MAX_SLACK = 4

_tls = threading.local()
_enabled = True


@dataclass
class PoolStats:
    hits: int = 0
    misses: int = 0
    parked: int = 0
    parked_bytes: int = 0
    recycled: int = 0
    dropped: int = 0


def _state():
    if not hasattr(_tls, "free"):
        _tls.free: List[torch.Tensor] = []
        _tls.stats = PoolStats()
    return _tls


def set_enabled(flag: bool) -> None:
    global _enabled
    _enabled = bool(flag)


def is_enabled() -> bool:
    return _enabled


def clear() -> None:
    """Drop every parked buffer of this thread (the counters of hits and misses are kept)."""
    st = _state()
    st.free.clear()
    st.stats.parked = 0
    st.stats.parked_bytes = 0


def build_overwritten(n: int, fill) -> torch.Tensor:
    """A buffer of ``n`` f64 elements that ``fill(buf)`` writes completely (ft-core/src/buffer_pool.rs:276).

    A parked buffer arrives holding its previous user's values, a fresh one holds zeros: ``fill`` must write every
    element before reading it, so a kernel using this carries a test that parks a poisoned buffer and compares bit
    patterns with the unpooled result."""
    buf = try_take_exact(n)
    if buf is None:
        buf = torch.zeros(n, dtype=torch.float64)
    fill(buf)
    return buf


def try_take_exact(n: int):
    st = _state()
    if not _enabled or n * 8 < MIN_POOLED_BYTES:
        return None
    best = -1
    for i, b in enumerate(st.free):
        if b.numel() >= n and b.numel() <= MAX_SLACK * n and (best < 0 or b.numel() < st.free[best].numel()):
            best = i
    if best < 0:
        st.stats.misses += 1
        return None
    b = st.free.pop(best)
    st.stats.hits += 1
    st.stats.parked = len(st.free)
    st.stats.parked_bytes -= b.numel() * 8
    return b[:n]


def take_filled(n: int, value: float) -> torch.Tensor:
    b = try_take_exact(n)
    if b is None:
        return torch.full((n,), value, dtype=torch.float64)
    return b.fill_(value)


def take_zeroed(n: int) -> torch.Tensor:
    return take_filled(n, 0.0)


def recycle(buf: torch.Tensor) -> bool:
    st = _state()
    base = buf._base if buf._base is not None else buf
    nbytes = base.numel() * 8
    if (not _enabled or base.dtype != torch.float64 or nbytes < MIN_POOLED_BYTES or len(st.free) >= MAX_PARKED
            or st.stats.parked_bytes + nbytes > MAX_PARKED_BYTES):
        st.stats.dropped += 1
        return False
    st.free.append(base.reshape(-1))
    st.stats.recycled += 1
    st.stats.parked = len(st.free)
    st.stats.parked_bytes += nbytes
    return True


def stats() -> PoolStats:
    return _state().stats


def device_stats(device=None) -> dict:
    """Caching-allocator counters of the CUDA device (allocated / reserved bytes, alloc retries)."""
    if not torch.cuda.is_available():
        return {}
    s = torch.cuda.memory_stats(device)
    return {k: s.get(k, 0) for k in ("allocated_bytes.all.current", "reserved_bytes.all.current",
                                     "allocated_bytes.all.peak", "num_alloc_retries")}
