"""Canary-padded output buffers: the stand-in for a memory checker's out-of-bounds write detection.

``Canary.empty(shape, dtype)`` hands out a tensor that sits between two guard bands filled with a byte
pattern; after the kernels under test have run, ``Canary.check()`` verifies that every band still holds the
pattern and names the allocation, the side and the first damaged byte otherwise.  Kernels are given these
tensors through their ``out=`` parameters on shapes that are not multiples of a tile, which is where a
stray store would land.  (The reference relies on Rust's bounds checks and Miri for the same purpose,
SECURITY notes in docs/planning; on this backend ``compute-sanitizer`` is not available to the test suite.)
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


class CanaryError(AssertionError):
    """A guard band next to a canary-padded tensor was overwritten."""


class Canary:
    def __init__(self, device, guard_bytes: int = 8192, pattern: int = 0xA5):
        self.device, self.guard, self.pattern = torch.device(device), int(guard_bytes), int(pattern) & 0xFF
        if self.guard % 256:
            raise ValueError("guard_bytes must be a multiple of 256 (the interior keeps the allocator's alignment)")
        self._allocs: List[Tuple[str, torch.Tensor, int]] = []

    def empty(self, shape: Sequence[int], dtype: torch.dtype, name: str = "") -> torch.Tensor:
        """An uninitialised (pattern-filled) tensor of ``shape`` with a guard band on either side."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        raw = torch.full((self.guard + nbytes + self.guard,), self.pattern, dtype=torch.uint8, device=self.device)
        self._allocs.append((name or f"alloc{len(self._allocs)}", raw, nbytes))
        return raw[self.guard:self.guard + nbytes].view(dtype).view(*shape)

    def violations(self) -> List[str]:
        out = []
        for name, raw, nbytes in self._allocs:
            for side, band, base in (("before", raw[:self.guard], -self.guard),
                                     ("after", raw[self.guard + nbytes:], nbytes)):
                bad = (band != self.pattern).nonzero()
                if bad.numel():
                    first = int(bad[0])
                    out.append(f"{name}: {int(bad.numel())} byte(s) written {side} the tensor, first at offset "
                               f"{base + first} from its start")
        return out

    def check(self) -> None:
        v = self.violations()
        if v:
            raise CanaryError("; ".join(v))
