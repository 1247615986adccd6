"""Host-side logic of the weight-gradient queue (no GPU: the grouped launch is replaced by a recorder)."""
import torch

from frankentorch_b200.ops import fused


class _Tape:
    def __init__(self):
        self.written = []
        self.leaf_grad_written_fn = self.written.append
        self.wgrad_queue = None


def _pair(tokens, m, n):
    return torch.zeros(tokens, m, dtype=torch.bfloat16), torch.zeros(tokens, n, dtype=torch.bfloat16)


def test_queue_launches_a_block_together_and_tells_the_observer_at_the_launch(monkeypatch):
    calls = []
    monkeypatch.setattr(fused.K, "gemm_grouped", lambda problems, **kw: calls.append([(a.shape, b.shape, acc) for a, b, _, acc in problems]))
    tape = _Tape()
    q = fused.WgradQueue(tape)
    assert q.tiles_of(2304, 768) == 72 and q.tiles_of(768, 3072) == 96 and q.tiles_of(200, 136) == 2
    bufs = [torch.zeros(1) for _ in range(4)]
    # fc2, fc1, proj: queued, nothing launched, observer silent
    for nid, (m, n) in enumerate(((768, 3072), (3072, 768), (768, 768))):
        q.add(*_pair(64, m, n), bufs[nid], False, 10 + nid)
    assert not calls and not tape.written and q.tiles == 96 + 96 + 24
    # qkv brings the block to 288 tiles: one launch of four problems, then four notifications in queue order
    q.add(*_pair(64, 2304, 768), bufs[3], True, 13)
    assert len(calls) == 1 and len(calls[0]) == 4 and calls[0][3][2] is True
    assert tape.written == [10, 11, 12, 13] and q.tiles == 0 and q.launches == 1
    # another reduction length, or a second contribution to a buffer already queued, flushes first
    q.add(*_pair(64, 768, 768), bufs[0], False, 20)
    q.add(*_pair(128, 768, 768), bufs[1], False, 21)
    assert len(calls) == 2 and len(calls[1]) == 1 and tape.written[-1] == 20
    q.add(*_pair(128, 768, 768), bufs[1], True, 21)
    assert len(calls) == 3 and tape.written[-1] == 21
    # the end of a backward pass flushes what is left; an empty flush does nothing
    q.flush()
    assert len(calls) == 4 and tape.written[-1] == 21 and q.launches == 4
    q.flush()
    assert len(calls) == 4
    # eight problems is the kernel's limit
    for i in range(8):
        q.add(*_pair(64, 128, 192), torch.zeros(1), False, 100 + i)
    assert len(calls) == 5 and len(calls[4]) == 8


def test_queue_only_takes_what_the_grouped_kernel_can_run():
    q = fused.WgradQueue(_Tape())
    dy, x = _pair(64, 768, 768)
    assert not q.accepts(dy, x)                       # CPU tensors keep the direct path
    assert fused.WgradQueue.tiles_of(50304, 768) > fused.WgradQueue.MAX_TILES_PER_PROBLEM   # the LM head stays alone
