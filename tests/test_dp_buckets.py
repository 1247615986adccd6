"""Bucket planning and shard bookkeeping of the bucketed data-parallel optimizer (host logic only)."""
import pytest
import torch

from frankentorch_b200.parallel.data_parallel import (Bucket, gather_arena_shard, plan_buckets,
                                                      scatter_shards_to_arena)


def _ranges(sizes, align=128):
    out, off = [], 0
    for n in sizes:
        end = off + (n + align - 1) // align * align
        out.append((off, end))
        off = end
    return out, off


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8, 16])
def test_buckets_tile_the_arena_and_shards_tile_each_bucket(world):
    ranges, used = _ranges([50304 * 64, 1024 * 64] + [64, 64, 3 * 64 * 64, 192, 64 * 64, 64] * 6 + [64, 64])
    numel = (used + 1024 * world - 1) // (1024 * world) * (1024 * world)
    bks = plan_buckets(ranges, numel, world, target_elems=200_000, forced_cuts=[ranges[1][1]])
    assert bks[0].lo == 0 and bks[-1].hi == numel
    assert bks[0].hi == ranges[1][1]                     # the forced cut behind the second parameter
    off = 0
    for a, b in zip(bks, bks[1:]):
        assert a.hi == b.lo
    for bk in bks:
        assert bk.off == off and bk.shard % 8 == 0 and bk.lo % 8 == 0
        off += bk.shard
        covered = 0
        for r in range(world):
            lo, hi = bk.owned(r)
            assert lo % 8 == 0 and (hi - lo) % 8 == 0 and hi <= bk.hi
            covered += hi - lo
        assert covered == bk.hi - bk.lo
    ends = {e for _, e in ranges} | {numel}
    assert all(bk.hi in ends for bk in bks)              # boundaries only at parameter ends


def test_bucket_table_is_capped():
    ranges, used = _ranges([1024] * 500)
    bks = plan_buckets(ranges, used, 8, target_elems=1024, max_buckets=64)
    assert len(bks) == 64 and bks[0].lo == 0 and bks[-1].hi == used


def test_shard_round_trip():
    ranges, used = _ranges([1000, 3000, 17, 5000, 129])
    for world in (1, 3, 8):
        bks = plan_buckets(ranges, used, world, target_elems=2500)
        total = sum(b.shard for b in bks)
        full = torch.arange(used, dtype=torch.float32)
        shards = [gather_arena_shard(bks, full, r, total) for r in range(world)]
        assert torch.equal(scatter_shards_to_arena(bks, shards, used), full)


def test_consolidate_bucket_sharded_checkpoint(tmp_path):
    from frankentorch_b200 import serialize
    ranges, used = _ranges([1000, 3000, 17, 5000, 129])
    world = 2
    bks = plan_buckets(ranges, used, world, target_elems=2500)
    total = sum(b.shard for b in bks)
    full = torch.arange(used, dtype=torch.float32) * 0.5
    layout = torch.tensor([[b.lo, b.hi, b.shard, b.off] for b in bks], dtype=torch.float64)
    stem = str(tmp_path / "s")
    for r in range(world):
        serialize.save_sharded({f"optim.m@bshard{r}": gather_arena_shard(bks, full, r, total),
                                "optim.m@layout": layout}, stem, r)
    merged = serialize.consolidate_shards(stem, world)
    assert torch.equal(merged["optim.m"], full)
    assert isinstance(bks[0], Bucket)
