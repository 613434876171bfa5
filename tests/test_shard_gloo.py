"""The multi-GPU host logic (row sharding, shard gather, combination of partial reductions) on two
gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tannic_b200 import shard


def test_shard_range_covers_everything_once():
    for total in (0, 1, 7, 8, 8192, 197):
        for world in (1, 2, 3, 4, 8):
            ranges = [shard.shard_range(total, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.shard_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)  # every rank builds the same full problem, then keeps its shard
        rows = 9
        full = torch.randn(rows, 5)
        y = torch.randn(1, 5)
        mine = shard.shard_leading(full, world, rank)
        local = torch.log(mine.abs() + 1) + y * y          # a row-sharded elementwise op, y replicated
        gathered = shard.gather_shards(local, rows)
        ok = torch.allclose(gathered, torch.log(full.abs() + 1) + y * y)
        # reduction along the sharded axis: partial sums, and argmax with the lowest-index tie rule
        total = shard.combine_sum(mine.sum(0))
        ok = ok and torch.allclose(total, full.sum(0), atol=1e-5)
        tied = full.clone()
        tied[2] = 100.0
        tied[7] = 100.0                                     # equal maxima in two different shards
        part = shard.shard_leading(tied, world, rank)
        start, _ = shard.shard_range(rows, world, rank)
        v, i = part.max(0)
        gv, gi = shard.combine_argmax(v, i, start)
        ok = ok and torch.equal(gi, torch.full((5,), 2)) and torch.equal(gv, torch.full((5,), 100.0))
        slow = shard.max_over_ranks(1.0 + rank)
        ok = ok and slow == float(world)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_and_partial_reductions():
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
