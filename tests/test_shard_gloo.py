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
        # even shards take the single-collective path into a reusable result buffer
        even = torch.arange(8 * 3, dtype=torch.float32).reshape(8, 3)
        buf = torch.empty_like(even)
        ok = ok and torch.equal(shard.gather_shards(shard.shard_leading(even, world, rank).contiguous(), 8, out=buf), even) and buf.data_ptr() == buf.data_ptr()
        # float64 partial sums keep their precision (float32 would lose the small term)
        big = torch.tensor([1e9 if rank == 0 else 0.123456789], dtype=torch.float64)
        ok = ok and float(shard.combine_sum(big)) == 1e9 + 0.123456789
        # 16-bit partials are combined in float32: 2048 + 1 is not representable in float16, 2048 + 2048 is
        half = shard.combine_sum(torch.tensor([2048.0], dtype=torch.float16))
        ok = ok and half.dtype == torch.float16 and float(half) == 4096.0
        # the Mesh handle: scatter, a row-independent op, gather; and reductions over the sharded axis
        mesh = shard.Mesh()
        sharded = mesh.scatter(full)
        ok = ok and sharded.offset == start and torch.equal(sharded.map(lambda t: t * 2).gather(), full * 2)
        ok = ok and torch.allclose(sharded.sum_over_rows(lambda t: t.sum(0)), full.sum(0), atol=1e-5)
        mv, mi = mesh.scatter(tied).argmax_over_rows(lambda t: t.max(0).values, lambda t: t.max(0).indices)
        ok = ok and torch.equal(mi, torch.full((5,), 2))
        try:
            mesh.wrap(full, rows)
            ok = False  # the whole tensor is not this rank's shard
        except ValueError:
            pass
        # a product computed piece by piece, every finished piece shipped while the next is computed:
        # rank r owns rows [r * 7, r * 7 + 7) of the whole result (7 rows do not split evenly into 3 pieces)
        a_full, w_mat = torch.randn(world * 7, 6), torch.randn(6, 4)
        whole = torch.full((world * 7, 4), float("nan"))
        calls = []

        def produce(lo, hi, dst):
            calls.append((lo, hi))
            dst.copy_(a_full[rank * 7 + lo:rank * 7 + hi] @ w_mat)

        shard.produce_and_gather(whole, 7, produce, pieces=3)
        ok = ok and torch.allclose(whole, a_full @ w_mat) and calls == [(0, 2), (2, 4), (4, 7)]
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
