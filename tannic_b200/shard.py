"""Sharding of the operator hot path over the GPUs of one box (one process per GPU).

Every benchmark workload splits on its leading dimension — rows of an elementwise op, images of
a convolution, batch entries of a matmul — with the small operands (a row-broadcast vector,
weights) replicated, so ranks exchange nothing on the data path. Collectives appear in exactly two
places, both outside the kernels:

  * `gather_shards`   — all-gather of the per-rank result shards when a consumer wants the whole
                        tensor on every rank;
  * `combine_sum` / `combine_argmax` — a reduction ALONG the sharded axis: per-rank partial sums are
                        all-reduced; for argmax every rank contributes (value, global index) and
                        the lowest index among equal maxima wins, the reference's tie rule
                        (src/cpu/argred.cpp:80-108).

The functions take whatever backend the process group was created with (NCCL on GPUs, gloo in the
CPU tests). The reference has no multi-device support at all (README.md:124).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of rank's contiguous share of `total` leading-dimension entries; the first
    `total % world` ranks get one extra entry."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_leading(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """This rank's rows of `t` (a view)."""
    start, stop = shard_range(t.shape[0], world, rank)
    return t[start:stop]


def world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def max_over_ranks(value: float, device=None) -> float:
    """Largest `value` over all ranks (timings are reported as the slowest rank's)."""
    w, _ = world()
    if w == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_shards(local: torch.Tensor, total_rows: int) -> torch.Tensor:
    """All-gather of leading-dimension shards produced with `shard_range` (shards may be uneven)."""
    w, r = world()
    if w == 1:
        return local
    sizes = [shard_range(total_rows, w, i) for i in range(w)]
    longest = max(b - a for a, b in sizes)
    padded = torch.zeros((longest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(w)]
    dist.all_gather(parts, padded)
    return torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)], dim=0)


def combine_sum(partial: torch.Tensor) -> torch.Tensor:
    """Sum over ranks of per-rank partial sums (accumulated in float32 / int64)."""
    w, _ = world()
    if w == 1:
        return partial
    acc = partial.to(torch.float32 if partial.is_floating_point() else torch.int64)
    dist.all_reduce(acc, op=dist.ReduceOp.SUM)
    return acc.to(partial.dtype)


def combine_argmax(local_value: torch.Tensor, local_index: torch.Tensor, offset: int):
    """Global (max value, argmax) along a sharded axis from each rank's local maximum and local
    index; `offset` is the global index of this rank's first entry. Equal maxima resolve to the
    lowest global index; a NaN never wins."""
    w, _ = world()
    gidx = local_index.to(torch.int64) + offset
    if w == 1:
        return local_value, gidx
    vals = [torch.empty_like(local_value) for _ in range(w)]
    idxs = [torch.empty_like(gidx) for _ in range(w)]
    dist.all_gather(vals, local_value.contiguous())
    dist.all_gather(idxs, gidx.contiguous())
    best_v, best_i = vals[0].clone(), idxs[0].clone()
    for v, i in zip(vals[1:], idxs[1:]):
        better = (v > best_v) | ((v == best_v) & (i < best_i)) | (torch.isnan(best_v) & ~torch.isnan(v))
        best_v = torch.where(better, v, best_v)
        best_i = torch.where(better, i, best_i)
    return best_v, best_i
