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


def gather_shards(local: torch.Tensor, total_rows: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather of leading-dimension shards produced with `shard_range` into the whole tensor on
    every rank. Even, dense shards go straight into the result buffer with one collective
    (`all_gather_into_tensor`; `out`, if given, is that buffer and is reused between calls); uneven
    ones are padded to the longest shard and trimmed."""
    w, r = world()
    if w == 1:
        return local
    if total_rows % w == 0 and local.is_contiguous() and local.shape[0] == total_rows // w:
        if out is None:
            out = torch.empty((total_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local)
        return out
    sizes = [shard_range(total_rows, w, i) for i in range(w)]
    longest = max(b - a for a, b in sizes)
    padded = torch.zeros((longest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(w)]
    dist.all_gather(parts, padded)
    return torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)], dim=0)


class PeerBuffer:
    """A result buffer that every rank of the box can write into: `local` is this rank's copy of the whole
    result (an ordinary CUDA tensor, allocated as symmetric memory), `peers[p]` is rank p's copy mapped into
    this process. A copy into `peers[p]` is a device-to-device `cudaMemcpyAsync` that the copy engines carry
    over NVLink: no SM is involved, so it runs beside a kernel that fills every SM. Plumbing only (torch's
    symmetric-memory allocator and rendezvous); no kernel of this library ever takes a peer's memory as an
    operand. CUDA + NCCL process groups only."""

    def __init__(self, shape, dtype, group=None):
        import os

        # only plain peer copies are used here: no multicast object is bound to the buffer (a process that dies while
        # its memory is bound to one can raise NVLink faults on its peers)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        device = torch.device("cuda", torch.cuda.current_device())
        self.local = symm.empty(tuple(shape), dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.local, self.group)
        w = dist.get_world_size(self.group)
        self.peers = [self.handle.get_buffer(p, tuple(shape), dtype) for p in range(w)]
        self.side = torch.cuda.Stream()
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)

    def fence(self):
        """Stream-ordered barrier over the group: whatever the ranks enqueued before it is complete
        everywhere before anything enqueued after it starts (a one-element all-reduce)."""
        dist.all_reduce(self._flag, group=self.group)


def produce_and_gather(out, rows_per_rank: int, produce, pieces: int | None = None) -> torch.Tensor:
    """Compute this rank's `rows_per_rank` leading rows of the whole result piece by piece and ship every
    finished piece to all other ranks while the next one is being computed.

    `out` is the WHOLE result on every rank ([world * rows_per_rank, ...], dense): a `PeerBuffer`, or a
    plain tensor. Rank r owns rows [r * rows_per_rank, (r + 1) * rows_per_rank). `produce(lo, hi, dst)`
    must enqueue, on the current stream, the work that writes local rows [lo, hi) into `dst` (a view of
    this rank's own rows of the result: nothing is staged or copied on the owner).

    With a `PeerBuffer` every finished piece is copied into the peers' buffers by the copy engines on a side
    stream (one `cudaMemcpyAsync` per peer and piece, ordered after the piece's kernel by an event), so the
    transfer costs the producing kernel no SM; a stream-ordered fence before the first piece (nobody still
    reads the previous result) and after the last copy (every piece has landed everywhere) brackets the call.
    With a plain tensor the N - 1 sends of a piece and the N - 1 receives of the peers' matching pieces go out
    as one grouped point-to-point call of the process group (NCCL: SM-based kernels, which overlap a
    persistent GEMM only if it leaves them SMs, see tn_set_sm_margin; gloo on CPU). Returns the whole result
    once every piece of every rank has arrived (in stream order). With one rank it just runs `produce`.
    `pieces` = None picks four pieces for two ranks, two for up to four and one beyond."""
    w, r = world()
    whole = out.local if isinstance(out, PeerBuffer) else out
    mine = whole[r * rows_per_rank:(r + 1) * rows_per_rank]
    if w == 1:
        produce(0, rows_per_rank, mine)
        return whole
    if pieces is None:
        # every copy or send costs a fixed few microseconds of idle link: with two ranks the kernel is the longer
        # part and four pieces hide most of the exchange; from four ranks on the exchange is the longer part and
        # fewer, larger pieces keep the links busier (measured on config 3: 4 / 2 / 1 pieces take 0.79 / 0.72 / 0.84 ms
        # on 4 GPUs and 1.00 / 0.88 / 0.86 ms on 8, where the exchange is four times the kernel)
        pieces = 4 if w <= 2 else 2 if w <= 4 else 1
    pieces = max(1, min(int(pieces), rows_per_rank))
    bounds = [(c * rows_per_rank // pieces, (c + 1) * rows_per_rank // pieces) for c in range(pieces)]
    bounds = [(lo, hi) for lo, hi in bounds if hi > lo]
    if isinstance(out, PeerBuffer):
        out.fence()
        main = torch.cuda.current_stream()
        for lo, hi in bounds:
            produce(lo, hi, mine[lo:hi])
            done = torch.cuda.Event()
            done.record(main)
            out.side.wait_event(done)
            with torch.cuda.stream(out.side):
                for k in range(1, w):
                    p = (r + k) % w  # every rank starts with a different peer
                    out.peers[p][r * rows_per_rank + lo:r * rows_per_rank + hi].copy_(mine[lo:hi], non_blocking=True)
        main.wait_stream(out.side)
        out.fence()
        return whole
    pending = []
    for lo, hi in bounds:
        produce(lo, hi, mine[lo:hi])
        ops = []
        for peer in range(w):
            if peer == r:
                continue
            ops.append(dist.P2POp(dist.isend, mine[lo:hi], peer))
            ops.append(dist.P2POp(dist.irecv, whole[peer * rows_per_rank + lo:peer * rows_per_rank + hi], peer))
        pending.extend(dist.batch_isend_irecv(ops))
    for req in pending:
        req.wait()
    return whole


def matmul_into_all(buffer: PeerBuffer, rows_per_rank: int, a_local: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The batch- or row-sharded product whose whole result every rank needs, as ONE kernel per rank: rank r
    computes its `rows_per_rank` rows of `a_local @ b` and the GEMM's epilogue stores every result tile into
    its slot of the whole result on this GPU and, through plain peer stores, on every other GPU
    (`tn_gemm_mirrored`), so NVLink carries a tile while the tensor cores work on the next one. A
    stream-ordered fence before the kernel (nobody still reads the previous result) and after it (every
    rank's tiles have landed everywhere) brackets the call. Returns this rank's copy of the whole result."""
    from . import ops as tb

    w, r = world()
    lo, hi = r * rows_per_rank, (r + 1) * rows_per_rank
    mine = buffer.local[lo:hi]
    if w == 1:
        tb.matmul(a_local, b, out=mine)
        return buffer.local
    buffer.fence()
    tb.matmul_mirrored(a_local, b, mine, [buffer.peers[(r + k) % w][lo:hi] for k in range(1, w)])
    buffer.fence()
    return buffer.local


def combine_sum(partial: torch.Tensor) -> torch.Tensor:
    """Sum over ranks of per-rank partial sums, accumulated as wide as the one-GPU reduction does
    (float32 for 16-bit floats, float64 for float32 / float64, int64 for integers)."""
    w, _ = world()
    if w == 1:
        return partial
    if not partial.is_floating_point():
        wide = torch.int64
    elif partial.dtype in (torch.float16, torch.bfloat16):
        wide = torch.float32
    else:
        wide = torch.float64
    acc = partial.to(wide)
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


class Mesh:
    """The GPUs of one box as seen from this process: the handle the reference leaves as a TODO
    (`class Mesh`, include/tannic/resources.hpp:194-197). One process drives one GPU; the mesh is the
    process group. `scatter` cuts a whole host tensor into this rank's resident shard, `Sharded`
    remembers where the shard sits in the whole, and the collectives above act on it."""

    def __init__(self):
        self.size, self.rank = world()

    def range(self, total: int) -> tuple[int, int]:
        return shard_range(total, self.size, self.rank)

    def scatter(self, whole: torch.Tensor, device=None) -> "Sharded":
        lo, hi = self.range(whole.shape[0])
        local = whole[lo:hi]
        if device is not None:
            local = local.to(device, non_blocking=True)
        return Sharded(self, local, whole.shape[0], lo)

    def wrap(self, local: torch.Tensor, total_rows: int) -> "Sharded":
        lo, hi = self.range(total_rows)
        if local.shape[0] != hi - lo:
            raise ValueError(f"rank {self.rank} owns rows [{lo}, {hi}) of {total_rows}, got {local.shape[0]}")
        return Sharded(self, local, total_rows, lo)


class Sharded:
    """A tensor split along its leading dimension over a Mesh: this rank's shard, the whole's leading
    extent and the shard's first global row."""

    def __init__(self, mesh: Mesh, local: torch.Tensor, total_rows: int, offset: int):
        self.mesh, self.local, self.total_rows, self.offset = mesh, local, total_rows, offset

    def map(self, fn) -> "Sharded":
        """Applies a row-independent op to the shard (rows in, the same rows out)."""
        return Sharded(self.mesh, fn(self.local), self.total_rows, self.offset)

    def gather(self, out: torch.Tensor | None = None) -> torch.Tensor:
        return gather_shards(self.local, self.total_rows, out=out)

    def sum_over_rows(self, reduce_local) -> torch.Tensor:
        """`reduce_local(shard)` gives this rank's partial sum over its rows; ranks are combined."""
        return combine_sum(reduce_local(self.local))

    def argmax_over_rows(self, max_local, argmax_local):
        return combine_argmax(max_local(self.local), argmax_local(self.local), self.offset)
