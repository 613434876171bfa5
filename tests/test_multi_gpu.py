"""Two ranks on two GPUs (child processes, NCCL): the piecewise produce-and-gather with both transports
against a product computed in one piece. Skipped on a box with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from tannic_b200 import ops as tb
        from tannic_b200 import shard
        import oracle

        rows, k, n = 700, 256, 520  # 700 rows per rank do not split evenly into 3 pieces
        a = oracle.fill((world * rows, k), torch.bfloat16, 300, "uniform", -1.0, 1.0)
        w = oracle.fill((n, k), torch.bfloat16, 301, "uniform", -1.0, 1.0)
        da, dw = a[rank * rows:(rank + 1) * rows].cuda(), w.cuda()
        whole = tb.matmul(a.cuda(), dw.t())  # every rank computes the full product once, as the expected value

        def produce(lo, hi, dst):
            tb.matmul(da[lo:hi], dw.t(), out=dst)

        ok = True
        plain = torch.zeros_like(whole)
        shard.produce_and_gather(plain, rows, produce, pieces=3)
        torch.cuda.synchronize()
        ok = ok and torch.equal(plain.view(torch.int16), whole.view(torch.int16))
        shared = shard.PeerBuffer(tuple(whole.shape), whole.dtype)
        for _ in range(2):  # the second call reuses the buffers the first one filled
            shared.local.zero_()
            shard.produce_and_gather(shared, rows, produce, pieces=3)
            torch.cuda.synchronize()
            ok = ok and torch.equal(shared.local.view(torch.int16), whole.view(torch.int16))
        # the same exchange inside the GEMM kernel: the epilogue stores every tile into the peers' buffers too
        for _ in range(2):
            shared.local.zero_()
            got = shard.matmul_into_all(shared, rows, da, dw.t())
            torch.cuda.synchronize()
            ok = ok and torch.equal(got.view(torch.int16), whole.view(torch.int16))
        ok = ok and tb.device_errors() == 0
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_produce_and_gather_on_two_gpus():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
