"""Host-side logic of the batch-sharded multi-GPU path, run as two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hingetreefortorch_b200 import distributed as htd


def test_shard_bounds_cover_every_row_once():
    for rows in (0, 1, 7, 8, 1048576, 100):
        for world in (1, 2, 3, 4, 8):
            bounds = [htd.shard_bounds(rows, r, world) for r in range(world)]
            assert bounds[0][0] == 0 and bounds[-1][1] == rows
            for (lo, hi), (lo2, hi2) in zip(bounds, bounds[1:]):
                assert hi == lo2 and 0 <= hi - lo - (hi2 - lo2) <= 1
    with pytest.raises(ValueError):
        htd.shard_bounds(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        full = torch.arange(10 * 3, dtype=torch.float32).view(10, 3)
        mine = htd.shard_rows(full)
        # a stand-in "model": parameters whose gradients depend on the rank's rows only
        thr = torch.nn.Parameter(torch.zeros(4, 7))
        w = torch.nn.Parameter(torch.zeros(4, 8, 2))
        ords = torch.nn.Parameter(torch.zeros(4, 7, dtype=torch.long), requires_grad=False)
        thr.grad = torch.full_like(thr, float(mine.sum()))
        w.grad = None if rank == 1 else torch.ones_like(w)  # a missing gradient counts as zero
        bucket = htd.GradientBucket([thr, w, ords])
        assert bucket.nbytes == 4 * (28 + 64)
        bucket.all_reduce()
        gathered = htd.gather_rows(mine * 2, full.shape[0])
        results[rank] = (thr.grad.clone(), w.grad.clone(), gathered, tuple(mine.shape))
    finally:
        dist.destroy_process_group()


def test_two_rank_gradient_bucket_and_row_gather():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    full = torch.arange(10 * 3, dtype=torch.float32).view(10, 3)
    for rank in range(world):
        thr_grad, w_grad, gathered, shape = results[rank]
        assert shape == (5, 3)
        assert torch.equal(thr_grad, torch.full((4, 7), float(full.sum())))   # sum over both shards
        assert torch.equal(w_grad, torch.ones(4, 8, 2))                       # 1 (rank 0) + 0 (rank 1)
        assert torch.equal(gathered, full * 2)
