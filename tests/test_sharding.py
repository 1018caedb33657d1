"""Host-side logic of the multi-GPU path on CPU: two gloo ranks shard a batch by image, reduce
their times with max and gather results on rank 0 in image order."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from smallframework_b200 import sharding


def test_shard_ranges_partition_the_batch():
    for total in (0, 1, 7, 64, 512, 4097):
        for world in (1, 2, 3, 4, 8):
            r = [sharding.shard_range(total, world, k) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == total
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in r]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.shard_range(512, 8, 3) == (192, 256)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def _worker(rank, world, port, total, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, e = sharding.shard_range(total, world, rank)
        # stand-in for the per-image result of the layer chain: a function of the image index
        local = torch.arange(b, e, dtype=torch.float32)[:, None] * torch.tensor([[1.0, 10.0, 100.0]])
        t = sharding.max_over_ranks(1.0 + rank)
        full = sharding.gather_to_host(local, total)
        dist.barrier()
        if rank == 0:
            np.save(out_path, np.concatenate([[t], full.numpy().ravel()]))
        else:
            assert full is None
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo(tmp_path):
    total, world = 9, 2
    out = str(tmp_path / "gathered.npy")
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, total, out), nprocs=world, join=True)
    data = np.load(out)
    assert data[0] == 2.0  # max over ranks of (1 + rank)
    want = (np.arange(total, dtype=np.float32)[:, None] * np.array([[1.0, 10.0, 100.0]])).ravel()
    assert np.array_equal(data[1:], want)
