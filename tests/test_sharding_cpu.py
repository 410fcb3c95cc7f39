"""Host-side sharding logic on CPU: shard boundaries and the world_size-2 gloo gather."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mircuda_b200 import sharding


def test_column_shards_cover_and_align():
    for n, world in [(6144, 8), (4096, 8), (24576, 8), (4096, 3), (300, 4), (100, 8), (129, 2)]:
        cursor = 0
        for rank in range(world):
            begin, end = sharding.column_shard(n, world, rank)
            assert begin == cursor and end >= begin
            assert begin % 128 == 0 or begin == n          # no scale atom is split
            cursor = end
        assert cursor == n
    with pytest.raises(ValueError):
        sharding.column_shard(128, 2, 2)


def _worker(rank, world, port, n, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k = 5, 64
        generator = torch.Generator().manual_seed(0)
        x = torch.randn(m, k, generator=generator)
        w = torch.randn(n, k, generator=generator)
        begin, end = sharding.column_shard(n, world, rank)
        local = x @ w[begin:end].T                         # this rank's [M, N_r] columns
        full = sharding.gather_columns(local)
        ok = torch.allclose(full, x @ w.T, atol=1e-5)
        results[rank] = bool(ok) and tuple(full.shape) == (m, n)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [256, 300])
def test_gather_columns_two_ranks_gloo(n):
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, n, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}
