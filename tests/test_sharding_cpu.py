"""CPU: the multi-GPU host logic -- shard ranges and the cross-rank reductions -- with two `gloo` ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_bounds_partition_the_batch(pkg):
    from cvcuda_b200 import sharding
    for n in (0, 1, 7, 128, 256, 1000, 1024):
        for world in (1, 2, 3, 4, 8):
            b = sharding.all_bounds(n, world)
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            sizes = [e - s for s, e in b]
            assert max(sizes) - min(sizes) <= 1 and sum(sizes) == n
    assert sharding.all_bounds(1024, 8) == [(i * 128, (i + 1) * 128) for i in range(8)]
    with pytest.raises(ValueError):
        sharding.shard_bounds(10, 2, 2)


def _worker(rank, world, port, root, results):
    import sys
    sys.path.insert(0, root)
    import __graft_entry__ as ge
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ge.load_package()
        from cvcuda_b200 import sharding
        items = list(range(101))
        mine = sharding.shard_list(items, world, rank)
        # every sample lands on exactly one rank
        total = sharding.sum_over_ranks(len(mine))
        checksum = sharding.sum_over_ranks(sum(mine))
        # the job is as slow as its slowest rank
        slowest = sharding.max_over_ranks(10.0 * (rank + 1))
        rate = sharding.aggregate_throughput(len(mine), 10.0 * (rank + 1))
        results[rank] = (len(mine), total, checksum, slowest, rate)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks(built):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, root, results), nprocs=2, join=True)
    assert results[0][0] + results[1][0] == 101 and abs(results[0][0] - results[1][0]) <= 1
    for r in (0, 1):
        _, total, checksum, slowest, rate = results[r]
        assert total == 101 and checksum == sum(range(101)) and slowest == 20.0
        assert rate == pytest.approx(101 / 0.020)
