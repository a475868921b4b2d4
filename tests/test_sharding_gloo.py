"""Multi-rank host logic on CPU: two gloo ranks shard a frontier, min-reduce the round's lower bound
and rebalance uneven shards.  Nothing here touches a GPU; a rank's 'bounds' are synthetic numbers."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist

    from ny_b200 import SPLIT_DTYPE, sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # 1. sharding covers the batch exactly once
        first, count = sharding.shard_bounds(4097, world, rank)
        # 2. global lower bound
        local_min = torch.tensor([3.5 - 2.0 * rank])
        sharding.allreduce_min(local_min, dist)
        # 3. rebalancing: rank 0 holds 10 domains, rank 1 holds 2
        n_local = 10 if rank == 0 else 2
        splits = np.zeros((n_local, 3), SPLIT_DTYPE)
        splits["relu"] = rank
        splits["neuron"] = np.arange(n_local)[:, None] * 10 + np.arange(3)[None, :]
        splits["sign"] = 1 - 2 * rank
        splits["beta"] = 0.25 * (rank + 1)
        ns = np.full(n_local, 3, np.int32)
        ns[0] = 1
        s2, n2 = sharding.exchange_domains(splits, ns, dist)
        again = sharding.exchange_domains(s2, n2, dist)  # already level: no movement
        ret[rank] = dict(first=first, count=count, gmin=float(local_min), n=len(n2),
                         keys=sorted((int(a["relu"][0]), int(a["neuron"][0]), int(c)) for a, c in zip(s2, n2)),
                         beta=sorted(float(a["beta"][0]) for a in s2), stable=len(again[1]) == len(n2))
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_reduce_and_rebalance():
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        r0, r1 = ret[0], ret[1]
    assert (r0["first"], r0["count"]) == (0, 2049) and (r1["first"], r1["count"]) == (2049, 2048)
    assert r0["gmin"] == r1["gmin"] == 1.5
    assert r0["n"] == 6 and r1["n"] == 6 and r0["stable"] and r1["stable"]
    all_keys = sorted(r0["keys"] + r1["keys"])
    expect = sorted([(0, i * 10, 1 if i == 0 else 3) for i in range(10)] + [(1, i * 10, 1 if i == 0 else 3) for i in range(2)])
    assert all_keys == expect  # every domain record survived the move exactly once
    assert r1["beta"].count(0.25) == 4 and r1["beta"].count(0.5) == 2


def test_rebalance_plan_properties():
    from ny_b200.sharding import plan_rebalance, shard_bounds

    assert plan_rebalance([5, 5, 5, 5]) == []
    assert plan_rebalance([6, 5, 5, 4]) == []          # within the 1.25 trigger
    for counts in ([100, 0, 0, 0], [7, 1, 9, 3, 0, 0, 20, 1], [0, 0, 3]):
        plan = plan_rebalance(counts)
        c = list(counts)
        for s, d, n in plan:
            assert n > 0 and c[s] >= n
            c[s] -= n
            c[d] += n
        assert sum(c) == sum(counts) and max(c) - min(c) <= 1
    tot = 0
    for r in range(8):
        f, n = shard_bounds(1003, 8, r)
        assert f == tot
        tot += n
    assert tot == 1003
