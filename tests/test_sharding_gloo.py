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


def _worker_alpha(rank, world, port, ret):
    import torch.distributed as dist

    from ny_b200 import SPLIT_DTYPE, bab, sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_pre = 7
        n_local = 9 if rank == 0 else 1
        fr = bab.Frontier(n_pre)
        splits = np.zeros((n_local, 2 + rank), SPLIT_DTYPE)          # the ranks' histories differ in depth
        splits["neuron"] = 100 * rank + np.arange(n_local)[:, None]
        ns = np.full(n_local, 2 + rank, np.int32)
        alpha = (1000.0 * rank + np.arange(n_local)[:, None] + 0.125 * np.arange(n_pre)[None, :]).astype(np.float32)
        fr.push(splits, ns, alpha)
        stats = {}
        bab._rebalance(fr, dist, "cpu", sharding, stats)
        n_after = len(fr)
        bab._rebalance(fr, dist, "cpu", sharding, stats)              # level now: the early return, nothing popped
        sp, n2, al = fr.pop(len(fr))
        ret[rank] = dict(n=n_after, depth=int(sp.shape[1]), has_alpha=al is not None, stats=dict(stats),
                         pairs=[(int(sp[d, 0]["neuron"]), float(al[d, 0]), float(al[d, 6])) for d in range(len(n2))])
    finally:
        dist.destroy_process_group()


def test_rebalance_moves_warm_start_slopes_with_their_records():
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_alpha, args=(world, port, ret), nprocs=world, join=True)
        r0, r1 = ret[0], ret[1]
    assert r0["n"] == 5 and r1["n"] == 5 and r0["has_alpha"] and r1["has_alpha"]
    assert r0["depth"] == 2 and r1["depth"] == 3      # pop() trims to the deepest history it returns
    # every record still carries the slopes it was created with: alpha[d, 0] = 1000 * rank + index = its neuron tag
    for r in (r0, r1):
        for neuron, a0, a6 in r["pairs"]:
            rank_of, idx = divmod(neuron, 100)
            assert a0 == 1000.0 * rank_of + idx and a6 == a0 + 0.75
    assert sorted(p[0] for p in r0["pairs"] + r1["pairs"]) == list(range(9)) + [100]
    rec_words = 3 * 4 + 1 + 7
    for r in (r0, r1):
        assert r["stats"] == {"records_moved": 4, "bytes_moved": 4 * rec_words * 4, "exchanges": 1}


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


class _OracleEngine:
    """Stand-in for the device engine in the sharded-search test: the same calls, answered by the CPU oracle (test
    infrastructure; the product path never does this).  Root bounds are the interval pass's, branching is the
    intercept score on the constrained-forward bounds."""

    def __init__(self, oracle, net):
        self.o = oracle
        self.onet = oracle.Net(net.weights, net.biases)
        self.bounded = 0

    def _with(self, spec):
        self.ospec = self.onet.with_spec(np.asarray(spec, np.float32))
        self.S = len(spec)

    def pgd_attack(self, net_id, spec, lo, hi, x0, steps, step):
        return np.full(len(x0), np.inf, np.float32), np.asarray(x0, np.float32), -1

    def crown_bounds(self, net_id, spec, lo, hi):
        self._with(spec)
        rl, ru = self.o.ibp_forward(self.ospec, lo, hi)
        cl, cu = self.o.crown(self.ospec, lo, hi)
        return cl[None].astype(np.float32), cu[None].astype(np.float32), rl[None, : -self.S], ru[None, : -self.S]

    def batch_upload(self, net_id, spec, lo, hi, inh_lo, inh_hi, splits, ns, mode=1, alpha=None):
        self._with(spec)
        self._b = (lo, hi, np.concatenate([inh_lo, np.full(self.S, -np.inf, np.float32)]),
                   np.concatenate([inh_hi, np.full(self.S, np.inf, np.float32)]), splits.copy(), ns.copy())

    def batch_run(self):
        lo, hi, il, iu, splits, ns = self._b
        self._r = self.o.bab_bound_batch(self.ospec, lo, hi, il, iu, splits, ns, 1)[:3]
        self.bounded += len(ns)

    def batch_download(self):
        return self._r

    def batch_select_branch(self, kind):
        lo, hi, il, iu, splits, ns = self._b
        relu, neuron = np.full(len(ns), -1, np.int32), np.full(len(ns), -1, np.int32)
        for d in range(len(ns)):
            pl, pu, bad = self.o.domain_bounds(self.ospec, lo, hi, il, iu, splits[d][: ns[d]], 1)
            pick = None if bad else self.o.select_intercept(self.ospec, pl, pu, splits[d][: ns[d]])
            if pick is not None:
                relu[d], neuron[d] = pick[0], pick[1]
        return relu, neuron, np.zeros(len(ns), np.float32)


def _search_problem():
    from ny_b200 import formats
    from ny_b200 import workloads as W

    wl = W.config_mlp_bab(seed=84, hidden=12, depth=2, n_in=3, n_out=3, eps=0.15, n_fix=0)
    mn = W.sample_min_margin(wl, 100000, 3)
    return wl, mn, formats


def _search_worker(rank, world, port, ret):
    import torch.distributed as dist

    from ny_b200 import bab
    from oracle import ny_oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl, mn, formats = _search_problem()
        eng = _OracleEngine(ny_oracle, wl.net)
        eng._with(wl.spec)
        root = ny_oracle.crown(eng.ospec, wl.in_lo, wl.in_hi)[0]
        s = int(np.argmax(mn - root))
        t = float(root[s] + 0.4 * (mn[s] - root[s]))
        prop = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], t)]])
        r = bab.verify(eng, 0, wl.net, prop, batch=2, max_rounds=400, dist=dist if world > 1 else None)
        ret[rank] = dict(status=r.status, rounds=r.rounds, bounded=r.domains_bounded, local=eng.bounded, open=r.open_domains)
    finally:
        if world > 1:
            dist.destroy_process_group()


def test_sharded_search_reaches_the_single_rank_verdict():
    """The branch-and-bound loop over two gloo ranks (bounds from the CPU oracle in place of the device): same
    verdict as one rank, both ranks do part of the work, and the ranks agree on the counters."""
    import torch.multiprocessing as mp

    with mp.Manager() as mgr:
        ret = mgr.dict()
        _search_worker(0, 1, 0, ret)
        single = dict(ret[0])
        port = _free_port()
        mp.spawn(_search_worker, args=(2, port, ret), nprocs=2, join=True)
        r0, r1 = dict(ret[0]), dict(ret[1])
    assert single["status"] == "verified" and single["bounded"] > 8, single
    assert r0["status"] == r1["status"] == "verified"
    assert r0["rounds"] == r1["rounds"] and r0["bounded"] == r1["bounded"] and r0["open"] == r1["open"] == 0
    assert r0["local"] > 0 and r1["local"] > 0                     # the frontier really was shared out
    assert r0["local"] + r1["local"] == r0["bounded"] - 1          # every domain bounded once (+ the root bound)
    assert r0["rounds"] < single["rounds"]                         # two shards per round: fewer rounds


class _HostRing:
    """Stand-in for the engine's device frontier with the same take / give contract over host memory: records leave
    from the back and arrive at the back, arrays are passed by address."""

    def __init__(self, records, lengths, max_depth):
        self.max_depth = max_depth
        self.rec = [np.array(r, np.int32).reshape(4 * max_depth) for r in records]
        self.len = [int(n) for n in lengths]

    def frontier_take(self, n, sp_addr, ns_addr):
        import ctypes

        n = min(n, len(self.rec))
        if n:
            sp = np.stack(self.rec[len(self.rec) - n:])
            ns = np.array(self.len[len(self.len) - n:], np.int32)
            ctypes.memmove(sp_addr, sp.ctypes.data, sp.nbytes)
            ctypes.memmove(ns_addr, ns.ctypes.data, ns.nbytes)
            del self.rec[len(self.rec) - n:], self.len[len(self.len) - n:]
        return n

    def frontier_give(self, n, sp_addr, ns_addr):
        import ctypes

        sp = np.empty((n, 4 * self.max_depth), np.int32)
        ns = np.empty(n, np.int32)
        ctypes.memmove(sp.ctypes.data, sp_addr, sp.nbytes)
        ctypes.memmove(ns.ctypes.data, ns_addr, ns.nbytes)
        self.rec += [r.copy() for r in sp]
        self.len += [int(x) for x in ns]


def _worker_resident(rank, world, port, ret):
    import torch.distributed as dist

    from ny_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        depth = 5
        n_local = 11 if rank == 0 else 0      # the state after the first rounds of a search: rank 0 holds everything
        recs = [np.full(4 * depth, 1000 * rank + i, np.int32) for i in range(n_local)]
        ring = _HostRing(recs, [1 + i % depth for i in range(n_local)], depth)
        stats = {}
        counts = sharding.gather_counts(len(ring.rec), dist)
        plan = sharding.exchange_resident(ring, depth, counts, dist, "cpu", stats=stats)
        counts2 = sharding.gather_counts(len(ring.rec), dist)
        plan2 = sharding.exchange_resident(ring, depth, counts2, dist, "cpu", stats=stats)   # level: nothing moves
        ret[rank] = dict(plan=plan, plan2=plan2, n=len(ring.rec), ids=[int(r[0]) for r in ring.rec], lens=list(ring.len),
                         whole=all(np.all(r == r[0]) for r in ring.rec), stats=stats)
    finally:
        dist.destroy_process_group()


def test_two_ranks_level_resident_frontiers_by_address():
    """The levelling of device-resident frontiers (records taken from one ring and given to another, array addresses
    in, one message per move) with a host-memory stand-in for the ring."""
    import torch.multiprocessing as mp

    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_resident, args=(world, port, ret), nprocs=world, join=True)
        r0, r1 = ret[0], ret[1]
    assert r0["plan"] == r1["plan"] == [(0, 1, 5)] and r0["plan2"] == r1["plan2"] == []
    assert (r0["n"], r1["n"]) == (6, 5)
    assert r0["ids"] == list(range(6)) and r1["ids"] == list(range(6, 11))   # the back of rank 0's ring moved, in order
    assert r1["lens"] == [1 + i % 5 for i in range(6, 11)] and r0["whole"] and r1["whole"]
    assert r0["stats"] == r1["stats"] == {"records_moved": 5, "bytes_moved": 5 * 21 * 4, "exchanges": 1}
