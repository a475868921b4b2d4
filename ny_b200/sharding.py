"""Multi-GPU driver logic for a sharded BaB frontier (one process per GPU).

Domains are independent, so every rank bounds its own shard with no data-path collective.  The only
exchanges are (1) the per-round min-reduce of the global lower bound and (2) rebalancing when pruning
and branching leave the shards uneven: counts are all-gathered, a deterministic plan is computed on
every rank, and split records move with point-to-point send/recv into local buffers (a peer's memory is
never an operand of a kernel).  The same code runs over NCCL (GPU tensors) and gloo (CPU tensors).
"""
from __future__ import annotations

import numpy as np

from .engine import SPLIT_DTYPE


def shard_bounds(n_total: int, world: int, rank: int):
    """Contiguous balanced shard of range(n_total): returns (first, count)."""
    base, rem = divmod(n_total, world)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def plan_rebalance(counts, trigger: float = 1.25):
    """Moves [(src, dst, n), ...] that level `counts` to within one domain of each other.  Returns []
    when max(counts) <= trigger * mean(counts).  Deterministic, so every rank derives the same plan."""
    counts = [int(c) for c in counts]
    world = len(counts)
    total = sum(counts)
    if world < 2 or total == 0 or max(counts) <= trigger * (total / world):
        return []
    target = [total // world + (1 if r < total % world else 0) for r in range(world)]
    surplus = [[r, counts[r] - target[r]] for r in range(world) if counts[r] > target[r]]
    deficit = [[r, target[r] - counts[r]] for r in range(world) if counts[r] < target[r]]
    plan = []
    i = j = 0
    while i < len(surplus) and j < len(deficit):
        n = min(surplus[i][1], deficit[j][1])
        plan.append((surplus[i][0], deficit[j][0], n))
        surplus[i][1] -= n
        deficit[j][1] -= n
        if surplus[i][1] == 0:
            i += 1
        if deficit[j][1] == 0:
            j += 1
    return plan


def allreduce_min(tensor, dist=None):
    """In-place MIN all-reduce of a 1-element tensor (the round's global lower bound)."""
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.MIN)
    return tensor


def gather_counts(n_local: int, dist, device="cpu"):
    import torch

    world = dist.get_world_size()
    mine = torch.tensor([n_local], dtype=torch.int64, device=device)
    out = [torch.zeros(1, dtype=torch.int64, device=device) for _ in range(world)]
    dist.all_gather(out, mine)
    return [int(t.item()) for t in out]


def exchange_domains(splits: np.ndarray, n_splits: np.ndarray, dist, device="cpu", trigger: float = 1.25):
    """Rebalances the local frontier (splits [D, max_splits], n_splits [D]) across ranks.  Domains leave
    from the end of the local arrays and arrive appended.  Returns the new (splits, n_splits)."""
    import torch

    rank = dist.get_rank()
    counts = gather_counts(len(n_splits), dist, device)
    plan = plan_rebalance(counts, trigger)
    max_splits = splits.shape[1]
    rec = max_splits * 4 + 1  # int32 words per domain: the split records and the count
    for src, dst, n in plan:
        if rank == src:
            keep = len(n_splits) - n
            buf = np.concatenate([splits[keep:].view(np.int32).reshape(n, max_splits * 4),
                                  n_splits[keep:].astype(np.int32).reshape(n, 1)], axis=1)
            dist.send(torch.from_numpy(np.ascontiguousarray(buf)).to(device), dst)
            splits, n_splits = splits[:keep], n_splits[:keep]
        elif rank == dst:
            t = torch.empty((n, rec), dtype=torch.int32, device=device)
            dist.recv(t, src)
            buf = t.cpu().numpy()
            got = np.ascontiguousarray(buf[:, : max_splits * 4]).view(SPLIT_DTYPE).reshape(n, max_splits)
            splits = np.concatenate([splits, got], axis=0)
            n_splits = np.concatenate([n_splits, buf[:, -1].astype(np.int32)])
    return splits, n_splits
