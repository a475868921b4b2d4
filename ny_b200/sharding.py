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


def exchange_domains(splits: np.ndarray, n_splits: np.ndarray, dist, device="cpu", trigger: float = 1.25,
                     alpha: np.ndarray | None = None, stats: dict | None = None, counts=None):
    """Rebalances the local frontier (splits [D, max_splits], n_splits [D]) across ranks.  Domains leave
    from the end of the local arrays and arrive appended.  Returns the new (splits, n_splits), or
    (splits, n_splits, alpha) when `alpha` ([D, n_pre] warm-start slopes; the split multipliers already live in
    the records) is given: the slopes travel in the same message as the records they belong to, so a moved
    domain starts on its new rank exactly as it would have on the old one.  Every rank must pass `alpha` or none
    of them.  `stats` accumulates exchanges, records_moved and bytes_moved (this rank's sends and receives);
    `counts` may carry the already gathered shard sizes."""
    import torch

    rank = dist.get_rank()
    if counts is None:
        counts = gather_counts(len(n_splits), dist, device)
    plan = plan_rebalance(counts, trigger)
    max_splits = splits.shape[1]
    n_al = 0 if alpha is None else int(alpha.shape[1])
    rec = max_splits * 4 + 1 + n_al  # int32 words per domain: the split records, the count, the slopes' bit patterns
    for src, dst, n in plan:
        if rank == src:
            keep = len(n_splits) - n
            parts = [splits[keep:].view(np.int32).reshape(n, max_splits * 4), n_splits[keep:].astype(np.int32).reshape(n, 1)]
            if n_al:
                parts.append(np.ascontiguousarray(alpha[keep:], np.float32).view(np.int32))
            buf = np.concatenate(parts, axis=1)
            dist.send(torch.from_numpy(np.ascontiguousarray(buf)).to(device), dst)
            splits, n_splits = splits[:keep], n_splits[:keep]
            if n_al:
                alpha = alpha[:keep]
        elif rank == dst:
            t = torch.empty((n, rec), dtype=torch.int32, device=device)
            dist.recv(t, src)
            buf = t.cpu().numpy()
            got = np.ascontiguousarray(buf[:, : max_splits * 4]).view(SPLIT_DTYPE).reshape(n, max_splits)
            splits = np.concatenate([splits, got], axis=0)
            n_splits = np.concatenate([n_splits, buf[:, max_splits * 4].astype(np.int32)])
            if n_al:
                alpha = np.concatenate([alpha, np.ascontiguousarray(buf[:, max_splits * 4 + 1:]).view(np.float32)], axis=0)
        if stats is not None and rank in (src, dst):
            stats["records_moved"] = stats.get("records_moved", 0) + n
            stats["bytes_moved"] = stats.get("bytes_moved", 0) + n * rec * 4
    if stats is not None and plan:
        stats["exchanges"] = stats.get("exchanges", 0) + 1
    if alpha is not None:
        return splits, n_splits, alpha
    return splits, n_splits


def exchange_resident(frontier, max_depth: int, counts, dist, device, trigger: float = 1.25, stats: dict | None = None):
    """Levels device-resident frontiers (one per rank) after `counts` (every rank's open domains, already gathered).
    `frontier` offers frontier_take(n, splits_address, counts_address) -> taken and frontier_give(n, splits_address,
    counts_address) over arrays on `device` (ny_b200.engine.B200Engine does, over the GPU's memory).  A move is one
    point-to-point message of int32 words, [n, 4 * max_depth + 1] (the split records, then the history length), device
    tensor to device tensor: nothing is staged through the host.  Returns the plan that ran."""
    import torch

    rank = dist.get_rank()
    plan = plan_rebalance(counts, trigger)
    words = 4 * max_depth
    for src, dst, n in plan:
        if rank == src:
            sp = torch.empty((n, words), dtype=torch.int32, device=device)
            ns = torch.empty((n,), dtype=torch.int32, device=device)
            taken = frontier.frontier_take(n, sp.data_ptr(), ns.data_ptr())
            if taken != n:
                raise RuntimeError(f"rank {rank} holds {taken} of the {n} domains the plan moves")
            dist.send(torch.cat([sp, ns[:, None]], dim=1).contiguous(), dst)
        elif rank == dst:
            msg = torch.empty((n, words + 1), dtype=torch.int32, device=device)
            dist.recv(msg, src)
            sp, ns = msg[:, :words].contiguous(), msg[:, words].contiguous()
            if msg.is_cuda:
                torch.cuda.current_stream(msg.device).synchronize()   # the arrays are complete before the engine reads them
            frontier.frontier_give(n, sp.data_ptr(), ns.data_ptr())
        if stats is not None and rank in (src, dst):
            stats["records_moved"] = stats.get("records_moved", 0) + n
            stats["bytes_moved"] = stats.get("bytes_moved", 0) + n * (words + 1) * 4
    if stats is not None and plan:
        stats["exchanges"] = stats.get("exchanges", 0) + 1
    return plan
