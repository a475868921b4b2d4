"""Branch-and-bound driver over the engine's batch calls: the caller side of the bound-propagation path.

Mirrors the loop of the reference's BetaCrownVerifier (crates/ny-propagate/src/beta_crown/engine/core.rs:492-735):
attack first (a counterexample ends the run), bound the root, then repeatedly pop a batch of open domains, bound
them on the device with their split constraints, drop the ones whose bound proves the property, pick a branching
neuron for the rest and push both children.  Statuses follow BabVerificationStatus (beta_crown/result.rs): verified,
violated (with a counterexample that was evaluated by an independent concrete forward pass), unknown, timeout.

The property is the violation region in disjunctive normal form (formats.Property): clauses of atoms
`c . y + d >= 0`.  An atom is refuted on a domain when the lower bound of `-c . y` exceeds `d`; a clause is refuted
when one of its atoms is; a domain is verified when every clause is refuted.
"""
from __future__ import annotations

import json
import os
import sys
import time
from dataclasses import dataclass

import numpy as np

from .engine import SPLIT_DTYPE
from .formats import Property
from .workloads import forward


@dataclass
class VerifyResult:
    status: str                      # "verified" | "violated" | "unknown" | "timeout"
    counterexample: np.ndarray | None = None
    output: np.ndarray | None = None
    rounds: int = 0
    domains_bounded: int = 0
    open_domains: int = 0
    root_lower: np.ndarray | None = None
    exchange: dict | None = None     # multi-rank runs: this rank's rebalancing traffic (exchanges, records_moved, bytes_moved)


def _rows(prop: Property):
    spec, thr, owner = [], [], []
    for ci, clause in enumerate(prop.violation):
        for atom in clause:
            spec.append(-np.asarray(atom.c, np.float32))
            # the clause is refuted when lower > d in real arithmetic: the fp32 threshold may only round upwards
            t32 = np.float32(atom.d)
            if float(t32) < float(atom.d):
                t32 = np.nextafter(t32, np.float32(np.inf))
            thr.append(t32)
            owner.append(ci)
    return np.stack(spec).astype(np.float32), np.array(thr, np.float32), np.array(owner, np.int32)


def _violates(prop: Property, y: np.ndarray) -> bool:
    """Is the concrete output y inside the violation region (some clause with all atoms true)?"""
    y = np.asarray(y, np.float64)
    return any(all(float(np.dot(a.c.astype(np.float64), y)) + a.d >= 0.0 for a in clause) for clause in prop.violation)


def _verified_mask(lower: np.ndarray, thr: np.ndarray, owner: np.ndarray, n_clauses: int) -> np.ndarray:
    """lower [D, S]: per domain, is every clause refuted by at least one of its atoms (strict, finite)?"""
    refuted = np.isfinite(lower) & (lower > thr[None, :])
    ok = np.ones(lower.shape[0], bool)
    for c in range(n_clauses):
        ok &= refuted[:, owner == c].any(axis=1)
    return ok


def frontier_to_arrays(frontier):
    """Structure-of-arrays form of a list of split histories: (splits [N, depth], n_splits [N])."""
    depth = max([1] + [len(s) for s in frontier])
    splits = np.zeros((len(frontier), depth), SPLIT_DTYPE)
    ns = np.zeros(len(frontier), np.int32)
    for d, s in enumerate(frontier):
        splits[d, : len(s)] = s
        ns[d] = len(s)
    return splits, ns


class Frontier:
    """The open domain set as blocks of structure-of-arrays records: split histories [n, depth] with their lengths
    [n] and, optionally, warm-start slopes [n, n_pre].  Batches leave from the front, children are appended at the
    back (breadth-first); nothing is copied when a block is appended."""

    def __init__(self, n_pre: int):
        from collections import deque

        self.blocks = deque()     # (splits, ns, alpha or None)
        self.n = 0
        self.n_pre = n_pre

    def __len__(self):
        return self.n

    def push(self, splits, ns, alpha=None):
        if len(ns) == 0:
            return
        splits = np.asarray(splits, SPLIT_DTYPE).reshape(len(ns), -1)
        self.blocks.append((splits, np.asarray(ns, np.int32), None if alpha is None else np.asarray(alpha, np.float32)))
        self.n += len(ns)

    def push_front(self, splits, ns):
        if len(ns) == 0:
            return
        splits = np.asarray(splits, SPLIT_DTYPE).reshape(len(ns), -1)
        self.blocks.appendleft((splits, np.asarray(ns, np.int32), None))
        self.n += len(ns)

    def pop(self, n: int):
        """The first n domains: (splits [n, depth of the deepest], ns [n], alpha [n, n_pre], or None unless every one
        of them has warm-start slopes)."""
        parts, got = [], 0
        while self.blocks and got < n:
            sp, ns, al = self.blocks.popleft()
            take = min(n - got, len(ns))
            if take < len(ns):
                self.blocks.appendleft((sp[take:], ns[take:], None if al is None else al[take:]))
            parts.append((sp[:take], ns[:take], None if al is None else al[:take]))
            got += take
        self.n -= got
        if not parts:
            return np.zeros((0, 1), SPLIT_DTYPE), np.zeros(0, np.int32), None
        ns = np.concatenate([p[1] for p in parts])
        depth = max(1, int(ns.max()))
        splits = np.zeros((got, depth), SPLIT_DTYPE)
        row = 0
        for sp, n_, _ in parts:
            w = min(depth, sp.shape[1])
            splits[row: row + len(n_), :w] = sp[:, :w]
            row += len(n_)
        alpha = None if any(p[2] is None for p in parts) else np.concatenate([p[2] for p in parts])
        return splits, ns, alpha

    def arrays(self):
        """Everything as two arrays (splits [N, deepest], ns [N]); the warm-start slopes are dropped."""
        return self.pop(self.n)[:2] if self.n else (np.zeros((0, 1), SPLIT_DTYPE), np.zeros(0, np.int32))

    def as_list(self):
        splits, ns = self.arrays()
        self.push(splits, ns)
        return [splits[d, : ns[d]].copy() for d in range(len(ns))]


def make_children(splits, ns, open_idx, relu, neuron, beta=None):
    """Both children of every open domain, in the order (d0 active, d0 inactive, d1 active, ...): the parent's history
    with the new split appended (multiplier 0); `beta` [D, depth] replaces the parents' multipliers.  Works on the
    records as rows of four 32-bit words (relu, neuron, sign, multiplier bits)."""
    k = len(open_idx)
    open_idx = np.asarray(open_idx, np.int64)
    n_par = ns[open_idx].astype(np.int64)
    depth = int(n_par.max()) + 1 if k else 1
    words = np.ascontiguousarray(splits).view(np.int32).reshape(splits.shape[0], splits.shape[1], 4)
    w = min(depth, splits.shape[1])
    par = words[open_idx, :w].copy()                                     # [k, w, 4]
    if beta is not None:
        bw = min(w, beta.shape[1])
        par[:, :bw, 3] = np.ascontiguousarray(beta[open_idx, :bw], np.float32).view(np.int32)
    par *= (np.arange(w)[None, :] < n_par[:, None])[:, :, None]          # records past a history's end are zero
    out = np.zeros((2 * k, depth, 4), np.int32)
    out[0::2, :w] = par
    out[1::2, :w] = par
    rows = np.arange(k)
    out[2 * rows, n_par, 0] = out[2 * rows + 1, n_par, 0] = relu[open_idx]
    out[2 * rows, n_par, 1] = out[2 * rows + 1, n_par, 1] = neuron[open_idx]
    out[2 * rows, n_par, 2] = 1
    out[2 * rows + 1, n_par, 2] = -1
    return out.reshape(2 * k, depth * 4).view(SPLIT_DTYPE).reshape(2 * k, depth), np.repeat(n_par + 1, 2).astype(np.int32)

def save_frontier(path, frontier, inh_lo, inh_hi, prop: Property, rounds: int, domains_bounded: int):
    """Dump of the open domain set (the reference's BaB has no checkpoint; its benchmark sweep resumes from metadata,
    lines 203-260 of the reference's README).  One .npz: split histories as structure of arrays, the inherited root bounds, the property's
    box and rows (so that a resume against another property is refused), and the counters."""
    splits, ns = frontier_to_arrays(frontier)
    spec, thr, owner = _rows(prop)
    tmp = str(path) + ".tmp.npz"
    np.savez(tmp, splits=splits, n_splits=ns, inh_lo=inh_lo, inh_hi=inh_hi, in_lo=prop.in_lo, in_hi=prop.in_hi, spec=spec,
             thr=thr, owner=owner, rounds=np.int64(rounds), domains_bounded=np.int64(domains_bounded))
    os.replace(tmp, path)


def load_frontier(path, prop: Property):
    """Inverse of save_frontier: (frontier, inh_lo, inh_hi, rounds, domains_bounded); ValueError when the dump
    belongs to another property."""
    z = np.load(path)
    spec, thr, owner = _rows(prop)
    same = (np.array_equal(z["in_lo"], prop.in_lo) and np.array_equal(z["in_hi"], prop.in_hi)
            and z["spec"].shape == spec.shape and np.array_equal(z["spec"], spec) and np.array_equal(z["thr"], thr)
            and np.array_equal(z["owner"], owner))
    if not same:
        raise ValueError("the frontier dump was written for another property")
    splits, ns = z["splits"].astype(SPLIT_DTYPE), z["n_splits"]
    frontier = [splits[d, : ns[d]].copy() for d in range(len(ns))]
    return frontier, z["inh_lo"], z["inh_hi"], int(z["rounds"]), int(z["domains_bounded"])


class _Metrics:
    """Per-round records as JSON lines (the shape of the reference's GraphDomainBatchMetricsSink records:
    --domain-batch-metrics-jsonl), and with NYB200_PROF=1 a stderr line per round like the reference's NY_ACASXU_PROF
    probe (`explored= ... rate=.../s`, beta_crown/engine/core.rs:372-394)."""

    def __init__(self, path):
        self._f = open(path, "a") if path else None
        self._prof = os.environ.get("NYB200_PROF", "") not in ("", "0")
        self._t0 = time.time()

    def round(self, **rec):
        rec["elapsed_s"] = round(time.time() - self._t0, 6)
        if self._f:
            self._f.write(json.dumps(rec) + "\n")
            self._f.flush()
        if self._prof:
            rate = rec["explored"] / max(rec["elapsed_s"], 1e-9)
            print(f"[nyb200] round={rec['round']} explored={rec['explored']} open={rec['open']} "
                  f"min_lower={rec['min_lower']:.6g} rate={rate:.0f}/s", file=sys.stderr)

    def close(self):
        if self._f:
            self._f.close()


def attack(eng, net_id, net, prop: Property, restarts: int = 256, steps: int = 50, seed: int = 0):
    """PGD on every atom's row from seeded uniform starts; a candidate counts only if an independent concrete forward
    pass (binary64, host) puts it inside the violation region.  Returns (x, y) or None."""
    spec, thr, owner = _rows(prop)
    g = np.random.Generator(np.random.PCG64(seed))
    lo, hi = prop.in_lo, prop.in_hi
    x0 = (lo + g.random((restarts, len(lo)), dtype=np.float32) * (hi - lo)).astype(np.float32)
    x0[0] = lo
    x0[1 % restarts] = hi
    eps = float((hi - lo).max()) / 2
    for s in range(spec.shape[0]):
        best, bx, _ = eng.pgd_attack(net_id, spec[s:s + 1], lo, hi, x0, steps, 0.25 * eps if eps > 0 else 0.0)
        for r in np.argsort(best)[:8]:
            x = np.clip(bx[r], lo, hi)
            y = forward(net, x)
            if _violates(prop, y):
                return x, y
    return None


def fsb_candidates(main, backup, k: int):
    """Candidate neurons of one domain for the filtered heuristic (select_fsb_neuron,
    beta_crown/engine/branching/sequential.rs:200-300): the k largest BaBSR scores, then the k smallest (most
    negative) backup scores that are not among them; non-candidates carry main < 0.  Stable order on ties."""
    cand = np.flatnonzero(main >= 0)
    if cand.size == 0:
        return cand
    by_main = cand[np.argsort(-main[cand], kind="stable")][:k]
    by_backup = cand[np.argsort(backup[cand], kind="stable")][:k]
    seen = set(int(i) for i in by_main)
    return np.array(list(by_main) + [int(i) for i in by_backup if int(i) not in seen], np.int64)


def _margin(lower, thr, owner, n_clauses):
    """Scalar progress of a domain: min over clauses of the best atom's (lower - threshold); > 0 means verified."""
    gap = lower - thr[None, :]
    out = np.full(lower.shape[0], np.inf, np.float32)
    for c in range(n_clauses):
        out = np.minimum(out, gap[:, owner == c].max(axis=1))
    return out


KFSB_REDUCE = {"min": np.minimum, "max": np.maximum, "mean": lambda a, b: (a + b) * np.float32(0.5)}


def kfsb_fallback_index(depth: int, n_candidates: int) -> int:
    """Which candidate a domain takes when none of its trial splits produced a usable score (the random fallback of
    select_kfsb_neuron, beta_crown/engine/branching/sequential.rs:535-552): a deterministic choice keyed by the
    domain's depth.  The reference keys its own by a SipHash of the depth; the key differs, the rule (any candidate
    is a valid split, the same domain always takes the same one) does not."""
    return int((np.uint64(depth) * np.uint64(0x9E3779B97F4A7C15) >> np.uint64(33)) % np.uint64(max(n_candidates, 1)))


def select_fsb(eng, net_id, net, prop: Property, inh_lo, inh_hi, take, open_idx, k: int = 3, reduce: str = "min"):
    """Filtered smart branching (kFSB) for the open domains `open_idx` of the batch `take` that has just been run (and
    scored with BaBSR): every candidate of fsb_candidates is tried - both children bounded in one device batch - and
    the two children's margins are combined by `reduce` (KfsbReduceOp, beta_crown/config/beta_config.rs:1942-1953:
    "min" the worse child - conservative, the default; "max" the better child; "mean" their midpoint;
    sequential.rs:482-507); the best combined score wins, within 1e-6 the larger BaBSR score decides, NaN scores never
    win.  A domain all of whose trials are NaN takes the candidate kfsb_fallback_index names.  Returns
    {domain index: (relu, neuron)}; a domain without candidates is missing from it."""
    if reduce not in KFSB_REDUCE:
        raise ValueError(f"unknown kFSB reduce operator {reduce!r}")
    spec, thr, owner = _rows(prop)
    n_clauses = len(prop.violation)
    main, backup = eng.batch_branch_scores(with_backup=True)
    offs = np.concatenate([[0], np.cumsum(net.dims[1:])]).astype(np.int64)
    trial, meta = [], []          # child split histories; (domain, flat neuron index) per pair of children
    for d in open_idx:
        for o in fsb_candidates(main[d], backup[d], k):
            r = int(np.searchsorted(offs[1:], o, side="right"))
            for sign in (1, -1):
                child = np.zeros(len(take[d]) + 1, SPLIT_DTYPE)
                child[: len(take[d])] = take[d]
                child[-1] = (r, int(o - offs[r]), sign, 0.0)
                trial.append(child)
            meta.append((int(d), int(o), r, int(o - offs[r])))
    if not trial:
        return {}
    splits, ns = frontier_to_arrays(trial)
    lower, _, infeasible = eng.bab_bound_batch(net_id, spec, prop.in_lo, prop.in_hi, inh_lo, inh_hi, splits, ns, mode=1)
    m = _margin(lower, thr, owner, n_clauses)
    m = np.where(infeasible != 0, np.float32(np.inf), m)       # an empty child needs no further work
    with np.errstate(invalid="ignore"):
        score = KFSB_REDUCE[reduce](m[0::2], m[1::2])
    best, tried = {}, {}
    for (d, o, r, j), w in zip(meta, score):
        tried.setdefault(d, []).append((r, j))
        if np.isnan(w):
            continue
        cur = best.get(d)
        if cur is None or w > cur[0] + 1e-6 or (abs(w - cur[0]) <= 1e-6 and main[d][o] > cur[1]):
            best[d] = (float(w), float(main[d][o]), r, j)
    out = {d: (v[2], v[3]) for d, v in best.items()}
    for d, cands in tried.items():
        if d not in out:
            out[d] = cands[kfsb_fallback_index(len(take[d]), len(cands))]
    return out


def verify(eng, net_id, net, prop: Property, *, batch: int = 1024, max_rounds: int = 64, max_domains: int = 1 << 20,
           pgd_restarts: int = 256, pgd_steps: int = 50, optimize_iterations: int = 0, branching: int = 1,
           timeout_s: float | None = None, metrics_jsonl=None, checkpoint=None, resume=None,
           warm_start: bool = True, fsb_k: int = 3, kfsb_reduce: str = "min", refinement: str = "parity", dist=None,
           dist_device="cpu") -> VerifyResult:
    """metrics_jsonl: append one JSON record per round; checkpoint: path that receives the open frontier whenever the
    run stops unresolved (round limit, timeout, domain limit); resume: path of such a dump to continue from (the attack
    and the root bound are skipped).
    batch: domains bounded per device call; optimize_iterations: projected-Adam steps on the slopes and split
    multipliers of every domain (0, the reference's throughput default `beta_iterations: 0`
    (beta_crown/config/beta_config.rs:1244), bounds each domain once with multipliers at zero: sound, but the search
    may then end "unknown" on properties that need the multipliers; 20 is the reference's root-level count);
    branching: 0 widest interval, 1 intercept score, 2 BaBSR, 3 filtered smart branching over the fsb_k best BaBSR and
    intercept candidates, the children's margins combined by kfsb_reduce ("min" | "max" | "mean") (2 and 3: Linear
    layers only); warm_start: with optimisation on, children start from their
    parent's optimised slopes and split multipliers instead of the heuristic slopes and zero.
    refinement: "parity" (every domain whose rounding charge is visible at the engine's tolerance is re-evaluated with
    binary64 contractions) or "verdict" (only the domains whose verdict the charge could change:
    nyb200_batch_set_thresholds; sound, several times faster on narrow boxes, a domain may be split once more).
    dist: an initialised torch.distributed module, one process per GPU: every rank runs this function with the same
    arguments, rank 0 attacks and bounds the root, and from then on every rank bounds its own shard of the frontier;
    per round the ranks exchange one small all-reduce (open domains, stop flags, the global lower bound) and level
    their shards point to point when they drift apart (ny_b200/sharding.py), warm-start slopes travelling with their
    split records.  All ranks return the same status.  No frontier dump is written in a multi-rank run (every rank
    holds only its shard)."""
    from . import sharding

    t0 = time.time()
    if not prop.violation:
        return VerifyResult("verified")
    spec, thr, owner = _rows(prop)
    n_clauses = len(prop.violation)
    world = dist.get_world_size() if dist is not None else 1
    rank = dist.get_rank() if dist is not None else 0
    metrics = _Metrics(metrics_jsonl if rank == 0 else None)
    n_pre = int(net.n_pre)
    frontier = Frontier(n_pre)
    exchange = {"exchanges": 0, "records_moved": 0, "bytes_moved": 0} if world > 1 else None
    res = VerifyResult("unknown")
    root = {"status": "unknown", "inh": None}
    if rank == 0:
        if resume is not None:
            hist, inh_lo, inh_hi, _, b0 = load_frontier(resume, prop)
            frontier.push(*frontier_to_arrays(hist))
            res.domains_bounded = b0                        # max_rounds counts this call's rounds
        else:
            ce = attack(eng, net_id, net, prop, pgd_restarts, pgd_steps)
            if ce is not None:
                res = VerifyResult("violated", ce[0], ce[1])
                root["status"] = "violated"
            else:
                # root: plain CROWN with CROWN-tightened intermediate bounds
                rlo, _, inter_lo, inter_hi = eng.crown_bounds(net_id, spec, prop.in_lo, prop.in_hi)
                res = VerifyResult("unknown", root_lower=rlo[0].copy(), domains_bounded=1)
                if _verified_mask(rlo, thr, owner, n_clauses)[0]:
                    res.status = root["status"] = "verified"
                inh_lo, inh_hi = inter_lo[0], inter_hi[0]
                frontier.push(np.zeros((1, 1), SPLIT_DTYPE), np.zeros(1, np.int32))
        root["bounded"] = res.domains_bounded
        if root["status"] == "unknown":
            root["inh"] = (np.asarray(inh_lo, np.float32), np.asarray(inh_hi, np.float32))
    if world > 1:   # every rank needs the verdict of the root phase and the inherited bounds
        box = [root]
        dist.broadcast_object_list(box, src=0)
        root = box[0]
    if root["status"] != "unknown":
        metrics.close()
        if rank != 0:
            res.status = root["status"]
        return res
    inh_lo, inh_hi = root["inh"]
    res.domains_bounded = root["bounded"]

    def stop(status):
        res.status = status
        res.exchange = exchange
        res.open_domains = len(frontier)
        if checkpoint is not None and len(frontier) and world == 1:
            save_frontier(checkpoint, frontier.as_list(), inh_lo, inh_hi, prop, res.rounds, res.domains_bounded)
        metrics.close()
        return res

    def agree(open_local, flag_local, min_local, bounded_local):
        """(open domains of all ranks, largest stop flag, global lower bound, domains bounded by all ranks this round)"""
        if world == 1:
            return open_local, flag_local, min_local, bounded_local
        import torch

        t = torch.tensor([float(open_local), float(bounded_local)], dtype=torch.float64, device=dist_device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        f = torch.tensor([float(flag_local)], dtype=torch.float64, device=dist_device)
        dist.all_reduce(f, op=dist.ReduceOp.MAX)
        m = torch.tensor([min_local], dtype=torch.float32, device=dist_device)
        sharding.allreduce_min(m, dist)
        return int(t[0].item()), int(f[0].item()), float(m[0].item()), int(t[1].item())

    STUCK, TIMEOUT = 1, 2
    total_open = agree(len(frontier), 0, float("inf"), 0)[0]
    while total_open > 0 and res.rounds < max_rounds:
        flag = TIMEOUT if (timeout_s is not None and time.time() - t0 > timeout_s) else 0
        if world > 1:   # level the shards before the round (also hands the root's first children around)
            _rebalance(frontier, dist, dist_device, sharding, exchange)
        splits, ns, alpha0 = frontier.pop(batch)
        D = len(ns)
        min_lower, n_done, n_inf = float("inf"), 0, 0
        if D and not flag:
            if not (warm_start and optimize_iterations > 1):
                alpha0 = None
            eng.batch_upload(net_id, spec, prop.in_lo, prop.in_hi, inh_lo, inh_hi, splits, ns, mode=1, alpha=alpha0)
            if refinement == "verdict":
                eng.batch_set_thresholds(thr)
            alpha1 = beta1 = None
            if optimize_iterations > 1:
                eng.batch_optimize(optimize_iterations, 0.1, 0.05)
                if warm_start:
                    alpha1, beta1 = eng.batch_download_params()
            else:
                eng.batch_run()
            lower, _, infeasible = eng.batch_download()
            done = _verified_mask(lower, thr, owner, n_clauses) | (infeasible != 0)
            feas = lower[infeasible == 0]
            min_lower = float(feas.min()) if feas.size else float("inf")
            n_done, n_inf = int(done.sum()), int((infeasible != 0).sum())
            open_idx = np.flatnonzero(~done)
            if len(open_idx):
                relu, neuron, _ = eng.batch_select_branch(2 if branching == 3 else branching)
                if branching == 3:   # filtered smart branching: the BaBSR / intercept candidates are tried on the device
                    take = [splits[d, : ns[d]] for d in range(D)]
                    for d, (r, j) in select_fsb(eng, net_id, net, prop, inh_lo, inh_hi, take, open_idx, fsb_k, kfsb_reduce).items():
                        relu[d], neuron[d] = r, j
                if np.any(relu[open_idx] < 0):
                    # every neuron of some domain is fixed and its bound still does not decide it: without a witness the
                    # honest answer is unknown; the undecided domains go back to the front of the queue
                    frontier.push_front(splits[open_idx], ns[open_idx])
                    flag = max(flag, STUCK)
                else:
                    child, child_ns = make_children(splits, ns, open_idx, relu, neuron, beta1)
                    child_alpha = None if alpha1 is None else np.repeat(alpha1[open_idx], 2, axis=0)
                    frontier.push(child, child_ns, child_alpha)
        elif D:
            frontier.push_front(splits, ns)
            D = 0
        total_open, flag, min_lower, bounded = agree(len(frontier), flag, min_lower, D)
        res.rounds += 1
        res.domains_bounded += bounded
        if bounded:
            metrics.round(round=res.rounds, batch=bounded, explored=res.domains_bounded, verified=n_done, infeasible=n_inf,
                          open=total_open, min_lower=min_lower, max_depth=int(ns.max()) if D else 0)
        if flag == TIMEOUT:
            return stop("timeout")
        if flag == STUCK:
            return stop("unknown")
        if total_open > max_domains:
            break
    return stop("verified" if total_open == 0 else "unknown")


def verify_resident(eng, net_id, net, prop: Property, *, batch: int = 1024, max_rounds: int = 64,
                    max_domains: int = 1 << 20, pgd_restarts: int = 256, pgd_steps: int = 50, branching: int = 1,
                    timeout_s: float | None = None, checkpoint=None, resume=None, optimize_iterations: int = 0,
                    refinement: str = "parity", dist=None, dist_device=None) -> VerifyResult:
    """The search of verify() with the open domain set kept on the device (nyb200_frontier_*): attack and root bound
    as there, then one device call per round that pops a batch, bounds it (one bound per domain, multipliers at
    zero), prunes verified and infeasible domains, picks every open domain's split neuron (0 width, 1 intercept,
    2 BaBSR) and appends both children.  Same order of domains as the host loop, hence the same counts and verdicts;
    optimize_iterations > 1: every domain's slopes and multipliers are optimised that many steps and children start
    from their parent's (nyb200_frontier_round_optimized: verify()'s warm-started search; records moved between ranks
    or resumed from a dump start cold).  refinement: "parity" re-evaluates with binary64 contractions every domain
    whose rounding charge is visible at the engine's tolerance (bounds as close to the binary64 path as the per-batch
    calls return them, and the host loop's domain counts); "verdict" only the domains whose verdict the charge could
    change (sound, and several times faster on narrow boxes, where the first rule flags nearly every domain; a domain
    may then be split once more).  What it leaves out is the metrics file.  checkpoint / resume: as in
    verify() (same file format: a dump written by either loop resumes in the other); single rank only.
    dist: an initialised torch.distributed module, one process per GPU, every rank calling with the same arguments:
    each rank keeps its own device frontier (the root starts on rank 0), bounds up to `batch` of its domains per round,
    and the ranks agree per round on the open total and the stop flags with one small all-gather, whose counts also
    drive the levelling of the shards: split records move from one GPU's frontier to another's, device to device
    (sharding.exchange_resident).  All ranks return the same status and the same totals."""
    from . import sharding

    t0 = time.time()
    if not prop.violation:
        return VerifyResult("verified")
    spec, thr, owner = _rows(prop)
    n_clauses = len(prop.violation)
    world = dist.get_world_size() if dist is not None else 1
    rank = dist.get_rank() if dist is not None else 0
    resumed = None
    if resume is not None:
        if world > 1:
            raise ValueError("a frontier dump resumes on a single rank")
        hist, inh_lo, inh_hi, _, b0 = load_frontier(resume, prop)
        resumed = frontier_to_arrays(hist)
        res = VerifyResult("unknown", domains_bounded=b0)
        max_depth = max_rounds + 2 + int(resumed[0].shape[1])
    else:
        # the root phase is deterministic: every rank runs it and reaches the same verdict and inherited bounds
        ce = attack(eng, net_id, net, prop, pgd_restarts, pgd_steps)
        if ce is not None:
            return VerifyResult("violated", ce[0], ce[1])
        rlo, _, inter_lo, inter_hi = eng.crown_bounds(net_id, spec, prop.in_lo, prop.in_hi)
        res = VerifyResult("unknown", root_lower=rlo[0].copy(), domains_bounded=1)
        if _verified_mask(rlo, thr, owner, n_clauses)[0]:
            res.status = "verified"
            return res
        inh_lo, inh_hi = inter_lo[0], inter_hi[0]
        max_depth = max_rounds + 2
    eng.frontier_create(net_id, spec, thr, owner, n_clauses, prop.in_lo, prop.in_hi, inh_lo, inh_hi,
                        max_depth=max_depth, capacity=min(2 * max_domains + 2 * batch, 1 << 22))
    if refinement not in ("parity", "verdict"):
        raise ValueError("refinement: parity or verdict")
    eng.frontier_set_refinement(refinement == "verdict")
    exchange = {"exchanges": 0, "records_moved": 0, "bytes_moved": 0} if world > 1 else None
    try:
        if resumed is not None:
            eng.frontier_upload(*resumed)
        if world > 1:
            import torch

            if rank != 0:   # the root belongs to rank 0's shard
                scratch = torch.empty((4 * max_depth + 1,), dtype=torch.int32, device=dist_device)
                eng.frontier_take(1, scratch.data_ptr(), scratch[4 * max_depth:].data_ptr())
        open_local = eng.frontier_count()
        total_open = max(open_local, 1)
        while total_open > 0 and res.rounds < max_rounds:
            timed_out = timeout_s is not None and time.time() - t0 > timeout_s
            bounded = stuck = 0
            if open_local > 0 and not timed_out:
                if optimize_iterations > 1:
                    bounded, _, _, stuck, open_local, _, _ = eng.frontier_round_optimized(batch, branching, optimize_iterations, 0.1, 0.05)
                else:
                    bounded, _, _, stuck, open_local, _, _ = eng.frontier_round(batch, branching)
            if world > 1:
                mine = torch.tensor([open_local, bounded, stuck, 1 if timed_out else 0], dtype=torch.int64, device=dist_device)
                every = [torch.zeros_like(mine) for _ in range(world)]
                dist.all_gather(every, mine)
                table = torch.stack(every).cpu().numpy()
                counts = [int(c) for c in table[:, 0]]
                total_open, bounded, stuck, timed_out = int(table[:, 0].sum()), int(table[:, 1].sum()), int(table[:, 2].max()), bool(table[:, 3].max())
            else:
                total_open = open_local
            res.rounds += 1
            res.domains_bounded += bounded
            if timed_out:
                res.status = "timeout"
                break
            if stuck or total_open > max_domains:
                break
            if world > 1 and total_open > 0:
                sharding.exchange_resident(eng, max_depth, counts, dist, dist_device, stats=exchange)
                open_local = eng.frontier_count()
        res.open_domains = total_open
        res.exchange = exchange
        if total_open == 0 and res.status == "unknown":
            res.status = "verified"
        if checkpoint is not None and world == 1 and total_open > 0:
            splits, ns = eng.frontier_download(max_depth)
            save_frontier(checkpoint, [splits[d, : ns[d]] for d in range(len(ns))], inh_lo, inh_hi, prop, res.rounds, res.domains_bounded)
    finally:
        eng.frontier_destroy()
    return res


def verify_resident_pool(pool, net_handle, net, prop: Property, *, batch: int = 1024, max_rounds: int = 64,
                         max_domains: int = 1 << 20, pgd_restarts: int = 256, pgd_steps: int = 50, branching: int = 1,
                         timeout_s: float | None = None, optimize_iterations: int = 0, refinement: str = "parity") -> VerifyResult:
    """verify_resident over the engines of an EnginePool (ny_b200.pool) on one GPU: one device frontier per engine, the
    root on the first, every engine bounding up to `batch` of its domains per round on its own stream and host thread,
    the shards levelled after the round by moving records from ring to ring on the device.  A round of a search is a
    chain of short launches with the host in between, so the engines' rounds overlap the way independent batches do.
    Same verdict as verify_resident and, when the search closes, the same domains; `batch` is per engine."""
    from concurrent.futures import ThreadPoolExecutor

    import torch

    from . import sharding

    t0 = time.time()
    if not prop.violation:
        return VerifyResult("verified")
    spec, thr, owner = _rows(prop)
    n_clauses = len(prop.violation)
    engines = pool.engines
    nids = pool._nets[net_handle]
    world = len(engines)
    ce = attack(engines[0], nids[0], net, prop, pgd_restarts, pgd_steps)
    if ce is not None:
        return VerifyResult("violated", ce[0], ce[1])
    rlo, _, inter_lo, inter_hi = engines[0].crown_bounds(nids[0], spec, prop.in_lo, prop.in_hi)
    res = VerifyResult("unknown", root_lower=rlo[0].copy(), domains_bounded=1)
    if _verified_mask(rlo, thr, owner, n_clauses)[0]:
        res.status = "verified"
        return res
    max_depth = max_rounds + 2
    device = torch.device("cuda", torch.cuda.current_device())
    for e, nid in zip(engines, nids):
        e.frontier_create(nid, spec, thr, owner, n_clauses, prop.in_lo, prop.in_hi, inter_lo[0], inter_hi[0],
                          max_depth=max_depth, capacity=min(2 * max_domains + 2 * batch, 1 << 22))
        e.frontier_set_refinement(refinement == "verdict")
    exchange = {"exchanges": 0, "records_moved": 0, "bytes_moved": 0}

    def one_round(i):
        if counts[i] == 0:
            return (0, 0, 0, 0, 0, 0, float("inf"))
        if optimize_iterations > 1:
            return engines[i].frontier_round_optimized(batch, branching, optimize_iterations, 0.1, 0.05)
        return engines[i].frontier_round(batch, branching)

    try:
        scratch = torch.empty((4 * max_depth + 1,), dtype=torch.int32, device=device)
        for e in engines[1:]:     # the root belongs to the first engine
            e.frontier_take(1, scratch.data_ptr(), scratch[4 * max_depth:].data_ptr())
        counts = [1] + [0] * (world - 1)
        total_open = 1
        with ThreadPoolExecutor(max_workers=world) as workers:
            while total_open > 0 and res.rounds < max_rounds:
                if timeout_s is not None and time.time() - t0 > timeout_s:
                    res.status = "timeout"
                    break
                stats = list(workers.map(one_round, range(world)))
                counts = [st[4] if counts[i] else 0 for i, st in enumerate(stats)]
                total_open = sum(counts)
                res.rounds += 1
                res.domains_bounded += sum(st[0] for st in stats)
                if any(st[3] for st in stats) or total_open > max_domains:
                    break
                for src, dst, n in sharding.plan_rebalance(counts):
                    sp = torch.empty((n, 4 * max_depth), dtype=torch.int32, device=device)
                    ns = torch.empty((n,), dtype=torch.int32, device=device)
                    engines[src].frontier_take(n, sp.data_ptr(), ns.data_ptr())
                    engines[dst].frontier_give(n, sp.data_ptr(), ns.data_ptr())
                    counts[src] -= n
                    counts[dst] += n
                    exchange["records_moved"] += n
                    exchange["bytes_moved"] += n * (4 * max_depth + 1) * 4
                    exchange["exchanges"] += 1
        res.open_domains = total_open
        res.exchange = exchange
        if total_open == 0 and res.status == "unknown":
            res.status = "verified"
    finally:
        for e in engines:
            e.frontier_destroy()
    return res


def _rebalance(frontier: "Frontier", dist, device, sharding, stats=None):
    """Levels the ranks' shards.  The shard sizes are gathered first and nothing else happens while they are level;
    otherwise the histories are padded to the deepest one of any rank and moved point to point, the warm-start
    slopes with them when every rank holds slopes for all of its open domains."""
    import torch

    counts = sharding.gather_counts(len(frontier), dist, device)
    if not sharding.plan_rebalance(counts):
        return
    splits, ns, alpha = frontier.pop(len(frontier))
    meta = torch.tensor([splits.shape[1], 1 if (alpha is not None or len(ns) == 0) else 0], dtype=torch.int64, device=device)
    agreed = [torch.zeros(2, dtype=torch.int64, device=device) for _ in range(dist.get_world_size())]
    dist.all_gather(agreed, meta)
    depth = max(int(t[0].item()) for t in agreed)
    # a rank with an empty shard holds no slopes to disagree about; one with domains but no slopes vetoes
    with_alpha = frontier.n_pre > 0 and all(int(t[1].item()) for t in agreed)
    if depth > splits.shape[1]:
        grown = np.zeros((len(ns), depth), SPLIT_DTYPE)
        grown[:, : splits.shape[1]] = splits
        splits = grown
    if with_alpha:
        if alpha is None:
            alpha = np.zeros((0, frontier.n_pre), np.float32)
        splits, ns, alpha = sharding.exchange_domains(splits, ns, dist, device, alpha=alpha, stats=stats, counts=counts)
        frontier.push(splits, ns, alpha)
    else:
        splits, ns = sharding.exchange_domains(splits, ns, dist, device, stats=stats, counts=counts)
        frontier.push(splits, ns)


def verify_root(eng, net_id, net, prop: Property, method: str = "crown") -> VerifyResult:
    """One bound of the whole box, no search (`ny verify --method ibp|crown`): verified when the interval pass (ibp)
    or plain CROWN with CROWN-tightened intermediates (crown) refutes every clause, violated when the box's centre
    is a counterexample, unknown otherwise."""
    if not prop.violation:
        return VerifyResult("verified")
    spec, thr, owner = _rows(prop)
    if method == "ibp":
        pl, pu = eng.ibp_forward_gpu(net_id, prop.in_lo, prop.in_hi)
        n_out = int(net.dims[-1])
        ylo, yhi = pl[0][-n_out:].astype(np.float64), pu[0][-n_out:].astype(np.float64)
        s64 = spec.astype(np.float64)
        terms = np.maximum(s64, 0) * ylo[None] + np.minimum(s64, 0) * yhi[None]
        # binary64 sum of exact products: its error is at most gamma_n * sum|terms|; remove it, then cast downwards
        n = terms.shape[1]
        gam = (n + 2) * 2.0 ** -53
        low = terms.sum(axis=1) - gam * np.abs(terms).sum(axis=1)
        l32 = low.astype(np.float32)
        lower = np.where(l32.astype(np.float64) > low, np.nextafter(l32, np.float32(-np.inf)), l32).astype(np.float32)[None]
    elif method == "crown":
        lower, _, _, _ = eng.crown_bounds(net_id, spec, prop.in_lo, prop.in_hi)
    else:
        raise ValueError(f"unknown method {method}")
    res = VerifyResult("unknown", root_lower=lower[0].copy(), domains_bounded=1)
    if _verified_mask(lower, thr, owner, len(prop.violation))[0]:
        res.status = "verified"
        return res
    x = ((prop.in_lo.astype(np.float64) + prop.in_hi.astype(np.float64)) * 0.5).astype(np.float32)
    y = forward(net, x)
    if _violates(prop, y):
        return VerifyResult("violated", x, y, 0, 1, 0, res.root_lower)
    res.open_domains = 1
    return res


# ------------------------------------------------------------------------------------------- input split
def input_split_scores(in_lo, in_hi, lower_a=None, lower=None, thr=None, coeff_thresh: float = 1e-3,
                       margin_weight: float = 1.0):
    """Score of every input dimension for a midpoint split, the margin-weighted smart-branching rule of the
    reference (BetaCrownVerifier::input_split_scores, beta_crown/engine/input_split.rs:111-243, default mode):
    max over spec rows of |lA[s, d]|.clamp(min = coeff_thresh) * width[d] / 2 + (lower[s] - thr[s]) * margin_weight;
    width only when there are no coefficients or all of them are zero; dimensions of zero or non-finite width get
    no score.  Returns (dims, scores), unsorted."""
    in_lo, in_hi = np.asarray(in_lo, np.float32), np.asarray(in_hi, np.float32)
    width = in_hi - in_lo
    ok = np.isfinite(width) & (width > 0)
    dims = np.flatnonzero(ok)
    if lower_a is None or not np.any(np.abs(lower_a) > 0):
        return dims, width[ok]
    a = np.abs(np.asarray(lower_a, np.float32))
    margin = np.zeros(a.shape[0], np.float32)
    if lower is not None and thr is not None:
        margin = (np.asarray(lower, np.float32) - np.asarray(thr, np.float32)) * np.float32(margin_weight)
    per_spec = np.maximum(a, np.float32(coeff_thresh)) * (width * np.float32(0.5))[None, :] + margin[:, None]
    score = per_spec.max(axis=0)
    keep = ok & np.isfinite(score)
    return np.flatnonzero(keep), score[keep]


def select_input_dimension(in_lo, in_hi, lower_a=None, lower=None, thr=None, **kw) -> int:
    """First maximum of input_split_scores; NaN scores never win (select_input_dimension_sb, input_split.rs:47-72).
    -1 when no dimension can be split."""
    dims, scores = input_split_scores(in_lo, in_hi, lower_a, lower, thr, **kw)
    best, best_score = -1, np.float32(-np.inf)
    for d, s in zip(dims, scores):
        if np.isnan(s):
            continue
        if best < 0 or s > best_score:
            best, best_score = int(d), s
    return best


def verify_input_split(eng, net_id, net, prop: Property, *, batch: int = 1024, max_rounds: int = 200,
                       max_domains: int = 1 << 20, pgd_restarts: int = 256, pgd_steps: int = 50,
                       timeout_s: float | None = None) -> VerifyResult:
    """Branch and bound over the INPUT box (the loop of the reference's input-split engine,
    beta_crown/engine/input_split.rs:262-460, batched): attack, then repeatedly bound a batch of sub-boxes with
    plain CROWN (all boxes in one device call), drop the verified ones, test the centre of every open box as a
    counterexample, and midpoint-split each along the dimension the smart-branching score picks.  What low-dimensional
    inputs (ACAS-shaped networks) use instead of ReLU splits."""
    t0 = time.time()
    if not prop.violation:
        return VerifyResult("verified")
    spec, thr, owner = _rows(prop)
    S, n0 = spec.shape[0], len(prop.in_lo)
    n_clauses = len(prop.violation)
    ce = attack(eng, net_id, net, prop, pgd_restarts, pgd_steps)
    if ce is not None:
        return VerifyResult("violated", ce[0], ce[1])
    res = VerifyResult("unknown")
    frontier_lo = [np.asarray(prop.in_lo, np.float32)]
    frontier_hi = [np.asarray(prop.in_hi, np.float32)]
    while frontier_lo and res.rounds < max_rounds:
        if timeout_s is not None and time.time() - t0 > timeout_s:
            res.status = "timeout"
            res.open_domains = len(frontier_lo)
            return res
        lo = np.stack(frontier_lo[:batch])
        hi = np.stack(frontier_hi[:batch])
        frontier_lo, frontier_hi = frontier_lo[batch:], frontier_hi[batch:]
        D = lo.shape[0]
        lower, _, _, _ = eng.crown_bounds(net_id, spec, lo, hi)
        lower_a, _ = eng.crown_input_coeffs(D, S, n0)
        if res.rounds == 0:
            res.root_lower = lower[0].copy()
        res.rounds += 1
        res.domains_bounded += D
        done = _verified_mask(lower, thr, owner, n_clauses)
        open_idx = np.flatnonzero(~done)
        if len(open_idx) == 0:
            continue
        centres = ((lo[open_idx].astype(np.float64) + hi[open_idx].astype(np.float64)) * 0.5).astype(np.float32)
        centres = np.clip(centres, lo[open_idx], hi[open_idx])
        ys = forward(net, centres)
        for x, y in zip(centres, ys):
            if _violates(prop, y):
                return VerifyResult("violated", x, y, res.rounds, res.domains_bounded, len(frontier_lo), res.root_lower)
        for d in open_idx:
            dim = select_input_dimension(lo[d], hi[d], lower_a[d], lower[d], thr)
            if dim < 0:
                res.open_domains = len(frontier_lo) + 1      # a point box that is neither verified nor violated
                return res
            mid = np.float32((np.float64(lo[d][dim]) + np.float64(hi[d][dim])) * 0.5)
            if not (lo[d][dim] < mid < hi[d][dim]):           # adjacent floats: the box cannot be split further
                res.open_domains = len(frontier_lo) + 1
                return res
            left_hi, right_lo = hi[d].copy(), lo[d].copy()
            left_hi[dim] = mid
            right_lo[dim] = mid
            frontier_lo += [lo[d], right_lo]
            frontier_hi += [left_hi, hi[d]]
        if len(frontier_lo) > max_domains:
            break
    res.open_domains = len(frontier_lo)
    if not frontier_lo:
        res.status = "verified"
    return res
