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


def _rows(prop: Property):
    spec, thr, owner = [], [], []
    for ci, clause in enumerate(prop.violation):
        for atom in clause:
            spec.append(-np.asarray(atom.c, np.float32))
            thr.append(np.float32(atom.d))
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


def verify(eng, net_id, net, prop: Property, *, batch: int = 1024, max_rounds: int = 64, max_domains: int = 1 << 20,
           pgd_restarts: int = 256, pgd_steps: int = 50, optimize_iterations: int = 0, branching: int = 1,
           timeout_s: float | None = None) -> VerifyResult:
    """batch: domains bounded per device call; optimize_iterations: projected-Adam steps on the slopes and split
    multipliers of every domain (0, the reference's throughput default `beta_iterations: 0`
    (beta_crown/config/beta_config.rs:1244), bounds each domain once with multipliers at zero: sound, but the search
    may then end "unknown" on properties that need the multipliers; 20 is the reference's root-level count);
    branching: 0 widest interval, 1 intercept score."""
    t0 = time.time()
    if not prop.violation:
        return VerifyResult("verified")
    spec, thr, owner = _rows(prop)
    n_clauses = len(prop.violation)
    ce = attack(eng, net_id, net, prop, pgd_restarts, pgd_steps)
    if ce is not None:
        return VerifyResult("violated", ce[0], ce[1])
    # root: plain CROWN with CROWN-tightened intermediate bounds
    rlo, _, inter_lo, inter_hi = eng.crown_bounds(net_id, spec, prop.in_lo, prop.in_hi)
    res = VerifyResult("unknown", root_lower=rlo[0].copy(), domains_bounded=1)
    if _verified_mask(rlo, thr, owner, n_clauses)[0]:
        res.status = "verified"
        return res
    inh_lo, inh_hi = inter_lo[0], inter_hi[0]
    frontier = [np.zeros(0, SPLIT_DTYPE)]
    while frontier and res.rounds < max_rounds:
        if timeout_s is not None and time.time() - t0 > timeout_s:
            res.status = "timeout"
            res.open_domains = len(frontier)
            return res
        take, frontier = frontier[:batch], frontier[batch:]
        depth = max(1, max(len(s) for s in take))
        D = len(take)
        splits = np.zeros((D, depth), SPLIT_DTYPE)
        ns = np.zeros(D, np.int32)
        for d, s in enumerate(take):
            splits[d, : len(s)] = s
            ns[d] = len(s)
        eng.batch_upload(net_id, spec, prop.in_lo, prop.in_hi, inh_lo, inh_hi, splits, ns, mode=1)
        if optimize_iterations > 1:
            eng.batch_optimize(optimize_iterations, 0.1, 0.05)
        else:
            eng.batch_run()
        lower, _, infeasible = eng.batch_download()
        res.rounds += 1
        res.domains_bounded += D
        done = _verified_mask(lower, thr, owner, n_clauses) | (infeasible != 0)
        if done.all():
            continue
        relu, neuron, _ = eng.batch_select_branch(branching)
        for d in np.flatnonzero(~done):
            if relu[d] < 0:
                # every neuron is fixed: the bound is exact on this piece, so the piece contains a violation
                # candidate; without a witness the honest answer is unknown
                res.open_domains = len(frontier) + 1
                return res
            for sign in (1, -1):
                child = np.zeros(len(take[d]) + 1, SPLIT_DTYPE)
                child[: len(take[d])] = take[d]
                child[-1] = (int(relu[d]), int(neuron[d]), sign, 0.0)
                frontier.append(child)
        if len(frontier) > max_domains:
            break
    res.open_domains = len(frontier)
    if not frontier:
        res.status = "verified"
    return res
