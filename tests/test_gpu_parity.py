"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Tolerances: interval forward bounds within 1e-5 relative of the oracle; output bounds within
1e-4 relative (the bar stated for this path), soundness against sampled concrete executions."""
import numpy as np
import pytest

from ny_b200 import workloads as W

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4
IBP_REL = 1e-5


@pytest.fixture(scope="module", params=["tf32x3", "f64"])
def eng(request):
    """Every parity case runs on both contraction paths: the tcgen05 3xTF32 default and the binary64 one."""
    from ny_b200 import B200Engine, engine

    e = B200Engine(0)
    e.set_path(engine.PATH_TF32X3 if request.param == "tf32x3" else engine.PATH_F64)
    e.path_name = request.param
    yield e
    e.close()


def _rel(a, b):
    """Largest deviation of a from the oracle's b, relative to max(|b|, 1e-2 * scale) where scale is the
    largest bound magnitude of the same domain.  The floor matters only for bounds that cancel to
    nearly zero: every fp32 coefficient carries a 2^-24 relative rounding that a sound method has to pay
    for against the variable's magnitude, so a bound that is 1000x smaller than its own terms cannot
    agree to 1e-4 of its value in any fp32-storage implementation (the reference's two engines differ
    there too).  Equivalent statement: 1e-4 relative with an absolute floor of 1e-6 of the domain scale."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    fin = np.isfinite(a) & np.isfinite(b)
    same_inf = (~fin) & (a == b)
    assert np.all(fin | same_inf), "non-finite mismatch"
    if not fin.any():
        return 0.0
    bb = np.where(fin, np.abs(b), 0.0)
    scale = bb.max(axis=-1, keepdims=True) if b.ndim > 1 else bb.max()
    den = np.maximum(np.maximum(bb, 1e-2 * scale), 1e-30)
    return float(np.max(np.where(fin, np.abs(a - b), 0.0) / den))


def _spec_net(wl):
    from ny_b200 import Network

    return Network(wl.net.weights + [wl.spec], wl.net.biases + [None])


def _setup(eng, oracle, wl):
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    return onet, ospec, nid, rl, ru


def _oracle_batch(oracle, ospec, wl, rl, ru, splits, ns, mode):
    # the oracle's network carries the spec as its last layer: extend the inherited bounds with that
    # layer's (unused) block
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    return oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits, ns, mode)


@pytest.mark.parametrize("cfg", ["small", "mid"])
def test_ibp_forward_matches_oracle(eng, oracle, cfg):
    wl = W.config_mlp_small() if cfg == "small" else W.config_mlp_bab(seed=4, hidden=96, depth=4, n_in=200)
    onet, _, nid, rl, ru = _setup(eng, oracle, wl)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    # Both sides round outward at every layer (the oracle steps one ulp past round-to-nearest, the
    # device rounds directed), so the one-ulp differences compound with depth: compare relative to the
    # interval's magnitude.
    tol = IBP_REL * np.maximum(np.abs(rl), np.abs(ru))
    assert np.all(np.abs(pl[0] - rl) <= tol) and np.all(np.abs(pu[0] - ru) <= tol)
    assert np.all(pl[0] <= pu[0])
    # per-domain boxes: two different boxes in one call
    lo2 = np.stack([wl.in_lo, wl.in_lo + 0.01 * (wl.in_hi - wl.in_lo)])
    hi2 = np.stack([wl.in_hi, wl.in_hi])
    pl2, pu2 = eng.ibp_forward_gpu(nid, lo2, hi2)
    assert np.array_equal(pl2[0], pl[0]) and np.array_equal(pu2[0], pu[0])
    r2l, r2u = oracle.ibp_forward(onet, lo2[1], hi2[1])
    assert np.all(np.abs(pl2[1] - r2l) <= tol) and np.all(np.abs(pu2[1] - r2u) <= tol)
    eng.release_network(nid)


def test_ibp_forward_many_boxes_matches_oracle(eng, oracle):
    """96 different boxes in one call: on the default path this is the tensor-core interval pass (D >= 64).  Its
    rounding slack widens every interval, so the device may sit outside the oracle's interval by that slack but
    never inside it by more than the oracle's own outward ulps; a box whose slack shows is re-run in binary64."""
    wl = W.config_mlp_bab(seed=9, hidden=128, depth=4, n_in=160)
    onet, _, nid, rl, ru = _setup(eng, oracle, wl)
    rng = np.random.default_rng(12)
    D = 96
    mid, rad = 0.5 * (wl.in_lo + wl.in_hi), 0.5 * (wl.in_hi - wl.in_lo)
    shrink = rng.uniform(0.1, 1.0, size=(D, 1)).astype(np.float32)
    shift = rng.uniform(-1, 1, size=(D, wl.in_lo.shape[0])).astype(np.float32) * (1 - shrink) * rad
    lo = (mid + shift - shrink * rad).astype(np.float32)
    hi = np.maximum((mid + shift + shrink * rad).astype(np.float32), lo)
    pl, pu = eng.ibp_forward_gpu(nid, lo, hi)
    for d in range(0, D, 7):
        ol, ou = oracle.ibp_forward(onet, lo[d], hi[d])
        tol = IBP_REL * np.maximum(np.abs(ol), np.abs(ou))
        assert np.all(np.abs(pl[d] - ol) <= tol) and np.all(np.abs(pu[d] - ou) <= tol), d
        assert np.all(pl[d] <= pu[d])
    eng.release_network(nid)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("cfg", ["small", "mid"])
def test_bab_bound_batch_matches_oracle(eng, oracle, cfg, mode):
    if cfg == "small":
        wl = W.config_mlp_small()
        wl.n_fix = 4
        D = 96
    else:
        wl = W.config_mlp_bab(seed=6, hidden=64, depth=4, n_in=196, eps=0.01, n_fix=8)
        D = 200
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0          # an unsplit (root) domain
    ns[1] = 1          # ragged split lists
    ns[2] = max(int(ns[2]) - 1, 0)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=mode)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits, ns, mode)
    assert np.array_equal(ginf.astype(bool), oinf.astype(bool))
    feas = ~oinf.astype(bool)
    assert feas.sum() > D // 2
    both = np.concatenate([olo, ohi], axis=1)
    assert _rel(np.concatenate([glo, ghi], axis=1)[feas], both[feas]) <= REL_TOL
    assert np.all(glo[feas] <= olo[feas] + 1e-6 * np.abs(both[feas]).max(axis=1, keepdims=True))  # never tighter than fp32 noise
    # verdicts (lower > 0) identical wherever the oracle is not within tolerance of the threshold
    clear = np.abs(olo) > REL_TOL * np.maximum(1.0, np.abs(olo))
    assert np.array_equal((glo > 0)[feas & clear.all(axis=1)], (olo > 0)[feas & clear.all(axis=1)])
    eng.release_network(nid)


def test_soundness_against_sampled_executions(eng, oracle):
    wl = W.config_mlp_bab(seed=8, hidden=48, depth=3, n_in=64, eps=0.03, n_fix=4)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    splits, ns = W.draw_domains(wl, rl, ru, 16)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    for d in range(16):
        if ginf[d]:
            continue
        mn = W.sample_min_margin(wl, 100000, 500 + d, splits[d][: ns[d]])
        ok = np.isfinite(mn)
        assert np.all(glo[d][ok] <= mn[ok]), d
    eng.release_network(nid)


def test_infeasible_and_empty_batches(eng, oracle):
    wl = W.config_mlp_bab(seed=5, hidden=32, depth=2, n_in=16, eps=0.01, n_fix=2)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    from ny_b200 import SPLIT_DTYPE, EngineError

    stable = np.flatnonzero(rl[:32] > 0)
    assert len(stable) > 0
    sp = np.zeros((2, 1), SPLIT_DTYPE)
    sp[0, 0] = (0, int(stable[0]), -1, 0.25)   # inactive split on a provably active neuron: empty domain
    sp[1, 0] = (0, int(stable[0]), 1, 0.25)    # consistent split
    ns = np.array([1, 1], np.int32)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, sp, ns, mode=1)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, sp, ns, 1)
    assert ginf.tolist() == [1, 0] and oinf.tolist() == [1, 0]
    assert np.all(glo[0] == np.inf) and np.all(ghi[0] == -np.inf)
    assert _rel(glo[1], olo[1]) <= REL_TOL
    # max_splits = 0: plain CROWN-style bound of the root domain
    sp0 = np.zeros((3, 0), SPLIT_DTYPE)
    glo0, _, _ = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, sp0, np.zeros(3, np.int32), mode=1)
    olo0, _, _, _ = _oracle_batch(oracle, ospec, wl, rl, ru, np.zeros((3, 1), SPLIT_DTYPE), np.zeros(3, np.int32), 1)
    assert _rel(glo0, olo0) <= REL_TOL and np.array_equal(glo0[0], glo0[2])
    # out-of-range split entries are refused, never silently used
    bad = np.zeros((1, 1), SPLIT_DTYPE)
    bad[0, 0] = (0, 9999, 1, 0.0)
    with pytest.raises(EngineError) as ei:
        eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, bad, np.array([1], np.int32))
    assert ei.value.code == 3
    with pytest.raises(EngineError):
        eng.bab_bound_batch(nid, wl.spec[:, :5], wl.in_lo, wl.in_hi, rl, ru, sp, ns)
    eng.release_network(nid)


def test_branching_matches_oracle_and_min_lower(eng, oracle):
    wl = W.config_mlp_bab(seed=12, hidden=40, depth=3, n_in=30, eps=0.02, n_fix=3)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    splits, ns = W.draw_domains(wl, rl, ru, 40)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    glo, ghi, ginf = eng.batch_download()
    pl, pu = eng.batch_download_pre_bounds()
    r, j, w = eng.batch_select_branch()
    r1, j1, w1 = eng.batch_select_branch(kind=1)
    feas = ginf == 0
    assert np.isclose(eng.batch_min_lower(), glo[feas].min())
    # verdicts with the reference's predicates, at thresholds that split the batch
    L = oracle.lib()
    for thr in (0.0, float(np.median(glo[feas].min(axis=1))), float(np.median(ghi[feas].max(axis=1))), float("inf")):
        st = eng.batch_verdicts(thr)
        for d in range(40):
            if ginf[d]:
                assert st[d] == 3
                continue
            ver = all(L.nyo_domain_verified(float(glo[d][s]), float(ghi[d][s]), thr) for s in range(glo.shape[1]))
            vio = any(L.nyo_domain_violated(float(glo[d][s]), float(ghi[d][s]), thr) for s in range(glo.shape[1]))
            assert st[d] == (1 if ver else (2 if vio else 0)), (thr, d)
    for d in range(40):
        if ginf[d]:
            continue
        got = oracle.select_largest_width(onet, pl[d], pu[d], splits[d][: ns[d]])
        assert got is not None and (int(r[d]), int(j[d])) == got[:2] and w[d] == np.float32(got[2])
        got1 = oracle.select_intercept(onet, pl[d], pu[d], splits[d][: ns[d]])
        assert got1 is not None and (int(r1[d]), int(j1[d])) == got1[:2] and w1[d] == np.float32(got1[2])
        opl, opu, oinf = oracle.domain_bounds(onet, wl.in_lo, wl.in_hi, rl, ru, splits[d][: ns[d]], 1)
        hid = int(wl.net.dims[1:-1].sum())
        tol = IBP_REL * np.maximum(np.abs(opl[:hid]), np.abs(opu[:hid]))
        assert np.all(np.abs(pl[d][:hid] - opl[:hid]) <= tol)
    eng.release_network(nid)


def test_gemm_f32_entry_point(eng):
    g = np.random.Generator(np.random.PCG64(3))
    a = g.standard_normal((37, 129)).astype(np.float32)
    b = g.standard_normal((129, 65)).astype(np.float32)
    c = eng.gemm_f32(37, 129, 65, a, b)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    if eng.path_name == "f64":
        assert np.array_equal(c, exact.astype(np.float32))  # binary64 accumulation, one rounding to fp32
    else:
        S = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
        assert np.max(np.abs(c - exact) / S) <= 2e-6  # within the rounding model of the 3xTF32 product


def test_full_size_batch_properties(eng, oracle):
    """Configuration of the benchmark (784 -> 8x256 -> 10, 4096 domains, 8 splits each): checked through
    size-independent properties, plus oracle parity on a 32-domain sample."""
    wl = W.config_mlp_bab()
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = pl[0], pu[0]
    D = 4096
    splits, ns = W.draw_domains(wl, rl, ru, D)
    lo, hi, inf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    lo2, hi2, inf2 = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    assert np.array_equal(lo, lo2) and np.array_equal(hi, hi2)            # deterministic
    perm = np.random.Generator(np.random.PCG64(1)).permutation(D)
    lop, hip, infp = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits[perm], ns[perm], mode=1)
    assert np.array_equal(lop, lo[perm]) and np.array_equal(infp, inf[perm])  # domains are independent
    feas = inf == 0
    assert np.all(lo[feas] <= hi[feas]) and np.all(np.isfinite(lo[feas]))
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    ospec = onet.with_spec(wl.spec)
    sel = np.arange(0, D, D // 32)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits[sel], ns[sel], 1)
    assert np.array_equal(oinf.astype(bool), inf[sel].astype(bool))
    f = ~oinf.astype(bool)
    assert _rel(lo[sel][f], olo[f]) <= REL_TOL and _rel(hi[sel][f], ohi[f]) <= REL_TOL
    d = int(np.flatnonzero(feas)[0])
    mn = W.sample_min_margin(wl, 100000, 77, splits[d][: ns[d]])
    ok = np.isfinite(mn)
    assert np.all(lo[d][ok] <= mn[ok])
    eng.release_network(nid)


def test_full_size_verdicts_and_split_decisions_identical(eng, oracle):
    """Benchmark configuration at full size (4096 domains): for 256 of them (every 16th) the verdicts at three
    thresholds and the branching decision (layer, neuron) are compared with the oracle's, computed by the oracle
    from its own bounds.  A comparison is only excused where the oracle's own number sits within 1e-4 (relative) of
    the deciding threshold, or its two best branching scores within 1e-5 of each other; those near-ties are counted
    and must stay rare.  Eight domains are also checked against 10^5 sampled executions each."""
    wl = W.config_mlp_bab()
    nid = eng.register_network(wl.net)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    ospec = onet.with_spec(wl.spec)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    D = 4096
    splits, ns = W.draw_domains(wl, rl, ru, D)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    glo, ghi, ginf = eng.batch_download()
    sel = np.arange(0, D, 16)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits[sel], ns[sel], 1)
    assert np.array_equal(oinf.astype(bool), ginf[sel].astype(bool))
    f = ~oinf.astype(bool)
    assert f.sum() >= 200
    assert _rel(np.concatenate([glo[sel], ghi[sel]], axis=1)[f], np.concatenate([olo, ohi], axis=1)[f]) <= REL_TOL
    # ---- verdicts at three thresholds that split the sample
    L = oracle.lib()
    S = olo.shape[1]
    worst = olo[f].min(axis=1)
    near_ties = 0
    for qt in (0.25, 0.5, 0.75):
        thr = float(np.quantile(worst, qt))
        st = eng.batch_verdicts(thr)[sel]
        for i in np.flatnonzero(f):
            ver = all(L.nyo_domain_verified(float(olo[i][s]), float(ohi[i][s]), thr) for s in range(S))
            vio = any(L.nyo_domain_violated(float(olo[i][s]), float(ohi[i][s]), thr) for s in range(S))
            want = 1 if ver else (2 if vio else 0)
            tie = np.any(np.abs(olo[i] - thr) <= REL_TOL * np.maximum(np.abs(olo[i]), np.abs(thr))) or \
                np.any(np.abs(ohi[i] - thr) <= REL_TOL * np.maximum(np.abs(ohi[i]), np.abs(thr)))
            if tie:
                near_ties += int(st[i] != want)
                continue
            assert st[i] == want, (qt, int(sel[i]), st[i], want)
    assert near_ties <= 4
    # ---- branching decisions (largest width and intercept score), from the oracle's own pre-activation bounds
    r0, j0, _ = eng.batch_select_branch()
    r1, j1, _ = eng.batch_select_branch(kind=1)
    pl, pu = eng.batch_download_pre_bounds()
    score_ties = 0
    for i in np.flatnonzero(f)[::2]:
        d = int(sel[i])
        opl, opu, _ = oracle.domain_bounds(onet, wl.in_lo, wl.in_hi, rl, ru, splits[d][: ns[d]], 1)
        for kind, (rr, jj) in enumerate(((r0, j0), (r1, j1))):
            got = oracle.select_largest_width(onet, opl, opu, splits[d][: ns[d]]) if kind == 0 else \
                oracle.select_intercept(onet, opl, opu, splits[d][: ns[d]])
            assert got is not None
            if (int(rr[d]), int(jj[d])) != got[:2]:
                # excused only when the oracle's score of the device's pick ties with its own best
                hid = int(wl.net.dims[1:-1].sum())
                off = int(np.concatenate([[0], np.cumsum(wl.net.dims[1:-1])])[int(rr[d])]) + int(jj[d])
                l, u = float(opl[off]), float(opu[off])
                sc = (u - l) if kind == 0 else (-l * u) / (u - l)
                assert off < hid and abs(sc - got[2]) <= 1e-5 * abs(got[2]), (d, kind, sc, got)
                score_ties += 1
    assert score_ties <= 2
    # ---- soundness on eight domains, 10^5 samples each
    for d in [int(x) for x in np.flatnonzero(ginf == 0)[:: max(1, int((ginf == 0).sum()) // 8)][:8]]:
        mn = W.sample_min_margin(wl, 100000, 200 + d, splits[d][: ns[d]])
        ok = np.isfinite(mn)
        assert np.all(glo[d][ok] <= mn[ok]), d
    eng.release_network(nid)


def test_entry_point_smoke():
    """The repository's smoke entry (one small invocation of the hot path checked against the oracle) stays green."""
    import __graft_entry__

    __graft_entry__.smoke()


def test_domain_major_relaxation_with_ragged_column_slab(eng, oracle):
    """A batch large enough for the domain-major relaxation kernel whose layer width (200) leaves the last
    128-column slab partly empty: lanes past the row's end must take part in the row reductions with zeros."""
    wl = W.config_mlp_bab(seed=71, hidden=200, depth=2, n_in=60, eps=0.03, n_fix=3)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    D = 1100
    splits, ns = W.draw_domains(wl, rl, ru, D)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    pick = np.r_[0:40, D - 40:D]
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits[pick], ns[pick], 1)
    assert np.array_equal(ginf[pick].astype(bool), oinf.astype(bool))
    feas = ~oinf.astype(bool)
    assert feas.sum() > 40
    assert _rel(np.concatenate([glo[pick], ghi[pick]], axis=1)[feas], np.concatenate([olo, ohi], axis=1)[feas]) <= REL_TOL
    eng.release_network(nid)


def test_batches_in_flight_on_an_engine_pool_match_a_single_engine(oracle):
    """ny_b200.pool.EnginePool: several engines on one GPU, each with its own stream, workspace and host thread, the
    batches handed out in turn.  Every batch's bounds are bit-identical to the ones a single engine returns for it."""
    from ny_b200 import B200Engine
    from ny_b200.pool import EnginePool

    wl = W.config_mlp_bab(seed=19, hidden=128, depth=4, n_in=96, eps=0.015, n_fix=6)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    batches = []
    for k in range(7):
        splits, ns = W.draw_domains(wl, rl, ru, 200 + 37 * k, first=1000 * k)
        batches.append((wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, 1))
    one = B200Engine(0)
    nid = one.register_network(wl.net)
    want = [one.bab_bound_batch(nid, *b) for b in batches]
    one.close()
    pool = EnginePool(0, 3)
    h = pool.register_network(wl.net)
    for _ in range(2):   # the second pass runs on warmed-up workspaces
        got = pool.bound_batches(h, batches)
        assert len(got) == len(want)
        for (gl, gu, gi), (wl_, wu, wi) in zip(got, want):
            assert np.array_equal(gl, wl_) and np.array_equal(gu, wu) and np.array_equal(gi, wi)
    # an engine's error surfaces after every thread has ended
    from ny_b200 import EngineError

    bad = list(batches)
    bad[4] = bad[4][:5] + (bad[4][5], bad[4][6][:-1], 1)     # n_splits shorter than the batch
    with pytest.raises(EngineError):
        pool.bound_batches(h, bad)
    pool.close()


def test_persistent_kernels_with_reserved_sms_return_the_same_bits(oracle):
    """nyb200_set_reserved_sms: the full-width persistent kernels leave SMs to a concurrent collective; the tiles are
    dealt to fewer CTAs, every tile is computed as before."""
    from ny_b200 import B200Engine

    wl = W.config_mlp_bab(seed=23, hidden=256, depth=4, n_in=300, eps=0.01, n_fix=6)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    splits, ns = W.draw_domains(wl, rl, ru, 1500)
    eng = B200Engine(0)
    nid = eng.register_network(wl.net)
    want = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns)
    for n in (1, 2, 40):
        eng.set_reserved_sms(n)
        got = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns)
        assert all(np.array_equal(a, b) for a, b in zip(got, want))
    from ny_b200 import EngineError

    with pytest.raises(EngineError):
        eng.set_reserved_sms(-1)
    eng.close()


def test_gemm_f32_keeps_the_round_to_nearest_error_model(eng):
    """GemmEngine::gemm_f32's precision contract (crates/ny-core/src/gemm.rs:318-324): |c - a.b| <= gamma_k sum|a||b|
    with gamma_k = k u / (1 - k u), u = 2^-24, for every contraction length - short ones included, where the 3xTF32
    product's own rate would be above gamma_k; gemm_f32_fast has no such contract and stays close to fp32."""
    g = np.random.Generator(np.random.PCG64(5))
    u = 2.0 ** -24
    for k in (1, 2, 5, 8, 16, 20, 21, 40, 64, 300):
        a = (g.standard_normal((70, k)) * np.exp(g.uniform(-3, 3, (70, k)))).astype(np.float32)
        b = (g.standard_normal((k, 33)) * np.exp(g.uniform(-3, 3, (k, 33)))).astype(np.float32)
        exact = a.astype(np.float64) @ b.astype(np.float64)
        S = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
        gamma = k * u / (1 - k * u)
        c = eng.gemm_f32(70, k, 33, a, b)
        # the result's own final rounding to fp32 is part of the model for k = 1 (gamma_1 = u)
        assert np.all(np.abs(c - exact) <= gamma * S * (1 + 1e-9) + 1e-45), k
        if k < 21 and eng.path_name != "f64":
            assert np.array_equal(c, exact.astype(np.float32)), k     # binary64 accumulation, one rounding
        f = eng.gemm_f32_fast(70, k, 33, a, b)
        assert np.max(np.abs(f - exact) / S) <= 2e-6, k
