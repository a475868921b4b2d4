"""Properties of the oracle's beta-CROWN restatement on small seeded networks (CPU only): it must
reduce to plain CROWN's backward when nothing is split, enclose concrete executions, and treat
splits the way the reference's tests expect (beta_crown/engine/tests/*.rs)."""
import numpy as np

from ny_b200 import workloads as W


def _small(seed=7, depth=3, hidden=24, n_in=12):
    wl = W.config_mlp_bab(seed=seed, hidden=hidden, depth=depth, n_in=n_in, n_out=5, eps=0.05, n_fix=3)
    return wl


def _onet(oracle, wl):
    return oracle.Net(wl.net.weights, wl.net.biases)


def test_unsplit_domain_encloses_samples(oracle):
    wl = _small()
    net = _onet(oracle, wl).with_spec(wl.spec)
    base = _onet(oracle, wl)
    pl, pu = oracle.ibp_forward(base, wl.in_lo, wl.in_hi)
    spl, spu = oracle.ibp_forward(net, wl.in_lo, wl.in_hi)
    lo, hi = oracle.beta_crown_bound(net, wl.in_lo, wl.in_hi, spl, spu, oracle.make_splits([]))
    mn = W.sample_min_margin(wl, 20000, 11)
    assert np.all(lo <= mn + 1e-6) and np.all(np.isfinite(lo)) and np.all(lo <= hi)
    assert np.allclose(pl, spl[: len(pl)])


def test_split_domains_enclose_constrained_samples_and_modes_nest(oracle):
    wl = _small(seed=9)
    net = _onet(oracle, wl).with_spec(wl.spec)
    rl, ru = oracle.ibp_forward(net, wl.in_lo, wl.in_hi)
    splits, ns = W.draw_domains(wl, rl, ru, 12)
    for mode in (0, 1):
        lo, hi, inf, _ = oracle.bab_bound_batch(net, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode, 2)
        for d in range(12):
            if inf[d]:
                continue
            mn = W.sample_min_margin(wl, 4000, 100 + d, splits[d][: ns[d]])
            ok = np.isfinite(mn)
            assert np.all(lo[d][ok] <= mn[ok] + 1e-5), (mode, d)


def test_beta_zero_inactive_split_zeroes_neuron(oracle):
    # with beta = 0, an inactive split behaves as a stable-inactive neuron: slopes (0, 0)
    wl = _small(seed=3)
    net = _onet(oracle, wl).with_spec(wl.spec)
    rl, ru = oracle.ibp_forward(net, wl.in_lo, wl.in_hi)
    unstable = np.flatnonzero((rl[:24] < 0) & (ru[:24] > 0))
    j = int(unstable[0])
    sp = oracle.make_splits([(0, j, -1, 0.0)])
    lo_s, _ = oracle.beta_crown_bound(net, wl.in_lo, wl.in_hi, rl, ru, sp)
    rl2, ru2 = rl.copy(), ru.copy()
    ru2[j] = 0.0  # the same relaxation arises from u <= 0
    lo_c, _ = oracle.beta_crown_bound(net, wl.in_lo, wl.in_hi, rl2, ru2, oracle.make_splits([]))
    assert np.array_equal(lo_s, lo_c)


def test_infeasible_clamp_is_reported(oracle):
    wl = _small(seed=5)
    net = _onet(oracle, wl).with_spec(wl.spec)
    rl, ru = oracle.ibp_forward(net, wl.in_lo, wl.in_hi)
    stable_pos = np.flatnonzero(rl[:24] > 0)
    if len(stable_pos) == 0:
        rl = rl.copy()
        rl[0] = 0.5
        ru = np.maximum(ru, 1.0)
        stable_pos = np.array([0])
    sp = oracle.make_splits([(0, int(stable_pos[0]), -1, 0.3)])
    _, _, inf = oracle.domain_bounds(net, wl.in_lo, wl.in_hi, rl, ru, sp, 0)
    assert inf


def test_largest_width_first_maximum_wins(oracle):
    net = oracle.Net([np.eye(4, 3), np.eye(3, 4), np.eye(2, 3)])
    pl = np.array([-1, -2, -2, 1, -1, -3, 5, 0, 0], np.float32)
    pu = np.array([1, 2, 2, 2, 1, 1, 6, 0, 0], np.float32)
    assert oracle.select_largest_width(net, pl, pu, oracle.make_splits([]))[:2] == (0, 1)
    assert oracle.select_largest_width(net, pl, pu, oracle.make_splits([(0, 1, 1, 0.0)]))[:2] == (0, 2)
    pl[4], pu[4] = np.nan, np.nan
    assert oracle.select_largest_width(net, pl, pu, oracle.make_splits([(0, 1, 1, 0), (0, 2, -1, 0)]))[:2] == (1, 1)


def _one_domain(oracle, seed=9):
    wl = _small(seed=seed)
    net = _onet(oracle, wl).with_spec(wl.spec)
    rl, ru = oracle.ibp_forward(net, wl.in_lo, wl.in_hi)
    splits, ns = W.draw_domains(wl, rl, ru, 1)
    sp = splits[0][: ns[0]].copy()
    sp["beta"] = np.linspace(0.05, 0.3, len(sp)).astype(np.float32)
    pl, pu, inf = oracle.domain_bounds(net, wl.in_lo, wl.in_hi, rl, ru, sp, 1)
    assert not inf
    rng = np.random.default_rng(seed)
    alpha = np.where((pl < 0) & (pu > 0), rng.uniform(0.2, 0.8, pl.shape), 0.0).astype(np.float32)
    return wl, net, sp, pl, pu, alpha


def test_joint_gradient_matches_central_differences(oracle):
    """The reference pins its joint alpha gradient by central finite differences
    (ny-core/src/joint_alpha_grad.rs tests; beta_crown/engine/optimization/gradients tests): same here,
    for alpha and for beta, against the value the same fold returns."""
    wl, net, sp, pl, pu, alpha = _one_domain(oracle)
    low, ga, gb = oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha)
    slo, _ = oracle.beta_crown_bound(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha)
    assert np.all(slo <= low + 1e-9) and np.allclose(slo, low, rtol=0, atol=1e-4)
    h = 1e-3
    unstable = np.flatnonzero((pl < 0) & (pu > 0) & (ga != 0))
    assert len(unstable) >= 5
    for i in unstable[:12]:
        ap, am = alpha.copy(), alpha.copy()
        ap[i] += h
        am[i] -= h
        fd = (oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, ap)[0].sum()
              - oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, am)[0].sum()) / (2 * h)
        assert abs(fd - ga[i]) <= 1e-3 * max(1.0, abs(fd)), (i, fd, ga[i])
    for q in range(len(sp)):
        s1, s2 = sp.copy(), sp.copy()
        s1["beta"][q] += h
        s2["beta"][q] -= h
        fd = (oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, s1, alpha)[0].sum()
              - oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, s2, alpha)[0].sum()) / (2 * h)
        assert abs(fd - gb[q]) <= 1e-3 * max(1.0, abs(fd)), (q, fd, gb[q])
    # stable and split neurons carry no alpha gradient
    assert np.all(ga[~((pl < 0) & (pu > 0))] == 0)


def test_optimisation_improves_and_stays_sound(oracle):
    wl, net, sp, pl, pu, alpha = _one_domain(oracle, seed=13)
    sp["beta"] = 0.0
    a0 = oracle.heuristic_alpha(net, pl, pu)
    lo0, hi0 = oracle.beta_crown_bound(net, wl.in_lo, wl.in_hi, pl, pu, sp, a0)
    bl, bu, a1, s1 = oracle.optimize(net, wl.in_lo, wl.in_hi, pl, pu, sp, a0, 20, 0.1, 0.05)
    assert np.all(bl >= lo0) and np.all(bu <= hi0)          # element-wise best includes iteration 1
    assert bl.sum() > lo0.sum()
    assert np.all((a1 >= 0) & (a1 <= 1)) and np.all(s1["beta"] >= 0)
    mn = W.sample_min_margin(wl, 4000, 5, sp)
    ok = np.isfinite(mn)
    assert np.all(bl[ok] <= mn[ok] + 1e-5)
    # one iteration is the plain bound
    bl1, bu1, _, _ = oracle.optimize(net, wl.in_lo, wl.in_hi, pl, pu, sp, a0, 1, 0.1, 0.05)
    assert np.array_equal(bl1, lo0) and np.array_equal(bu1, hi0)


def test_intercept_branching_first_maximum_and_nan(oracle):
    """picked.rs:153-233: score (-l*u)/(u-l), strict '>' (first maximum wins), NaN bounds and split neurons skipped."""
    net = oracle.Net([np.eye(4, dtype=np.float32), np.ones((1, 4), np.float32)], [None, None])
    pre_lo = np.array([-1.0, -2.0, -2.0, np.nan, 0.0], np.float32)
    pre_hi = np.array([1.0, 2.0, 2.0, 5.0, 0.0], np.float32)
    got = oracle.select_intercept(net, pre_lo, pre_hi, oracle.make_splits([]))
    assert got[:2] == (0, 1) and got[2] == np.float32(1.0)            # neurons 1 and 2 tie at 1.0: the first wins
    got = oracle.select_intercept(net, pre_lo, pre_hi, oracle.make_splits([(0, 1, 1, 0.0)]))
    assert got[:2] == (0, 2)
    assert oracle.select_intercept(net, np.full(5, 1, np.float32), np.full(5, 2, np.float32), oracle.make_splits([])) is None


def test_worst_row_gradient_is_that_rows_gradient(oracle):
    """With the single-row objective the gradient is the finite difference of that row's bound alone."""
    wl, net, sp, pl, pu, alpha = _one_domain(oracle, seed=17)
    low, _, _ = oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha)
    row = int(np.argmin(low))
    import ctypes as C
    ga = np.zeros(net.n_pre, np.float32)
    gb = np.zeros(len(sp), np.float32)
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    args = [np.ascontiguousarray(x, np.float32) for x in (wl.in_lo, wl.in_hi, pl, pu)]
    oracle.lib().nyo_joint_gradient_rows(C.byref(net.c), f(args[0]), f(args[1]), f(args[2]), f(args[3]), sp.ctypes.data,
                                         len(sp), f(alpha), None, f(ga), f(gb), row)
    h = 1e-3
    idx = np.flatnonzero(ga != 0)[:8]
    assert len(idx) > 0
    for i in idx:
        ap, am = alpha.copy(), alpha.copy()
        ap[i] += h
        am[i] -= h
        fd = (oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, ap)[0][row]
              - oracle.joint_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, am)[0][row]) / (2 * h)
        assert abs(fd - ga[i]) <= 1e-3 * max(1.0, abs(fd))


def test_dual_alpha_upper_gradient_and_optimisation(oracle):
    """Upper-path slopes: gradient against central differences of the upper bounds; the dual optimisation leaves the
    lower bounds where shared slopes put them and tightens the upper ones."""
    wl, net, sp, pl, pu, alpha = _one_domain(oracle, seed=19)
    rng = np.random.default_rng(3)
    aup = np.where((pl < 0) & (pu > 0), rng.uniform(0.2, 0.8, pl.shape), 0.0).astype(np.float32)
    up, g = oracle.upper_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha, aup)
    _, shi = oracle.beta_crown_bound_dual(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha, aup)
    assert np.all(shi >= up - 1e-9) and np.allclose(shi, up, rtol=0, atol=1e-4)
    h = 1e-3
    idx = np.flatnonzero(g != 0)[:10]
    assert len(idx) >= 3
    for i in idx:
        p_, m_ = aup.copy(), aup.copy()
        p_[i] += h
        m_[i] -= h
        fd = (oracle.upper_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha, p_)[0].sum()
              - oracle.upper_gradient(net, wl.in_lo, wl.in_hi, pl, pu, sp, alpha, m_)[0].sum()) / (2 * h)
        assert abs(fd - g[i]) <= 1e-3 * max(1.0, abs(fd))
    a0 = oracle.heuristic_alpha(net, pl, pu)
    bl, bu, _, _ = oracle.optimize(net, wl.in_lo, wl.in_hi, pl, pu, sp, a0, 15, 0.1, 0.05)
    dl, du, _, aup1, _ = oracle.optimize_dual(net, wl.in_lo, wl.in_hi, pl, pu, sp, a0, 15, 0.1, 0.05)
    assert np.array_equal(dl, bl) and np.all(du <= bu + 1e-6) and du.sum() < bu.sum()
    assert np.all((aup1 >= 0) & (aup1 <= 1))


def test_babsr_scores_hand_case():
    """1 -> 2 -> 1 with W1 = (1, -1), b1 = (0.5, 0), W2 = (1, 1), one spec row (1), both neurons on [-1, 1]:
    r0 = 1/2, r1 = 1/2, c = 1 for both; neuron 0: |min(0.5 * (-1/2), 0.5 * 1/2) + 0| = 0.25, neuron 1 (no bias): 0.
    A split neuron and a stable one are not candidates (-1)."""
    import numpy as np
    from oracle import ny_oracle as O

    ws = [np.array([[1.0], [-1.0]], np.float32), np.array([[1.0, 1.0]], np.float32)]
    bs = [np.array([0.5, 0.0], np.float32), None]
    spec = np.array([[1.0]], np.float32)
    sc, pick = O.babsr_scores(ws, bs, spec, np.array([-1, -1, 0], np.float32), np.array([1, 1, 0], np.float32))
    assert sc.tolist() == [0.25, 0.0] and pick == (0, 0)
    sc, pick = O.babsr_scores(ws, bs, spec, np.array([-1, -1, 0], np.float32), np.array([1, 1, 0], np.float32),
                              split_mask=np.array([True, False, False]))
    assert sc.tolist() == [-1.0, 0.0] and pick == (0, 1)
    sc, pick = O.babsr_scores(ws, bs, spec, np.array([0.5, 0.1, 0], np.float32), np.array([1, 1, 0], np.float32))
    assert sc.tolist() == [-1.0, -1.0] and pick == (-1, -1)
    # negative coefficient: the intercept term min(c, 0) * r1 enters; spec row (-1): c = -1, b = 0.5:
    # |min(-0.5 * (-1/2), -0.5 * 1/2) + (-1) * 1/2| = |-0.25 - 0.5| = 0.75
    sc, _ = O.babsr_scores(ws, bs, -spec, np.array([-1, -1, 0], np.float32), np.array([1, 1, 0], np.float32))
    assert sc.tolist() == [0.75, 0.5]


def _babsr_reference_cases():
    """The two hand-computed cases of the reference's own branching tests
    (crates/ny-propagate/src/beta_crown/engine/tests/branching.rs:998-1143), restated with an identity first layer in
    front of the reference's leading ReLU: (weights, biases, spec, pre_lo, pre_hi, expected scores per hidden neuron,
    expected (relu, neuron), expected best score)."""
    eye = np.eye(2, dtype=np.float32)
    # relu -> Linear [[-3, -0.5]], box [-1, 1]^2: scores |min(lA, 0) * intercept| = 1.5 and 0.25, pick neuron 0
    one = ([eye, np.array([[-3.0, -0.5]], np.float32)], [None, None], np.array([[1.0]], np.float32),
           np.array([-1, -1, -3.5], np.float32), np.array([1, 1, 0.0], np.float32), [1.5, 0.25], (0, 0), 1.5)
    # relu0 -> Linear [[2,-1],[0,3]] -> relu1 -> Linear [[-1,-4]]; relu1's pre-activation bounds given as [-1, 1]:
    # coefficients 1.0 / 5.5 at relu0 and 1.0 / 4.0 at relu1, intercept 0.5 everywhere; pick relu0 neuron 1, score 2.75
    two = ([eye, np.array([[2.0, -1.0], [0.0, 3.0]], np.float32), np.array([[-1.0, -4.0]], np.float32)], [None, None, None],
           np.array([[1.0]], np.float32), np.array([-1, -1, -1, -1, -10], np.float32), np.array([1, 1, 1, 1, 10], np.float32),
           [0.5, 2.75, 0.5, 2.0], (0, 1), 2.75)
    return [one, two]


def test_babsr_restatement_matches_the_reference_hand_computed_answers():
    from oracle import ny_oracle as O

    for ws, bs, spec, lo, hi, scores, pick, best in _babsr_reference_cases():
        sc, got = O.babsr_scores(ws, bs, spec, lo, hi)
        assert got == pick
        assert np.allclose(sc, scores, atol=1e-6) and abs(float(sc.max()) - best) < 1e-6


# ---- optimiser restatements pinned to the reference's own known answers (tests/golden/optimizer_reference.json) ----
def _golden_opt():
    import json
    import os

    with open(os.path.join(os.path.dirname(__file__), "golden", "optimizer_reference.json")) as f:
        return json.load(f)


def test_adam_clipping_step_known_answers(oracle):
    G = _golden_opt()
    for c in G["adam_clipping"]:
        n = len(c["x"])
        x, m, v = oracle.adam_clipping_step(np.zeros(n, np.float32), np.zeros(n, np.float32), 1, c["gradient"], c["x"], c["lo"],
                                            c["hi"], c["lr0"], c["lr_decay"], c["beta1"], c["beta2"], c["eps"])
        assert np.all(np.abs(x - np.array(c["expected"], np.float32)) < c["tol"]), c["name"]
    c = G["adam_clipping_lr_decay"]
    x = np.array(c["x0"], np.float32)
    m = v = np.zeros(1, np.float32)
    steps = []
    for t in (1, 2):
        xn, m, v = oracle.adam_clipping_step(m, v, t, c["gradient"], x, c["lo"], c["hi"], c["lr0"], c["lr_decay"], c["beta1"], c["beta2"], c["eps"])
        steps.append(float(xn[0] - x[0]))
        x = xn
    assert np.all(np.abs(np.array(steps) - np.array(c["expected_steps"])) < c["tol"])      # step 1 uses lr0, then decays
    c = G["project_nan"]
    pt = np.array([float(p) for p in c["point"]], np.float32)
    # a zero step leaves the point where projection puts it: NaN -> lower end, above the box -> upper end
    xn, _, _ = oracle.adam_clipping_step(np.zeros(2, np.float32), np.zeros(2, np.float32), 1, [0.0, 0.0], pt, c["lo"], c["hi"], 0.0)
    assert xn.tolist() == c["expected"]


def test_beta_updates_known_answers(oracle):
    G = _golden_opt()
    c = G["beta_plain_step"]
    vals, mg = oracle.beta_plain_step(c["values"], c["grads"], c["lr"])
    assert np.all(np.abs(vals - np.array(c["expected_values"], np.float32)) < c["tol"]) and abs(mg - c["expected_max_grad"]) < c["tol"]
    c = G["beta_signed"]
    sp = oracle.make_splits([(0, i, 1 if a else -1, b) for i, (a, b) in enumerate(zip(c["active"], c["values"]))])
    assert (sp["beta"] * sp["sign"]).tolist() == c["expected"]
    c = G["beta_adam"]
    cfg = c["config"]
    z = lambda: {k: np.zeros(1, np.float32) for k in ("value", "m", "v", "v_max")}
    st, _ = oracle.beta_adam_step(z(), [c["grad"]], 1, **cfg)
    s1 = c["step1"]
    assert abs(st["m"][0] - s1["m"]) < s1["m_tol"] and abs(st["v"][0] - s1["v"]) < s1["v_tol"] and abs(st["value"][0] - s1["value"]) < s1["value_tol"]
    prev = st["value"][0]
    for t in range(2, c["monotone_steps"] + 1):
        st, _ = oracle.beta_adam_step(st, [c["grad"]], t, **cfg)
        assert st["value"][0] > prev
        prev = st["value"][0]
    assert abs(st["m"][0] - c["m_after_5"]) < c["m5_tol"]
    c = G["beta_adam_clip"]
    a, _ = oracle.beta_adam_step(z(), [c["grad"]], 1, grad_clip=c["grad_clip"])
    b, _ = oracle.beta_adam_step(z(), [c["same_value_as_grad"]], 1, grad_clip=c["grad_clip"])
    assert abs(a["m"][0] - c["m"]) < 1e-6 and abs(a["v"][0] - c["v"]) < 1e-7 and abs(a["value"][0] - b["value"][0]) < c["tol"]
    # AMSGrad keeps the running maximum of v: after a large gradient a small one moves beta less than plain Adam does
    sa, sp_ = z(), z()
    for t, g in enumerate([5.0, 0.1, 0.1], start=1):
        sa, _ = oracle.beta_adam_step(sa, [g], t, amsgrad=True)
        sp_, _ = oracle.beta_adam_step(sp_, [g], t, amsgrad=False)
    assert sa["v_max"][0] >= sa["v"][0] and sa["value"][0] <= sp_["value"][0]
