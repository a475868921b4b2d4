"""GPU parity tests for networks with residual connections (identity skips around two convolutions) against the
oracle evaluated on a sequential lowering of the same network: the skipped activation is carried as extra neurons
through identity rows (oracle.lower_residual), which changes no value - relu is the identity on a non-negative
interval - so the bounds of the original neurons are the same network's bounds."""
import numpy as np
import pytest

from ny_b200 import workloads as W
from test_gpu_parity import _rel, REL_TOL, IBP_REL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["tf32x3", "f64"])
def eng(request):
    from ny_b200 import B200Engine, engine

    e = B200Engine(0)
    e.set_path(engine.PATH_TF32X3 if request.param == "tf32x3" else engine.PATH_F64)
    e.path_name = request.param
    yield e
    e.close()


def _small(seed=61, eps=0.02, n_fix=3):
    return W.config_resnet(seed=seed, eps=eps, n_fix=n_fix, in_chw=(2, 8, 8), channels=4, blocks=2, n_out=5)


def _lowered(oracle, wl):
    ws, bs = oracle.lower_network(wl.net.weights, wl.net.biases)
    lw, lb, widths = oracle.lower_residual(ws, bs, wl.net.skips)
    onet = oracle.Net(lw, lb)
    wide = [w.shape[0] for w in lw]
    # index of every original neuron inside the lowered network's pre-activation layout
    idx, off = [], 0
    for k, n in enumerate(widths):
        idx.append(off + np.arange(n))
        off += wide[k]
    return onet, np.concatenate(idx)


def test_lowering_is_the_same_function(oracle):
    wl = _small()
    onet, _ = _lowered(oracle, wl)
    g = np.random.Generator(np.random.PCG64(1))
    x = wl.in_lo + g.random((16, len(wl.in_lo))) * (wl.in_hi - wl.in_lo)
    assert np.abs(onet.forward(x) - W.forward(wl.net, x)).max() < 1e-12


def test_residual_ibp_matches_oracle(eng, oracle):
    wl = _small()
    onet, idx = _lowered(oracle, wl)
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    tol = IBP_REL * np.maximum(np.abs(rl[idx]), np.abs(ru[idx])) + 1e-7
    assert np.all(np.abs(pl[0] - rl[idx]) <= tol) and np.all(np.abs(pu[0] - ru[idx]) <= tol)
    eng.release_network(nid)


@pytest.mark.parametrize("mode", [0, 1])
def test_residual_bab_bound_batch_matches_oracle(eng, oracle, mode):
    wl = _small(seed=62)
    onet, idx = _lowered(oracle, wl)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    D = 64
    splits, ns = W.draw_domains(wl, rl[idx], ru[idx], D)
    ns = ns.copy()
    ns[0] = 0
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl[idx], ru[idx], splits, ns, mode=mode)
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits, ns, mode)
    assert np.array_equal(ginf.astype(bool), oinf.astype(bool))
    feas = ~oinf.astype(bool)
    assert feas.sum() > D // 2
    assert _rel(np.concatenate([glo, ghi], axis=1)[feas], np.concatenate([olo, ohi], axis=1)[feas]) <= REL_TOL
    for d in np.flatnonzero(feas)[:5]:
        mn = W.sample_min_margin(wl, 20000, 300 + d, splits[d][: ns[d]])
        ok = np.isfinite(mn)
        assert np.all(glo[d][ok] <= mn[ok]), d
    eng.release_network(nid)


def test_residual_optimisation_matches_oracle(eng, oracle):
    """alpha/beta optimisation through residual blocks (the adjoint of relu(pre_j) joins pre_k's) against the oracle's
    loop on the lowered network."""
    wl = _small(seed=64, eps=0.03)
    onet, idx = _lowered(oracle, wl)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    D, iters = 24, 8
    splits, ns = W.draw_domains(wl, rl[idx], ru[idx], D)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl[idx], ru[idx], splits, ns, mode=1)
    eng.batch_optimize(iters, 0.1, 0.05)
    glo, ghi, ginf = eng.batch_download()
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    # one update (two iterations) moves every free slope by +-lr: the device's step directions must be the
    # oracle's wherever the gradient is not numerically zero (a missing or misplaced skip term would flip many)
    eng.batch_optimize(2, 0.1, 0.05)
    galpha, _ = eng.batch_download_params()
    n, rels, agree, total = 0, [], 0, 0
    n_hidden = int(wl.net.dims[1:-1].sum())
    for d in range(D):
        sp = splits[d][: ns[d]]
        pl, pu, bad = oracle.domain_bounds(ospec, wl.in_lo, wl.in_hi, rl2, ru2, sp, 1)
        assert bool(ginf[d]) == bool(bad)
        if bad:
            continue
        a0 = oracle.heuristic_alpha(ospec, pl, pu)
        olo, ohi, _, _ = oracle.optimize(ospec, wl.in_lo, wl.in_hi, pl, pu, sp, a0, iters, 0.1, 0.05)
        rels.append(_rel(np.concatenate([glo[d], ghi[d]]), np.concatenate([olo, ohi])))
        _, _, a1, _ = oracle.optimize(ospec, wl.in_lo, wl.in_hi, pl, pu, sp, a0, 2, 0.1, 0.05)
        _, ga, _ = oracle.joint_gradient(ospec, wl.in_lo, wl.in_hi, pl, pu, sp, a0)
        free = (np.abs(ga) > 1e-4 * np.abs(ga).max())[idx[:n_hidden]]
        agree += int(np.sum(np.isclose(galpha[d][:n_hidden][free], a1[idx[:n_hidden]][free], atol=1e-6)))
        total += int(free.sum())
        n += 1
    assert n > D // 2 and total > 0
    assert agree >= 0.995 * total, (agree, total)
    # Adam's sign-like steps make single trajectories diverge where a gradient is numerically zero: per domain
    # within a few 1e-3, typically far closer
    assert max(rels) <= 5e-3 and np.median(rels) <= 3e-4, (max(rels), np.median(rels))
    eng.release_network(nid)


def test_residual_pgd(eng, oracle):
    wl = _small(seed=63, eps=0.08)
    onet, idx = _lowered(oracle, wl)
    nid = eng.register_network(wl.net)
    g = np.random.Generator(np.random.PCG64(4))
    K, steps = 64, 25
    x0 = (wl.in_lo + g.random((K, len(wl.in_lo)), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)
    best0, bx0, _ = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, 0, 0.01)
    start = (W.forward(wl.net, x0) @ wl.spec.astype(np.float64).T).min(axis=1)
    assert np.allclose(best0, start, rtol=1e-5, atol=1e-6)
    eps = float((wl.in_hi - wl.in_lo).max()) / 2
    best, bx, ce = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, steps, 0.25 * eps)
    true = (W.forward(wl.net, bx) @ wl.spec.astype(np.float64).T).min(axis=1)
    assert np.allclose(best, true, rtol=1e-5, atol=1e-6) and np.all(best <= start + 1e-6) and best.mean() < start.mean()
    obest, _ = oracle.pgd_attack(onet.weights, onet.biases, wl.spec, wl.in_lo, wl.in_hi, x0, steps, 0.25 * eps)
    scale = np.abs(start).mean()
    assert np.abs(best - obest).max() <= 0.05 * scale and np.abs(best - obest).mean() <= 0.005 * scale
    eng.release_network(nid)


@pytest.mark.parametrize("seed,eps", [(61, 0.02), (63, 0.05), (65, 0.01)])
def test_residual_crown_ibp_matches_oracle(eng, oracle, seed, eps):
    """Plain CROWN with the CROWN-IBP collection on a residual network against the oracle's pipeline on the
    sequential lowering: within 1e-4 of the reference-faithful value, within 1e-5 once the oracle's certified error
    channel is left out (the device discharges roundings where they occur), never looser than the reference, sound
    against samples, and with intermediate bounds inside the interval pass's."""
    wl = _small(seed=seed, eps=eps)
    onet, idx = _lowered(oracle, wl)
    nid = eng.register_network(wl.net)
    glo, ghi, gil, giu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    ospec = onet.with_spec(wl.spec)
    olo, ohi = oracle.crown(ospec, wl.in_lo, wl.in_hi)
    nlo, nhi = oracle.crown(ospec, wl.in_lo, wl.in_hi, error_channel=False)
    scale = max(np.abs(olo).max(), np.abs(ohi).max())
    assert np.abs(glo[0] - olo).max() <= 1e-4 * scale and np.abs(ghi[0] - ohi).max() <= 1e-4 * scale
    assert np.abs(glo[0] - nlo).max() <= 1e-5 * scale and np.abs(ghi[0] - nhi).max() <= 1e-5 * scale
    assert np.all(glo[0] >= olo - 1e-6 * scale) and np.all(ghi[0] <= ohi + 1e-6 * scale)
    mn = W.sample_min_margin(wl, 100000, 7)
    assert np.all(glo[0] <= mn)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    nh = len(idx) - wl.net.dims[-1]
    tol = 1e-5 * np.maximum(np.abs(pl[0][:nh]), np.abs(pu[0][:nh])) + 1e-6
    assert np.all(gil[0][:nh] >= pl[0][:nh] - tol) and np.all(giu[0][:nh] <= pu[0][:nh] + tol)
    assert (giu[0][:nh] - gil[0][:nh]).sum() < 0.5 * (pu[0][:nh] - pl[0][:nh]).sum()
    # the root bounds feed a batch: tighter inherited bounds give bounds at least as tight
    splits, ns = W.draw_domains(wl, gil[0][: wl.net.n_pre], giu[0][: wl.net.n_pre], 8)
    lo_c, hi_c, _ = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, gil[0], giu[0], splits, ns, mode=1)
    lo_i, hi_i, _ = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, pl[0], pu[0], splits, ns, mode=1)
    assert np.all(lo_c >= lo_i - 1e-4 * np.abs(lo_i) - 1e-5)
    eng.release_network(nid)


def test_resnet_full_size(eng, oracle):
    """The residual configuration at full size (3x32x32, conv stem 64 + 4 residual blocks + avgpool + FC, box
    +-1/255, 9 rows): 64 split domains through the bound batch, the unsplit domain against sampled executions, a
    short attack against the concrete network."""
    wl = W.config_resnet()
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = pl[0], pu[0]
    assert np.all(rl <= ru)
    D = 64
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    feas = ginf == 0
    assert feas.sum() > D // 2 and np.all(np.isfinite(glo[feas])) and np.all(glo[feas] <= ghi[feas])
    mn = W.sample_min_margin(wl, 300, 9000, splits[0][:0], chunk=100)
    assert np.all(np.isfinite(mn)) and np.all(glo[0] <= mn) and np.all(ghi[0] >= mn - 1e30)
    g = np.random.Generator(np.random.PCG64(8))
    K = 32
    x0 = (wl.in_lo + g.random((K, len(wl.in_lo)), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)
    eps = float((wl.in_hi - wl.in_lo).max()) / 2
    best, bx, ce = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, 10, 0.25 * eps)
    true = (W.forward(wl.net, bx) @ wl.spec.astype(np.float64).T).min(axis=1)
    start = (W.forward(wl.net, x0) @ wl.spec.astype(np.float64).T).min(axis=1)
    assert np.allclose(best, true, rtol=1e-4, atol=1e-5) and np.all(best <= start + 1e-5) and best.mean() < start.mean()
    assert np.all(glo[0].min() <= best + 1e-5)          # the unsplit domain's bound is below every attacked point
    eng.release_network(nid)


def test_resnet_full_size_against_the_native_oracle(eng, oracle):
    """The residual configuration at full size against the oracle's native evaluation (kernel taps, identity branches
    joined in place: no lowering to dense matrices, which would be 65536 x 65536 here): the interval pass, and four
    split domains of a 64-domain batch to the parity tolerance."""
    wl = W.config_resnet()
    nat = oracle.Net(wl.net.weights, wl.net.biases, skips=wl.net.skips)
    nid = eng.register_network(wl.net)
    nl, nu = oracle.ibp_forward(nat, wl.in_lo, wl.in_hi)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    n = wl.net.n_pre
    tol = 1e-5 * np.maximum(np.abs(nl[:n]), np.abs(nu[:n])) + 1e-6
    assert np.all(np.abs(pl[0] - nl[:n]) <= tol) and np.all(np.abs(pu[0] - nu[:n]) <= tol)
    rl, ru = pl[0].copy(), pu[0].copy()
    D = 64
    splits, ns = W.draw_domains(wl, rl, ru, D)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    ospec = nat.with_spec(wl.spec)
    pick = np.array([0, 21, 42, 63])
    olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits[pick], ns[pick], 1)  # one call: the oracle runs its domains on separate threads
    checked = 0
    for i, d in enumerate(pick):
        assert bool(oinf[i]) == bool(ginf[d])
        if oinf[i]:
            continue
        got, ref = np.concatenate([glo[d], ghi[d]]), np.concatenate([olo[i], ohi[i]])
        scale = np.abs(ref).max()
        assert np.all(np.abs(got - ref) <= 1e-4 * np.maximum(np.abs(ref), 1e-2 * scale)), d
        checked += 1
    assert checked >= 3
    eng.release_network(nid)


def _skip_mlp(skips, seed=71, n_in=12, hidden=20, depth=6, n_out=4, eps=0.05, n_fix=3):
    """A ReLU MLP with the given identity branches {k: j} and a margin specification."""
    from ny_b200 import Network

    base = W.make_mlp([n_in] + [hidden] * depth + [n_out], seed)
    net = Network(base.weights, base.biases, skips)
    g = np.random.Generator(np.random.PCG64(seed + 1))
    x0 = g.uniform(-1, 1, n_in).astype(np.float32)
    y = W.forward(net, x0)
    c = int(np.argmax(y))
    spec = np.zeros((n_out - 1, n_out), np.float32)
    for i, j in enumerate([j for j in range(n_out) if j != c]):
        spec[i, c], spec[i, j] = 1.0, -1.0
    return W.Workload("skip-mlp", net, x0, (x0 - eps).astype(np.float32), (x0 + eps).astype(np.float32), spec, n_fix, seed)


@pytest.mark.parametrize("skips", [{3: 1, 5: 0}, {3: 0, 5: 2}, {3: 1, 5: 1}], ids=["nested", "overlapping", "shared-source"])
def test_nested_overlapping_and_shared_source_skips_match_oracle(eng, oracle, skips):
    """Identity branches that nest (a block inside a block), overlap (the second starts inside the first and ends
    after it) or start at the same variable: the interval pass, the bound batch in both child-bound modes and the
    attack against the oracle's native evaluation of the same network (identity branches joined in place), and the
    unsplit domain against sampled executions."""
    wl = _skip_mlp(skips)
    nat = oracle.Net(wl.net.weights, wl.net.biases, skips=wl.net.skips)
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    nl, nu = oracle.ibp_forward(nat, wl.in_lo, wl.in_hi)
    n = wl.net.n_pre
    tol = IBP_REL * np.maximum(np.abs(nl[:n]), np.abs(nu[:n])) + 1e-7
    assert np.all(np.abs(pl[0] - nl[:n]) <= tol) and np.all(np.abs(pu[0] - nu[:n]) <= tol)
    rl, ru = pl[0].copy(), pu[0].copy()
    D, S = 24, wl.spec.shape[0]
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    ospec = nat.with_spec(wl.spec)
    for mode in (0, 1):
        glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=mode)
        olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits, ns, mode)
        assert np.array_equal(ginf != 0, oinf != 0)
        f = oinf == 0
        assert f.sum() > D // 2
        assert _rel(np.concatenate([glo[f], ghi[f]], axis=1), np.concatenate([olo[f], ohi[f]], axis=1)) <= REL_TOL
    mn = W.sample_min_margin(wl, 20000, 123, splits[0][:0])
    assert np.all(glo[0] <= mn)
    # the attack's gradient follows the same branches: its reported objective is the network's value at its point
    g = np.random.Generator(np.random.PCG64(9))
    x0 = (wl.in_lo + g.random((16, len(wl.in_lo)), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)
    best, bx, _ = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, 10, 0.0125)
    true = (W.forward(wl.net, bx) @ wl.spec.astype(np.float64).T).min(axis=1)
    start = (W.forward(wl.net, x0) @ wl.spec.astype(np.float64).T).min(axis=1)
    assert np.allclose(best, true, rtol=1e-4, atol=1e-5) and best.mean() < start.mean()
    # and the parameter optimisation's adjoint: optimised bounds stay sound and do not get worse
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    plo, _, pinf = eng.batch_download()
    eng.batch_optimize(8, 0.1, 0.05)
    qlo, _, _ = eng.batch_download()
    ok = pinf == 0
    scale = np.abs(plo[ok]).max()
    assert np.all(qlo[ok] >= plo[ok] - 1e-5 * scale) and qlo[ok].sum() > plo[ok].sum()
    assert np.all(qlo[0] <= mn)
    eng.release_network(nid)


@pytest.mark.parametrize("kind", ["linear", "conv"])
def test_projection_block_lowering_bounds(eng, oracle, kind):
    """out = F(z) + P(z) (GpuResnetSegment::ResidualProj, crates/ny-core/src/gemm.rs:1658-1669) registered through
    lower_projection_block: the lowered network is the same function, its device bounds match the oracle on the same
    layers and enclose sampled executions of the ORIGINAL two-branch network."""
    from ny_b200 import Conv2d, Network, lower_projection_block

    g = np.random.Generator(np.random.PCG64(77))
    rn = lambda *s: (g.standard_normal(s) * np.sqrt(2.0 / np.prod(s[1:]))).astype(np.float32)
    if kind == "linear":
        n0, nz, h, no, nout = 10, 12, 16, 14, 4
        stem = (rn(nz, n0), rn(nz))
        F = [(rn(h, nz), rn(h)), (rn(no, h), rn(no))]
        P = (rn(no, nz), rn(no))
        head = (rn(nout, no), rn(nout))
        low = lower_projection_block(F, P)
        net = Network([stem[0]] + [w for w, _ in low] + [head[0]], [stem[1]] + [b for _, b in low] + [head[1]])

        def original(x):
            z = np.maximum(x @ stem[0].astype(np.float64).T + stem[1], 0)
            f = np.maximum(z @ F[0][0].astype(np.float64).T + F[0][1], 0) @ F[1][0].astype(np.float64).T + F[1][1]
            out = np.maximum(f + z @ P[0].astype(np.float64).T + P[1], 0)
            return out @ head[0].astype(np.float64).T + head[1]
    else:
        c0, cz, c1, co, nout = 2, 3, 4, 5, 4
        stem = Conv2d(rn(cz, c0, 3, 3), rn(cz), (1, 1), (1, 1), (8, 8))
        F1 = Conv2d(rn(c1, cz, 3, 3), rn(c1), (2, 2), (1, 1), (8, 8))
        F2 = Conv2d(rn(co, c1, 3, 3), rn(co), (1, 1), (1, 1), (4, 4))
        P = Conv2d(rn(co, cz, 1, 1), rn(co), (2, 2), (0, 0), (8, 8))
        head = (rn(nout, co * 16), rn(nout))
        low = lower_projection_block([(F1, None), (F2, None)], (P, None))
        n0 = c0 * 64
        net = Network([stem] + [w for w, _ in low] + [head[0]], [None] + [None for _ in low] + [head[1]])

        def original(x):
            z = np.maximum(stem.apply(x), 0)
            out = np.maximum(F2.apply(np.maximum(F1.apply(z), 0)) + P.apply(z), 0)
            return out @ head[0].astype(np.float64).T + head[1]
    x0 = g.uniform(0.2, 0.8, n0).astype(np.float32)
    lo, hi = (x0 - 0.03).astype(np.float32), (x0 + 0.03).astype(np.float32)
    xs = lo + g.random((4000, n0)) * (hi.astype(np.float64) - lo)
    assert np.abs(W.forward(net, xs[:64]) - original(xs[:64])).max() < 1e-9       # the same function
    spec = np.zeros((nout - 1, nout), np.float32)
    spec[:, 0] = 1.0
    spec[np.arange(nout - 1), 1 + np.arange(nout - 1)] = -1.0
    wl = W.Workload("proj", net, x0, lo, hi, spec, 3, 77)
    nid = eng.register_network(net)
    nat = oracle.Net(net.weights, net.biases)
    pl, pu = eng.ibp_forward_gpu(nid, lo, hi)
    rl, ru = pl[0].copy(), pu[0].copy()
    D, S = 16, spec.shape[0]
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    glo, ghi, ginf = eng.bab_bound_batch(nid, spec, lo, hi, rl, ru, splits, ns, mode=1)
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    olo, ohi, oinf, _ = oracle.bab_bound_batch(nat.with_spec(spec), lo, hi, rl2, ru2, splits, ns, 1)
    assert np.array_equal(ginf != 0, oinf != 0)
    f = oinf == 0
    assert _rel(np.concatenate([glo[f], ghi[f]], axis=1), np.concatenate([olo[f], ohi[f]], axis=1)) <= REL_TOL
    margins = original(xs) @ spec.astype(np.float64).T
    assert np.all(glo[0] <= margins.min(axis=0)) and np.all(ghi[0] >= margins.max(axis=0))
    eng.release_network(nid)


@pytest.mark.parametrize("stride", [1, 2])
def test_wide_convolutions_match_the_native_oracle(eng, oracle, stride):
    """Convolutions with 32 and 36 channels (the small residual test networks have 4): a 3x3 stride-1 layer (nine taps
    per output pixel) or a 4x4 stride-2 layer (four stride-parity classes of four taps) against the oracle's native
    convolution (the sums of layers/convolution/conv2d/bound.rs:601-900), the unsplit domain against sampled
    executions, and the parameter optimisation's checkpointed passes through the same layers."""
    from ny_b200 import Conv2d, Network

    g = np.random.Generator(np.random.PCG64(90 + stride))
    rn = lambda *s: (g.standard_normal(s) * np.sqrt(2.0 / np.prod(s[1:]))).astype(np.float32)
    c0, c1, c2, nout = 2, 32, 36, 5
    hw = 8
    stem = Conv2d(rn(c1, c0, 3, 3), rn(c1), (1, 1), (1, 1), (hw, hw))
    if stride == 1:
        mid = Conv2d(rn(c2, c1, 3, 3), rn(c2), (1, 1), (1, 1), (hw, hw))
    else:
        mid = Conv2d(rn(c2, c1, 4, 4), rn(c2), (2, 2), (1, 1), (hw, hw))
    head_w, head_b = rn(nout, mid.out_features), rn(nout)
    net = Network([stem, mid, head_w], [None, None, head_b])
    n0 = c0 * hw * hw
    x0 = g.uniform(0.2, 0.8, n0).astype(np.float32)
    lo, hi = (x0 - 0.01).astype(np.float32), (x0 + 0.01).astype(np.float32)
    spec = np.zeros((nout - 1, nout), np.float32)
    spec[:, 0] = 1.0
    spec[np.arange(nout - 1), 1 + np.arange(nout - 1)] = -1.0
    wl = W.Workload("wide-conv", net, x0, lo, hi, spec, 3, 90)
    nid = eng.register_network(net)
    nat = oracle.Net(net.weights, net.biases)
    pl, pu = eng.ibp_forward_gpu(nid, lo, hi)
    rl, ru = pl[0].copy(), pu[0].copy()
    D, S = 16, spec.shape[0]
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    glo, ghi, ginf = eng.bab_bound_batch(nid, spec, lo, hi, rl, ru, splits, ns, mode=1)
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    olo, ohi, oinf, _ = oracle.bab_bound_batch(nat.with_spec(spec), lo, hi, rl2, ru2, splits, ns, 1)
    assert np.array_equal(ginf != 0, oinf != 0)
    f = oinf == 0
    assert f.sum() > D // 2
    assert _rel(np.concatenate([glo[f], ghi[f]], axis=1), np.concatenate([olo[f], ohi[f]], axis=1)) <= REL_TOL
    mn = W.sample_min_margin(wl, 4000, 91, splits[0][:0], chunk=1000)
    assert np.all(glo[0] <= mn)
    # and the parameter optimisation, whose checkpointed passes go through the same layers
    eng.batch_upload(nid, spec, lo, hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    plo, _, pinf = eng.batch_download()
    eng.batch_optimize(6, 0.1, 0.05)
    qlo, _, _ = eng.batch_download()
    ok = pinf == 0
    # (the plain run's flagged domains were re-evaluated in binary64, the optimisation's evaluations carry their
    # rounding charge: equal parameters may come out a few 1e-5 of the scale lower)
    assert np.all(qlo[ok] >= plo[ok] - 2e-4 * np.abs(plo[ok]).max()) and np.all(qlo[0] <= mn)
    eng.release_network(nid)
