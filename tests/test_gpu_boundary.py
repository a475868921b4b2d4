"""The reference-shaped entry points (layer lists in backward order with caller-baked relaxation slopes, per-domain
signed multipliers and abs-max tables: the operands of ny's GpuCrownBackward trait methods) against the split-list
calls and the oracle.  The relaxation tables are baked on the host from the device's own pre-activation bounds with
the arithmetic the engine uses, so both routes see the same tables."""
import numpy as np
import pytest

from ny_b200 import workloads as W
from test_gpu_parity import _rel, _setup, REL_TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from ny_b200 import B200Engine

    e = B200Engine(0)
    yield e
    e.close()


def _round(x64, up):
    r = np.asarray(x64, np.float64).astype(np.float32)
    if up:
        bad = r.astype(np.float64) < x64
        return np.where(bad, np.nextafter(r, np.float32(np.inf)), r).astype(np.float32)
    bad = r.astype(np.float64) > x64
    return np.where(bad, np.nextafter(r, np.float32(-np.inf)), r).astype(np.float32)


def _bake_beta(l, u, code):
    """The beta-CROWN table of one layer from its pre-activation interval and split codes (+1 / -1 / 0), in the
    engine's arithmetic: chord slope u / max(u - l, 1e-8) in fp32, intercept the smallest fp32 that keeps the chord
    above ReLU at both ends, lower slope [u > -l]."""
    l, u = l.astype(np.float32), u.astype(np.float32)
    ls = np.zeros_like(l); us = np.zeros_like(l); ui = np.zeros_like(l)
    act = (code > 0) | ((code == 0) & (l >= 0))
    ls[act] = 1; us[act] = 1
    un = (code == 0) & (l < 0) & (u > 0)
    w = np.maximum((u - l).astype(np.float32), np.float32(1e-8))
    s = (u / w).astype(np.float32)
    i1 = _round(s.astype(np.float64) * (-l.astype(np.float64)), True)
    i2 = _round(u.astype(np.float64) - _round(s.astype(np.float64) * u.astype(np.float64), False).astype(np.float64), True)
    us[un] = s[un]
    ui[un] = np.maximum(np.maximum(i1, i2), 0)[un]
    ls[un] = (u[un] > -l[un]).astype(np.float32)
    return ls, us, ui


def _domain_tables(wl, pl, pu, splits, n):
    """Per ReLU (forward order): (ls, us, ui), signed beta, abs-max, for one domain."""
    dims = [int(x) for x in wl.net.dims]
    offs = np.concatenate([[0], np.cumsum(dims[1:])]).astype(int)
    out = []
    for k in range(len(dims) - 2):
        lo, hi = pl[offs[k]:offs[k + 1]], pu[offs[k]:offs[k + 1]]
        code = np.zeros(dims[k + 1], np.int32); sb = np.zeros(dims[k + 1], np.float32)
        for q in range(n):
            s = splits[q]
            if s["relu"] == k:
                code[s["neuron"]] = s["sign"]; sb[s["neuron"]] = s["beta"] * s["sign"]
        ls, us, ui = _bake_beta(lo, hi, code)
        out.append((ls, us, ui, sb, np.maximum(np.abs(lo), np.abs(hi)).astype(np.float32)))
    return out


def _layers(wl, tabs):
    """Backward-order layer list (output -> input) with the baked tables."""
    L = len(wl.net.weights)
    layers = []
    for k in range(L - 1, -1, -1):
        layers.append(("linear", wl.net.weights[k], wl.net.biases[k]))
        if k > 0:
            ls, us, ui = tabs[k - 1][:3]
            layers.append(("act", ls, us, None, ui))
    return layers


def test_batched_call_with_baked_tables_matches_the_split_list_call(eng, oracle):
    wl = W.config_mlp_bab(seed=41, hidden=64, depth=4, n_in=100, eps=0.01, n_fix=6)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    D = 96
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy(); ns[0] = 0
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    glo, ghi, ginf = eng.batch_download()
    pl, pu = eng.batch_download_pre_bounds()
    feas = np.flatnonzero(ginf == 0)
    domains = []
    for d in feas:
        tabs = _domain_tables(wl, pl[d], pu[d], splits[d], int(ns[d]))
        domains.append({"layers": _layers(wl, tabs), "lo": wl.in_lo, "hi": wl.in_hi,
                        "node_abs": [t[4] for t in tabs][::-1], "beta_signed": [t[3] for t in tabs][::-1]})
    blo, bhi = eng.crown_resnet_beta_batched(domains, wl.spec)
    scale = np.maximum(np.abs(glo[feas]).max(axis=1, keepdims=True), np.abs(ghi[feas]).max(axis=1, keepdims=True))
    # Same relaxation tables and the same kernels; the one operand that differs is q, the weight of the rounding charge:
    # the split-list call takes |W| z_upper from its interval pass, this call can only use |W| node_abs (the abs-max
    # table bounds the post-activation from above, loosely where |l| > u).  So the baked route charges a little more:
    # never tighter than the split-list route, and within a fraction of the charge (2e-5 of the domain's scale).
    assert np.all(blo <= glo[feas] + 1e-6 * scale) and np.all(bhi >= ghi[feas] - 1e-6 * scale)
    assert np.all(np.abs(blo - glo[feas]) <= 2e-5 * scale) and np.all(np.abs(bhi - ghi[feas]) <= 2e-5 * scale)
    # and the oracle agrees with both
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)]); ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    sel = feas[:24]
    olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits[sel], ns[sel], 1)
    assert _rel(np.concatenate([blo[:24], bhi[:24]], axis=1), np.concatenate([olo, ohi], axis=1)) <= REL_TOL
    # a heterogeneous batch (a domain with other weight tensors) is refused as a whole
    from ny_b200 import EngineError
    other = [("linear", l[1].copy(), l[2]) if l[0] == "linear" else l for l in domains[1]["layers"]]
    bad = [domains[0], dict(domains[1], layers=other)]
    with pytest.raises(EngineError) as ei:
        eng.crown_resnet_beta_batched(bad, wl.spec)
    assert ei.value.code == 3
    eng.release_network(nid)


def test_crown_backward_with_baked_slopes_matches_the_reference_bound(eng, oracle):
    """crown_backward_gpu_sound's operands: plain-CROWN slopes baked by the caller (here from the oracle's tightened
    intermediate bounds, the chord of activations/relu/mod.rs:105-132), one box.  The result is the oracle's final
    backward pass (before its intersection with the forward bounds) to 1e-4; the seeded form started at the last
    hidden layer with the spec pushed through the last Linear by hand gives the same numbers."""
    wl = W.config_mlp_small()
    onet = oracle.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    olo, ohi, il, iu = oracle.crown(onet, wl.in_lo, wl.in_hi, want_intermediate=True)
    dims = [int(x) for x in wl.net.dims]
    offs = np.concatenate([[0], np.cumsum(dims[1:])]).astype(int)
    tabs = []
    for k in range(len(dims) - 2):
        l, u = il[offs[k]:offs[k + 1]].astype(np.float64), iu[offs[k]:offs[k + 1]].astype(np.float64)
        ls = np.zeros(dims[k + 1], np.float32); us = np.zeros_like(ls); ui = np.zeros_like(ls)
        ls[l >= 0] = 1; us[l >= 0] = 1
        un = (l < 0) & (u > 0)
        lam = np.nextafter((u / np.where(un, u - l, 1)).astype(np.float32), np.float32(np.inf))
        icp = np.nextafter((-lam.astype(np.float64) * l).astype(np.float32), np.float32(np.inf))
        us[un] = lam[un]; ui[un] = icp[un]; ls[un] = (u[un] > -l[un]).astype(np.float32)
        tabs.append((ls, us, ui))
    layers = _layers(wl, tabs)
    glo, ghi = eng.crown_backward(layers, wl.spec, wl.in_lo, wl.in_hi)
    # the oracle's published bound is this pass intersected with forward bounds: never looser than the pass itself
    scale = np.abs(olo).max()
    assert np.all(glo <= olo + 1e-6 * scale) and np.all(ghi >= ohi - 1e-6 * scale)
    # the pass itself against the device's own CROWN pipeline in the reference convention (same tables by construction)
    from ny_b200 import engine as E
    nid = eng.register_network(wl.net)
    eng.set_error_channel(E.ERRCH_REFERENCE)
    try:
        plo, phi, pil, piu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    finally:
        eng.set_error_channel(E.ERRCH_IMMEDIATE)
    assert np.all(np.abs(plo[0] - glo) <= 1e-4 * scale)
    # and the oracle's own final pass: the same tables through the same algorithm
    assert np.all(np.abs(glo - olo) <= 1e-6 * scale) and np.all(np.abs(ghi - ohi) <= 1e-6 * scale)
    # seeded: push the spec through the last Linear on the host, start at the last hidden layer
    Wl, bl = wl.net.weights[-1].astype(np.float64), wl.net.biases[-1]
    a = (wl.spec.astype(np.float64) @ Wl).astype(np.float32)
    b = np.zeros(len(a), np.float32) if bl is None else (wl.spec.astype(np.float64) @ bl.astype(np.float64)).astype(np.float32)
    slo, shi = eng.crown_backward(layers[1:], None, wl.in_lo, wl.in_hi, seed=(a, a, b, b))
    # the frontier is taken as exact (gemm.rs:3380-3386): the seeded pass does not carry the first contraction's cast
    # and gamma terms, which the six layers below amplify to a few 1e-4 of the bound; it is the tighter of the two
    assert np.all(slo >= glo - 1e-6 * scale) and np.all(shi <= ghi + 1e-6 * scale)
    assert np.all(np.abs(slo - glo) <= 1e-3 * scale) and np.all(np.abs(shi - ghi) <= 1e-3 * scale)
    eng.release_network(nid)


def test_beta_adam_call_improves_and_matches_the_batch_optimiser(eng, oracle):
    wl = W.config_mlp_bab(seed=43, hidden=48, depth=3, n_in=40, eps=0.03, n_fix=4)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    D = 32
    splits, ns = W.draw_domains(wl, rl, ru, D)
    splits["beta"] = 0.0
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    glo, ghi, ginf = eng.batch_download()
    pl, pu = eng.batch_download_pre_bounds()
    feas = np.flatnonzero(ginf == 0)
    domains = []
    for d in feas:
        tabs = _domain_tables(wl, pl[d], pu[d], splits[d], int(ns[d]))
        domains.append({"layers": _layers(wl, tabs), "lo": wl.in_lo, "hi": wl.in_hi, "node_abs": [t[4] for t in tabs][::-1],
                        "beta_signed": [t[3] for t in tabs][::-1], "splits": splits[d][: ns[d]]})
    blo, bhi, beta = eng.crown_resnet_beta_batched_adam(domains, wl.spec, iterations=6, beta_lr=0.05, tolerance=0.0)
    gscale = np.abs(glo[feas]).max(axis=1, keepdims=True)
    assert np.all(blo >= glo[feas] - 2e-5 * gscale) and blo.sum() > glo[feas].sum()   # (the baked route's charge is a little larger)
    assert np.all(beta >= 0)
    # the same optimisation through the split-list batch: AMSGrad rule, beta only
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_optimize(6, 0.0, 0.05, lr_decay=1.0, clip_beta=0.0, rule=2)
    rlo, rhi, _ = eng.batch_download()
    scale = np.abs(rlo[feas]).max(axis=1, keepdims=True)
    assert np.all(np.abs(blo - rlo[feas]) <= 1e-4 * scale)
    eng.release_network(nid)


def test_gemm_f64_triplet(eng):
    g = np.random.Generator(np.random.PCG64(9))
    m, k, n = 37, 129, 65
    a = g.standard_normal((m, k)); w = g.standard_normal((k, n)); err = np.abs(g.standard_normal((m, k))) * 1e-7
    c = eng.gemm_f64_triplet(m, k, n, [a, np.abs(a), err], [w, np.abs(w), np.abs(w)])
    for got, (x, y) in zip(c, [(a, w), (np.abs(a), np.abs(w)), (err, np.abs(w))]):
        exact = x @ y
        assert np.max(np.abs(got - exact)) <= 1e-13 * np.max(np.abs(x) @ np.abs(y))
    one = eng.gemm_f64(m, k, n, a, w)
    assert np.array_equal(c[0], one)
