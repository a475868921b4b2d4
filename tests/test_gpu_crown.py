"""GPU tests of the plain-CROWN pipeline (CROWN-IBP intermediate bounds): the device result against the reference's
own golden values (crates/ny-propagate/src/tests/crown/reference.rs, the same numbers that pin the oracle) and
against the oracle on seeded networks, including the reference's CPU-runnable configuration
(MLP 5 -> 6x50 -> 5, box x0 +- 0.05, 4 rows y0 - yj)."""
import numpy as np
import pytest

from ny_b200 import workloads as W
from test_gpu_parity import _rel, REL_TOL
from test_oracle_golden import B1, B2, B3, FC1, FC2, FC3

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["tf32x3", "f64"])
def eng(request):
    from ny_b200 import B200Engine, engine

    e = B200Engine(0)
    e.set_path(engine.PATH_TF32X3 if request.param == "tf32x3" else engine.PATH_F64)
    e.path_name = request.param
    yield e
    e.close()


def _net(weights, biases=None):
    from ny_b200 import Network

    return Network([np.asarray(w, np.float32) for w in weights],
                   None if biases is None else [np.asarray(b, np.float32) for b in biases])


def test_golden_toy_model(eng):
    """reference.rs:22-158: 2-2-1 net on [-1,2] x [-2,1]: CROWN [-3, 3]."""
    nid = eng.register_network(_net([[[1, -1], [2, -1]], [[1, -1]]]))
    lo, hi, _, _ = eng.crown_bounds(nid, np.eye(1, dtype=np.float32), [-1, -2], [2, 1])
    assert abs(lo[0, 0] - (-3.0)) < 1e-4 and abs(hi[0, 0] - 3.0) < 1e-4
    assert lo[0, 0] <= -3.0 and hi[0, 0] >= 3.0
    eng.release_network(nid)


def test_golden_deep_model(eng):
    """reference.rs:160-380: 3-4-4-2 MLP, eps 0.1 around 0.5: the published 8-digit CROWN bounds."""
    nid = eng.register_network(_net([FC1, FC2, FC3], [B1, B2, B3]))
    lo, hi, _, _ = eng.crown_bounds(nid, np.eye(2, dtype=np.float32), [0.4] * 3, [0.6] * 3)
    np.testing.assert_allclose(lo[0], [0.00820859, -0.01063502], atol=1e-4, rtol=0)   # the reference's own tolerance
    np.testing.assert_allclose(hi[0], [0.01113450, -0.00282869], atol=1e-4, rtol=0)
    tol = 2e-7 if eng.path_name == "f64" else 2e-6
    np.testing.assert_allclose(lo[0], [0.00820859, -0.01063502], atol=tol, rtol=0)
    np.testing.assert_allclose(hi[0], [0.01113450, -0.00282869], atol=tol, rtol=0)
    eng.release_network(nid)


def test_golden_tiny_model_intersection(eng):
    """reference.rs:382-467: 2-2-2 net on [0,1]^2, CROWN after the IBP intersection: [0, 1.5] and [0, 1]."""
    nid = eng.register_network(_net([[[1, 1], [1, -1]], [[1, 0], [0, 1]]], [[-0.5, 0], [0, 0]]))
    lo, hi, _, _ = eng.crown_bounds(nid, np.eye(2, dtype=np.float32), [0, 0], [1, 1])
    np.testing.assert_allclose(lo[0], [0, 0], atol=1e-5)
    np.testing.assert_allclose(hi[0], [1.5, 1.0], atol=1e-5)
    eng.release_network(nid)


@pytest.mark.parametrize("cfg", ["cpu_config", "mid"])
def test_crown_between_reference_and_exact_arithmetic(eng, oracle, cfg):
    """On deeper networks the reference's plain-CROWN bound carries a certified per-coefficient error matrix
    through every layer (err' = cast + gamma*S + err*|W|), which grows with the product of the layers' |W| norms:
    at depth 6 it loosens the bound by about 2e-3 of its value.  The device discharges every rounding at the
    layer where it occurs, so its bound is tighter than the reference's and cannot agree with it to 1e-4; what is
    asserted instead is the order  reference <= device <= exact-arithmetic CROWN  (the device is never looser
    than the reference and never beats the value of the same algorithm in exact arithmetic), closeness to the
    exact value, agreement with the oracle once its error channel is left out, and sampled soundness."""
    wl = W.config_mlp_small() if cfg == "cpu_config" else W.config_mlp_bab(seed=51, hidden=64, depth=4, n_in=100, eps=0.01)
    onet = oracle.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    glo, ghi, gil, giu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    olo, ohi = oracle.crown(onet, wl.in_lo, wl.in_hi)
    nlo, nhi = oracle.crown(onet, wl.in_lo, wl.in_hi, error_channel=False)
    (xlo, xhi), _ = oracle.crown_exact_f64(wl.net.weights, wl.net.biases, wl.spec, wl.in_lo, wl.in_hi)
    scale = max(np.abs(xlo).max(), np.abs(xhi).max())
    tiny = 1e-6 * scale
    assert np.all(glo[0] >= olo - tiny) and np.all(ghi[0] <= ohi + tiny)          # never looser than the reference
    assert np.all(glo[0] <= xlo + tiny) and np.all(ghi[0] >= xhi - tiny)          # never beats exact arithmetic
    assert np.all(np.abs(glo[0] - xlo) <= np.abs(olo - xlo) + tiny)               # at least as close as the reference
    assert np.abs(glo[0] - xlo).max() <= 1e-4 * scale and np.abs(ghi[0] - xhi).max() <= 1e-4 * scale
    assert np.abs(glo[0] - nlo).max() <= 2e-4 * scale and np.abs(ghi[0] - nhi).max() <= 2e-4 * scale
    mn = W.sample_min_margin(wl, 100000, 77)
    assert np.all(glo[0] <= mn)
    # CROWN is never looser than IBP on these rows
    ibl, ibu = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    S = wl.spec.shape[0]
    assert np.all(glo[0] >= ibl[-S:] - 1e-5 * np.abs(ibl[-S:]))
    eng.release_network(nid)


@pytest.mark.parametrize("cfg", ["cpu_config", "mid", "deep8"])
def test_crown_reference_error_channel_matches_the_reference_bound(eng, oracle, cfg):
    """With the reference's own error convention selected (per-coefficient error matrices carried to the input box,
    nyb200_set_error_channel(REFERENCE)), plain CROWN returns the reference's CPU bound on the CPU-runnable
    configuration (5 -> 6x50 -> 5), a mid-size network and an 8-layer one, where the default convention is 2e-3
    tighter.  The bar is 1e-4 of the bound vector's scale plus the pipeline's own conditioning: every layer's slopes
    are quotients of the previous layers' bounds, so a last-place difference in the first layer's bounds (summation
    order of the gamma term) grows about fivefold per layer; the oracle's answer to the same box widened by one fp32
    ulp measures that growth (3e-5 on the first network, 3e-4 on the 8-layer one), and the device has to stay within
    four times it.  The backward pass alone, fed identical slopes, agrees to 1e-6 (test_gpu_boundary.py)."""
    from ny_b200 import engine as E

    wl = {"cpu_config": lambda: W.config_mlp_small(),
          "mid": lambda: W.config_mlp_bab(seed=51, hidden=64, depth=4, n_in=100, eps=0.01),
          "deep8": lambda: W.config_mlp_bab(seed=53, hidden=48, depth=8, n_in=40, eps=0.005)}[cfg]()
    onet = oracle.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    eng.set_error_channel(E.ERRCH_REFERENCE)
    try:
        glo, ghi, gil, giu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    finally:
        eng.set_error_channel(E.ERRCH_IMMEDIATE)
    olo, ohi, oil, oiu = oracle.crown(onet, wl.in_lo, wl.in_hi, want_intermediate=True)
    wlo, whi, wil, wiu = oracle.crown(onet, np.nextafter(wl.in_lo, np.float32(-np.inf)),
                                      np.nextafter(wl.in_hi, np.float32(np.inf)), want_intermediate=True)
    n_pre = wl.net.n_pre
    cond = max(np.abs(wlo - olo).max(), np.abs(whi - ohi).max(),
               np.abs(wil[:n_pre] - oil[:n_pre]).max(), np.abs(wiu[:n_pre] - oiu[:n_pre]).max())

    def close(a, b):
        a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
        scale = np.abs(b[np.isfinite(b)]).max()
        return np.all(np.abs(a - b) <= 1e-4 * scale + 4.0 * cond)

    assert close(glo[0], olo) and close(ghi[0], ohi)
    assert close(gil[0], oil[:n_pre]) and close(giu[0], oiu[:n_pre])
    # and it is the looser of the two conventions
    dlo, dhi, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    scale = np.abs(olo).max()
    assert np.all(dlo[0] >= glo[0] - 1e-6 * scale) and np.all(dhi[0] <= ghi[0] + 1e-6 * scale)
    mn = W.sample_min_margin(wl, 100000, 78)
    assert np.all(glo[0] <= mn)
    eng.release_network(nid)


def test_crown_batch_of_boxes(eng, oracle):
    wl = W.config_mlp_bab(seed=52, hidden=48, depth=3, n_in=32, eps=0.02)
    onet = oracle.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    lo, hi = W.draw_input_cells(wl, 3)
    glo, ghi, _, _ = eng.crown_bounds(nid, wl.spec, lo, hi)
    for d in range(lo.shape[0]):
        olo, ohi = oracle.crown(onet, lo[d], hi[d])
        assert _rel(np.concatenate([glo[d], ghi[d]]), np.concatenate([olo, ohi])) <= REL_TOL, d
    one_lo, one_hi, _, _ = eng.crown_bounds(nid, wl.spec, lo[5], hi[5])
    assert np.array_equal(one_lo[0], glo[5]) and np.array_equal(one_hi[0], ghi[5])
    eng.release_network(nid)


def test_crown_under_relu_splits_matches_oracle_and_tightens_the_batch(eng, oracle):
    """Per-domain CROWN-tightened intermediate bounds for ReLU-split domains (nyb200_crown_bounds_split: the CROWN-IBP
    collection of network/ibp/crown_ibp.rs:32-420 under the clamps of constraints/lookups.rs:138-185): bounds,
    intermediates and infeasibility against the oracle's pipeline with the same clamps, sampled executions that satisfy
    the splits, the unsplit domain equal to the plain pipeline; then the same domains through the bound batch with
    their own tightened intermediates as inherited bounds (nyb200_batch_set_inherited), which may only help."""
    wl = W.config_mlp_bab(seed=57, hidden=40, depth=4, n_in=24, eps=0.03, n_fix=3)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = pl[0].copy(), pu[0].copy()
    D, S = 24, wl.spec.shape[0]
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    glo, ghi, gil, giu, ginf = eng.crown_bounds_split(nid, wl.spec, wl.in_lo, wl.in_hi, splits, ns)
    plo, phi, pil, piu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    assert np.array_equal(glo[0], plo[0]) and np.array_equal(gil[0], pil[0]) and ginf[0] == 0     # no split: the plain pipeline
    n_pre = wl.net.n_pre
    checked = 0
    for d in range(D):
        sp = splits[d][: ns[d]]
        olo, ohi, oil, oiu, oinf = oracle.crown_split(ospec, wl.in_lo, wl.in_hi, sp)
        assert bool(ginf[d]) == oinf, d
        if oinf:
            continue
        scale = max(np.abs(olo).max(), np.abs(ohi).max())
        assert np.all(np.abs(glo[d] - olo) <= 2e-4 * scale) and np.all(np.abs(ghi[d] - ohi) <= 2e-4 * scale), d
        iscale = max(np.abs(oil[:n_pre]).max(), np.abs(oiu[:n_pre]).max())
        assert np.all(np.abs(gil[d] - oil[:n_pre]) <= 2e-4 * iscale) and np.all(np.abs(giu[d] - oiu[:n_pre]) <= 2e-4 * iscale), d
        for s in sp:                                   # the clamps are visible in the returned intermediates
            o = int(np.concatenate([[0], np.cumsum(wl.net.dims[1:])])[s["relu"]] + s["neuron"])
            assert (gil[d][o] >= 0) if s["sign"] > 0 else (giu[d][o] <= 0)
        mn = W.sample_min_margin(wl, 20000, 400 + d, sp)
        ok = np.isfinite(mn)
        assert np.all(glo[d][ok] <= mn[ok]), d
        checked += 1
    assert checked > D // 2
    # the bound batch on the same domains: shared root bounds, then every domain's own tightened intermediates
    zero_beta = splits.copy()
    zero_beta["beta"] = 0.0
    b0, _, inf0 = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, zero_beta, ns, mode=1)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, zero_beta, ns, mode=1)
    eng.batch_set_inherited(gil, giu)
    eng.batch_run()
    b1, _, inf1 = eng.batch_download()
    ok = (inf0 == 0) & (inf1 == 0) & (ginf == 0)
    scale = np.abs(b0[ok]).max()
    assert ok.sum() > D // 2
    assert np.all(b1[ok] >= b0[ok] - 2e-4 * scale) and b1[ok].sum() > b0[ok].sum()
    for d in np.flatnonzero(ok)[:6]:
        mn = W.sample_min_margin(wl, 20000, 400 + d, splits[d][: ns[d]])
        fin = np.isfinite(mn)
        assert np.all(b1[d][fin] <= mn[fin]), d
    eng.release_network(nid)
