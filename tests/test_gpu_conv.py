"""GPU parity tests for networks with Conv2d layers: the interval convolution, the CROWN backward step as a
transposed convolution and the parameter adjoint through a convolution, against the oracle evaluated on the
dense lowering of the same layers (oracle.conv2d_dense, pinned to the reference's conv known answers)."""
import copy

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


def _setup_conv(eng, oracle, wl):
    ws, bs = oracle.lower_network(wl.net.weights, wl.net.biases)
    onet = oracle.Net(ws, bs)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    return onet, ospec, nid, rl, ru


def _small_cnn(seed=31, eps=0.02, n_fix=4):
    return W.config_cnn(seed=seed, eps=eps, n_fix=n_fix, in_chw=(2, 8, 8), convs=((4, 3, 1, 1), (6, 4, 2, 1)), fcs=(24, 5))


def _ext(rl, ru, S):
    return (np.concatenate([rl, np.full(S, -np.inf, np.float32)]), np.concatenate([ru, np.full(S, np.inf, np.float32)]))


def test_conv_known_answers_on_device(eng):
    """conv2d/tests.rs:46-66 and :561-584 through the device interval pass: y = 2x + 0.5 and y = -2x + 1 on a
    2x2 image with a 1x1 kernel."""
    from ny_b200 import Conv2d, Network

    lo = np.array([1, 2, 3, 4], np.float32)
    hi = np.array([5, 6, 7, 8], np.float32)
    for wv, bv, el, eu in ((2.0, 0.5, [2.5, 4.5, 6.5, 8.5], [10.5, 12.5, 14.5, 16.5]),
                           (-2.0, 1.0, [-9, -11, -13, -15], [-1, -3, -5, -7])):
        conv = Conv2d(np.full((1, 1, 1, 1), wv, np.float32), np.array([bv], np.float32), (1, 1), (0, 0), (2, 2))
        nid = eng.register_network(Network([conv, np.eye(4, dtype=np.float32)], [None, None]))
        pl, pu = eng.ibp_forward_gpu(nid, lo, hi)
        assert np.allclose(pl[0][:4], el, atol=1e-5) and np.allclose(pu[0][:4], eu, atol=1e-5)
        assert np.all(pl[0][:4] <= el) and np.all(pu[0][:4] >= eu)
        eng.release_network(nid)


def test_conv_geometry_and_nan_kernels_are_refused(eng):
    """Zero stride, an output size that does not match the geometry and non-finite kernels are errors
    (conv2d/tests.rs:874-927, :1169-1200), never a silently wrong bound."""
    import ctypes as C

    from ny_b200 import EngineError
    from ny_b200.engine import LayerDesc, _fp

    def create(desc, w):
        descs = (LayerDesc * 1)(desc)
        nid = C.c_int32(0)
        w = np.ascontiguousarray(w, np.float32)
        return eng._L.nyb200_net_create_layers(eng._h, 1, descs, _fp(w), None, C.byref(nid))

    good = LayerDesc(1, 16, 9, 0, 1, 4, 4, 1, 3, 3, 2, 2, 1, 1, 0, 0)
    assert create(good, np.ones(4)) == 0
    zero_stride = LayerDesc(1, 16, 9, 0, 1, 4, 4, 1, 3, 3, 2, 2, 0, 1, 0, 0)
    assert create(zero_stride, np.ones(4)) == 2
    wrong_out = LayerDesc(1, 16, 16, 0, 1, 4, 4, 1, 4, 4, 2, 2, 1, 1, 0, 0)
    assert create(wrong_out, np.ones(4)) == 2
    big_kernel = LayerDesc(1, 4, 1, 0, 1, 2, 2, 1, 1, 1, 3, 3, 1, 1, 0, 0)
    assert create(big_kernel, np.ones(9)) == 2
    assert create(good, np.array([1, np.nan, 1, 1])) == 4
    with pytest.raises(EngineError):
        from ny_b200 import Conv2d

        Conv2d(np.ones((1, 1, 2, 2), np.float32), None, (0, 1), (0, 0), (4, 4))


def test_conv_ibp_matches_oracle(eng, oracle):
    wl = _small_cnn()
    onet, _, nid, rl, ru = _setup_conv(eng, oracle, wl)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    tol = IBP_REL * np.maximum(np.abs(rl), np.abs(ru)) + 1e-7
    assert np.all(np.abs(pl[0] - rl) <= tol) and np.all(np.abs(pu[0] - ru) <= tol)
    lo2 = np.stack([wl.in_lo, wl.in_lo + 0.25 * (wl.in_hi - wl.in_lo)])
    hi2 = np.stack([wl.in_hi, wl.in_hi - 0.25 * (wl.in_hi - wl.in_lo)])
    pl2, pu2 = eng.ibp_forward_gpu(nid, lo2, hi2)
    r2l, r2u = oracle.ibp_forward(onet, lo2[1], hi2[1])
    assert np.all(np.abs(pl2[1] - r2l) <= tol) and np.all(np.abs(pu2[1] - r2u) <= tol)
    eng.release_network(nid)


@pytest.mark.parametrize("mode", [0, 1])
def test_conv_bab_bound_batch_matches_oracle(eng, oracle, mode):
    wl = _small_cnn(seed=32)
    onet, ospec, nid, rl, ru = _setup_conv(eng, oracle, wl)
    D = 72
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    ns[1] = 1
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=mode)
    rl2, ru2 = _ext(rl, ru, wl.spec.shape[0])
    olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits, ns, mode)
    assert np.array_equal(ginf.astype(bool), oinf.astype(bool))
    feas = ~oinf.astype(bool)
    assert feas.sum() > D // 2
    assert _rel(np.concatenate([glo, ghi], axis=1)[feas], np.concatenate([olo, ohi], axis=1)[feas]) <= REL_TOL
    for d in np.flatnonzero(feas)[:6]:
        mn = W.sample_min_margin(wl, 20000, 700 + d, splits[d][: ns[d]])
        ok = np.isfinite(mn)
        assert np.all(glo[d][ok] <= mn[ok]), d
    eng.release_network(nid)


def test_conv_optimisation_matches_oracle(eng, oracle):
    wl = _small_cnn(seed=33, eps=0.03)
    onet, ospec, nid, rl, ru = _setup_conv(eng, oracle, wl)
    D, iters = 40, 8
    splits, ns = W.draw_domains(wl, rl, ru, D)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_optimize(iters, 0.1, 0.05)
    glo, ghi, ginf = eng.batch_download()
    rl2, ru2 = _ext(rl, ru, wl.spec.shape[0])
    checked = 0
    for d in range(D):
        sp = splits[d][: ns[d]]
        pl, pu, bad = oracle.domain_bounds(ospec, wl.in_lo, wl.in_hi, rl2, ru2, sp, 1)
        assert bool(ginf[d]) == bool(bad)
        if bad:
            continue
        olo, ohi, _, _ = oracle.optimize(ospec, wl.in_lo, wl.in_hi, pl, pu, sp, oracle.heuristic_alpha(ospec, pl, pu),
                                         iters, 0.1, 0.05)
        assert _rel(np.concatenate([glo[d], ghi[d]]), np.concatenate([olo, ohi])) <= 1e-3, d
        checked += 1
    assert checked > D // 2
    eng.release_network(nid)


def test_cnn_full_size_split_domains(eng, oracle):
    """CNN 3x32x32 -> conv(16,k4,s2,p1) -> conv(32,k4,s2,p1) -> FC 2048->100 -> FC 100->10, box +-2/255, 9 rows,
    1024 BaB domains fixing 8 unstable neurons each: whole-batch properties, oracle parity and sampled soundness
    on a few domains."""
    wl = W.config_cnn()
    onet, ospec, nid, rl, ru = _setup_conv(eng, oracle, wl)
    D = 1024
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    feas = ginf == 0
    assert feas.sum() > D // 2 and np.all(np.isfinite(glo[feas])) and np.all(glo[feas] <= ghi[feas])
    # a split domain is a subset of the root domain: with the same slopes and beta = 0 its bound could only
    # improve; with beta > 0 it stays a valid bound, so it must still enclose the domain's own samples
    rl2, ru2 = _ext(rl, ru, wl.spec.shape[0])
    for d in (0, 1, 513, 1023):
        sp = splits[d][: ns[d]]
        olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits[d:d + 1], ns[d:d + 1], 1)
        assert bool(oinf[0]) == bool(ginf[d])
        if oinf[0]:
            continue
        assert _rel(np.concatenate([glo[d], ghi[d]]), np.concatenate([olo[0], ohi[0]])) <= REL_TOL, d
        if d == 0:  # the unsplit domain: every sample of the box qualifies
            mn = W.sample_min_margin(wl, 4000, 8000, sp, chunk=1000)
            assert np.all(np.isfinite(mn)) and np.all(glo[d] <= mn)
    eng.release_network(nid)


def test_cnn_full_size_against_the_native_convolution_oracle(eng, oracle):
    """The same full-size configuration against the oracle's native convolution (kernel taps and the transposed
    convolution of the backward pass, layers/convolution/conv2d/bound.rs:86-268, 601-900; no dense lowering): the
    interval pass and six split domains of the 1024-domain batch."""
    wl = W.config_cnn()
    nat = oracle.Net(wl.net.weights, wl.net.biases)
    nid = eng.register_network(wl.net)
    nl, nu = oracle.ibp_forward(nat, wl.in_lo, wl.in_hi)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    n = wl.net.n_pre
    tol = 1e-5 * np.maximum(np.abs(nl[:n]), np.abs(nu[:n])) + 1e-6
    assert np.all(np.abs(pl[0] - nl[:n]) <= tol) and np.all(np.abs(pu[0] - nu[:n]) <= tol)
    rl, ru = pl[0].copy(), pu[0].copy()
    D = 1024
    splits, ns = W.draw_domains(wl, rl, ru, D)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    rl2, ru2 = _ext(rl, ru, wl.spec.shape[0])
    ospec = nat.with_spec(wl.spec)
    checked = 0
    for d in (0, 7, 300, 511, 777, 1023):
        olo, ohi, oinf, _ = oracle.bab_bound_batch(ospec, wl.in_lo, wl.in_hi, rl2, ru2, splits[d:d + 1], ns[d:d + 1], 1)
        assert bool(oinf[0]) == bool(ginf[d])
        if oinf[0]:
            continue
        assert _rel(np.concatenate([glo[d], ghi[d]]), np.concatenate([olo[0], ohi[0]])) <= REL_TOL, d
        checked += 1
    assert checked >= 4
    eng.release_network(nid)


def test_conv_crown_pipeline_matches_oracle(eng, oracle):
    """Plain CROWN with CROWN-IBP intermediates through convolutions (partial passes run transposed convolutions)
    against the oracle's pipeline on the dense lowering; this network is shallow enough for direct parity."""
    wl = _small_cnn(seed=34, eps=0.01)
    onet, ospec, nid, rl, ru = _setup_conv(eng, oracle, wl)
    glo, ghi, gil, giu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    olo, ohi = oracle.crown(ospec, wl.in_lo, wl.in_hi)
    nlo, nhi = oracle.crown(ospec, wl.in_lo, wl.in_hi, error_channel=False)
    scale = max(np.abs(olo).max(), np.abs(ohi).max())
    assert np.all(glo[0] >= olo - 1e-6 * scale) and np.all(ghi[0] <= ohi + 1e-6 * scale)   # never looser than the reference
    assert np.abs(glo[0] - nlo).max() <= 2e-4 * scale and np.abs(ghi[0] - nhi).max() <= 2e-4 * scale
    mn = W.sample_min_margin(wl, 50000, 31)
    assert np.all(glo[0] <= mn)
    eng.release_network(nid)
