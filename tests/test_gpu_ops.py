"""The stand-alone operators of the engine trait (binary64 product, fused transposed convolution), the cooperative
deadline, the exported joint gradient and the batched point gradients."""
import numpy as np
import pytest

from ny_b200 import ConvTransposeParams, EngineError, engine
from ny_b200 import workloads as W
from test_gpu_parity import _setup

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["tf32x3", "f64"])
def eng(request):
    from ny_b200 import B200Engine

    e = B200Engine(0)
    e.set_path(engine.PATH_TF32X3 if request.param == "tf32x3" else engine.PATH_F64)
    e.path_name = request.param
    yield e
    e.close()


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (65, 17, 33), (200, 300, 130), (3, 1000, 2)])
def test_gemm_f64_is_a_binary64_product(eng, m, k, n):
    g = np.random.Generator(np.random.PCG64(m * 1000 + n))
    a, b = g.standard_normal((m, k)), g.standard_normal((k, n))
    c = eng.gemm_f64(m, k, n, a, b)
    # one fused multiply-add chain over k per element: inside the standard bound gamma_k |A||B| of the exact product
    exact = (a.astype(np.longdouble) @ b.astype(np.longdouble)).astype(np.float64)
    bound = (k + 1) * 2.0 ** -53 * (np.abs(a) @ np.abs(b)) + 1e-300
    assert np.all(np.abs(c - exact) <= bound)
    # and reproducible: the same chain in numpy (k increasing, fma = exact product + one rounding) for a small case
    if m * n <= 4:
        ref = np.zeros((m, n))
        for i in range(m):
            for j in range(n):
                acc = np.longdouble(0)
                for kk in range(k):
                    acc = np.longdouble(np.float64(np.longdouble(a[i, kk]) * np.longdouble(b[kk, j]) + acc))
                ref[i, j] = float(acc)
        assert np.allclose(c, ref, rtol=1e-15, atol=0)
    with pytest.raises(EngineError):
        eng.gemm_f64(m, k + 1, n, a, b)


@pytest.mark.parametrize("ic,ih,iw,oc,kh,kw,sh,sw,ph,pw", [
    (3, 32, 32, 16, 4, 4, 2, 2, 1, 1),      # first convolution of the CNN configuration
    (16, 16, 16, 32, 4, 4, 2, 2, 1, 1),     # its second
    (5, 9, 7, 4, 3, 3, 1, 1, 1, 1),         # stride 1, odd sizes
    (2, 8, 11, 3, 3, 2, 2, 3, 0, 1),        # ragged kernel / stride / padding
])
def test_conv_transpose_2d_matches_the_dense_lowering(eng, oracle, ic, ih, iw, oc, kh, kw, sh, sw, ph, pw):
    g = np.random.Generator(np.random.PCG64(ic * 100 + oc))
    w = g.standard_normal((oc, ic, kh, kw)).astype(np.float32)
    oh, ow = (ih + 2 * ph - kh) // sh + 1, (iw + 2 * pw - kw) // sw + 1
    S = 5
    a_nchw = g.standard_normal((S, oc, oh, ow)).astype(np.float32)
    a_reshaped = np.ascontiguousarray(a_nchw.transpose(0, 2, 3, 1)).reshape(S * oh * ow, oc)   # pixel-major, channel-minor
    p = ConvTransposeParams(S, oc, ic, oh, ow, ih, iw, kh, kw, sh, sw, ph, pw)
    out = eng.conv_transpose_2d(a_reshaped, w.reshape(oc, ic * kh * kw), p)
    dense, _ = oracle.conv2d_dense(w, None, (sh, sw), (ph, pw), (ih, iw))
    ref = a_nchw.reshape(S, -1).astype(np.float64) @ dense.astype(np.float64)
    mag = np.abs(a_nchw.reshape(S, -1)).astype(np.float64) @ np.abs(dense).astype(np.float64)
    assert out.shape == ref.shape
    assert np.all(np.abs(out - ref) <= 2.0 ** -23 * np.abs(ref) + 1e-12 * mag)    # binary64 sum, one fp32 rounding
    bad = ConvTransposeParams(S, oc, ic, oh + 1, ow, ih, iw, kh, kw, sh, sw, ph, pw)
    with pytest.raises(EngineError) as ei:
        eng.conv_transpose_2d(np.zeros((S * (oh + 1) * ow, oc), np.float32), w.reshape(oc, -1), bad)
    assert ei.value.code == engine.SHAPE


def test_deadline_stops_between_units_of_work_and_clears(eng, oracle):
    wl = W.config_mlp_bab(seed=31, hidden=48, depth=3, n_in=40, eps=0.03, n_fix=3)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    splits, ns = W.draw_domains(wl, rl, ru, 32)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    want = eng.batch_download()
    eng.set_deadline(0.0)                      # already over: every multi-launch call must decline
    try:
        for call in (eng.batch_run, lambda: eng.batch_optimize(4), lambda: eng.batch_gradient(0),
                     lambda: eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi),
                     lambda: eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, wl.x0[None, :], 3, 0.01),
                     lambda: eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns),
                     lambda: eng.gemm_f64(2, 2, 2, np.eye(2), np.eye(2))):
            with pytest.raises(EngineError) as ei:
                call()
            assert ei.value.code == engine.DEADLINE
        eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
        with pytest.raises(EngineError) as ei:
            eng.batch_run()
        assert ei.value.code == engine.DEADLINE
        with pytest.raises(EngineError):       # an aborted run has no results
            eng.batch_download()
    finally:
        eng.set_deadline(None)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.set_deadline(3600.0)                   # far away: no effect
    eng.batch_run()
    got = eng.batch_download()
    eng.set_deadline(None)
    for a, b in zip(want, got):
        assert np.array_equal(a, b)
    eng.release_network(nid)


@pytest.mark.parametrize("objective", [0, 1])
def test_joint_gradient_matches_oracle(eng, oracle, objective):
    wl = W.config_mlp_bab(seed=33, hidden=40, depth=3, n_in=30, eps=0.04, n_fix=3)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    D, S = 24, wl.spec.shape[0]
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.set_refine_tolerance(0.0)              # both evaluations on the same contraction path, no binary64 re-run
    eng.set_fusion(False)                      # the gradient's pass keeps per-layer checkpoints: one launch per layer
    try:
        grad = eng.batch_gradient(objective)
        lo, hi, inf = eng.batch_download()
        eng.batch_run()
        plo, phi, _ = eng.batch_download()
    finally:
        eng.set_refine_tolerance(5e-5)
        eng.set_fusion(True)
    assert np.array_equal(lo, plo) and np.array_equal(hi, phi)       # the evaluation is the plain bound
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    n_hidden = int(wl.net.dims[1:-1].sum())
    offs = np.concatenate([[0], np.cumsum(wl.net.dims[1:-1])])
    checked = 0
    for d in range(D):
        sp = splits[d][: ns[d]]
        pl, pu, bad = oracle.domain_bounds(ospec, wl.in_lo, wl.in_hi, rl2, ru2, sp, 1)
        assert bool(inf[d]) == bool(bad)
        if bad:
            continue
        a0 = oracle.heuristic_alpha(ospec, pl, pu)
        row = -1 if objective == 0 else int(np.argmin(lo[d]))      # the device ascends its own smallest row
        low, ga, gb = oracle.joint_gradient(ospec, wl.in_lo, wl.in_hi, pl, pu, sp, a0, only_row=row)
        m = ((pl < 0) & (pu > 0))[:n_hidden].copy()
        idx = [int(offs[s["relu"]] + s["neuron"]) for s in sp]
        m[idx] = False
        scale = max(float(np.abs(ga[:n_hidden]).max()), float(np.abs(gb).max()) if len(gb) else 0.0, 1e-6)
        assert np.abs(grad[d][:n_hidden][m] - ga[:n_hidden][m]).max() <= 2e-3 * scale
        if len(idx):
            assert np.abs(grad[d][idx] - gb).max() <= 2e-3 * scale
        rest = np.ones(n_hidden, bool)
        rest[m] = False
        rest[idx] = False
        assert np.all(grad[d][:n_hidden][rest] == 0) and np.all(grad[d][n_hidden:] == 0)
        checked += 1
    assert checked > D // 2
    with pytest.raises(EngineError):
        eng.batch_gradient(2)
    eng.release_network(nid)


def test_point_vjp_batched_matches_numpy(eng):
    wl = W.config_mlp_bab(seed=35, hidden=56, depth=3, n_in=37, n_out=6, eps=0.1, n_fix=0)
    net = wl.net
    nid = eng.register_network(net)
    K = 70
    g = np.random.Generator(np.random.PCG64(9))
    x = (wl.in_lo + g.random((K, 37), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)
    rows = g.standard_normal((K, 6)).astype(np.float32)        # a different cotangent per restart
    # numpy: forward in binary64, masks, reverse chain
    z = x.astype(np.float64)
    masks = []
    for k, (w, b) in enumerate(zip(net.weights, net.biases)):
        z = z @ w.astype(np.float64).T + b.astype(np.float64)
        if k < len(net.weights) - 1:
            masks.append(z > 0)
            z = np.maximum(z, 0)
    vals = (rows.astype(np.float64) * z).sum(axis=1)
    gr = rows.astype(np.float64)
    for k in range(len(net.weights) - 1, -1, -1):
        if k < len(net.weights) - 1:
            gr = gr * masks[k]
        gr = gr @ net.weights[k].astype(np.float64)
    tol = 1e-5 if eng.path_name == "f64" else 2e-4
    got, gv = eng.point_vjp_batched(nid, rows, x=x)
    scale = np.abs(gr).max()
    assert np.abs(got - gr).max() <= tol * scale and np.abs(gv - vals).max() <= tol * max(1.0, np.abs(vals).max())
    # caller-supplied masks: the same gradients; an all-ones mask gives the purely linear chain
    mk = np.zeros((K, net.n_pre), np.float32)
    mk[:, : sum(m.shape[1] for m in masks)] = np.concatenate(masks, axis=1)
    got2 = eng.point_vjp_batched(nid, rows, masks=mk)
    assert np.abs(got2 - gr).max() <= tol * scale
    lin = rows.astype(np.float64)
    for k in range(len(net.weights) - 1, -1, -1):
        lin = lin @ net.weights[k].astype(np.float64)
    got3 = eng.point_vjp_batched(nid, rows, masks=np.ones((K, net.n_pre), np.float32))
    assert np.abs(got3 - lin).max() <= tol * np.abs(lin).max()
    with pytest.raises(EngineError):
        eng.point_vjp_batched(nid, rows)
    with pytest.raises(EngineError):
        eng.point_vjp_batched(nid, rows, x=x, masks=mk)
    eng.release_network(nid)


def test_babsr_scores_and_picks_match_oracle(eng, oracle):
    wl = W.config_mlp_bab(seed=37, hidden=40, depth=3, n_in=30, eps=0.04, n_fix=3)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    D = 32
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    _, _, inf = eng.batch_download()
    relu, neuron, best = eng.batch_select_branch(2)
    scores, backups = eng.batch_branch_scores(with_backup=True)
    assert np.array_equal(scores, eng.batch_branch_scores())
    pl, pu = eng.batch_download_pre_bounds()
    dims = wl.net.dims
    offs = np.concatenate([[0], np.cumsum(dims[1:])]).astype(int)
    n_hidden = int(offs[len(wl.net.weights) - 1])
    tol = 1e-5 if eng.path_name == "f64" else 1e-3
    agree = 0
    for d in range(D):
        mask = np.zeros(wl.net.n_pre, bool)
        for s in splits[d][: ns[d]]:
            mask[int(offs[s["relu"]] + s["neuron"])] = True
        sc, pick, bk = oracle.babsr_scores(wl.net.weights, wl.net.biases, wl.spec, pl[d], pu[d], mask, with_backup=True)
        got = scores[d][:n_hidden]
        gb = backups[d][:n_hidden]
        assert np.array_equal(gb > 0.5, bk > 0.5) and np.all(gb[bk <= 0.5] <= 0)
        if (bk <= 0.5).any():
            assert np.abs(gb - bk)[bk <= 0.5].max() <= tol * max(float(np.abs(bk[bk <= 0.5]).max()), 1e-6)
        assert np.array_equal(got < 0, sc < 0)                          # same candidate set
        assert np.all(scores[d][n_hidden:] == -1)
        cand = sc >= 0
        if cand.any():
            assert np.abs(got[cand] - sc[cand]).max() <= tol * max(float(sc[cand].max()), 1e-6)
            top = np.sort(sc[cand])[::-1]
            clear = len(top) == 1 or top[0] - top[1] > 4 * tol * top[0]
            if clear:
                assert (int(relu[d]), int(neuron[d])) == pick
                agree += 1
            assert abs(best[d] - top[0]) <= tol * max(float(top[0]), 1e-6)
        else:
            assert relu[d] == -1 and neuron[d] == -1
    assert agree >= D // 2
    # driven from the search: the BaBSR choice is a valid split everywhere (unstable, unsplit neuron)
    for d in range(D):
        if relu[d] >= 0:
            o = int(offs[relu[d]] + neuron[d])
            assert pl[d][o] < 0 < pu[d][o]
    eng.release_network(nid)



def test_babsr_on_the_reference_hand_computed_cases(eng):
    """The device's BaBSR scores and pick on the two hand-computed cases of the reference's branching tests
    (beta_crown/engine/tests/branching.rs:998-1143): 1.5 / 0.25 with neuron 0 chosen; 0.5 / 2.75 / 0.5 / 2.0 with
    relu0 neuron 1 chosen at 2.75.  The given pre-activation bounds are taken as they are (clamp-only child bounds)."""
    from ny_b200 import Network, SPLIT_DTYPE
    from test_oracle_beta_crown import _babsr_reference_cases

    for ws, bs, spec, lo, hi, scores, pick, best in _babsr_reference_cases():
        net = Network(ws, bs)
        nid = eng.register_network(net)
        n_hidden = int(net.dims[1:-1].sum())
        box_lo, box_hi = -np.ones(2, np.float32), np.ones(2, np.float32)
        eng.batch_upload(nid, spec, box_lo, box_hi, lo[:net.n_pre], hi[:net.n_pre], np.zeros((1, 1), SPLIT_DTYPE),
                         np.zeros(1, np.int32), mode=0)
        eng.batch_run()
        relu, neuron, _ = eng.batch_select_branch(2)
        sc = eng.batch_branch_scores()[0][:n_hidden]
        assert (int(relu[0]), int(neuron[0])) == pick
        assert np.allclose(sc, scores, atol=1e-5) and abs(float(sc.max()) - best) < 1e-5
        eng.release_network(nid)
