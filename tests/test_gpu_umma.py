"""tcgen05 (3xTF32) contraction: checked through the C ABI against exact binary64 products, and
the whole beta-CROWN batch on that path against the CPU oracle."""
import numpy as np
import pytest

from ny_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from ny_b200 import B200Engine, engine

    e = B200Engine(0)
    e.set_path(engine.PATH_TF32X3)
    yield e
    e.close()


def _umma_eps(K):
    # rounding model of the kernel: operand split + 4 full-scale and 8 small tensor-memory steps per
    # 32-wide K chunk + fp32 chunk sums
    chunks = (K + 31) // 32
    return 0.75 * 2.0 ** -20 + 4 * 2.0 ** -23 + 8 * 2.0 ** -33 + chunks * 2.0 ** -24


@pytest.mark.parametrize("m,k,n", [(128, 32, 256), (128, 256, 256), (300, 256, 256), (1000, 10, 256),
                                   (257, 256, 784), (64, 50, 50), (5, 7, 3), (4096, 512, 512)])
def test_umma_gemm_within_rounding_model(eng, m, k, n):
    g = np.random.Generator(np.random.PCG64(m * 7 + k * 3 + n))
    a = (g.standard_normal((m, k)) * np.exp(g.uniform(-3, 3, (m, 1)))).astype(np.float32)
    b = g.standard_normal((k, n)).astype(np.float32)
    c = eng.gemm_f32(m, k, n, a, b)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    S = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    err = np.abs(c.astype(np.float64) - exact)
    ratio = float(np.max(err / np.maximum(S, 1e-300)))
    assert np.all(np.isfinite(c))
    assert ratio <= _umma_eps(k), (ratio, _umma_eps(k))


def test_umma_gemm_adversarial_same_sign_and_cancellation(eng):
    # all-positive operands maximise the accumulator magnitude; alternating signs maximise cancellation
    m, k, n = 256, 256, 256
    g = np.random.Generator(np.random.PCG64(99))
    for kind in ("positive", "alternating", "tiny_plus_huge"):
        a = g.random((m, k)).astype(np.float32) + 0.5
        b = g.random((k, n)).astype(np.float32) + 0.5
        if kind == "alternating":
            a[:, ::2] *= -1
        if kind == "tiny_plus_huge":
            a[:, :8] *= 1e6
            b[8:, :] *= 1e-3
        c = eng.gemm_f32(m, k, n, a, b)
        exact = a.astype(np.float64) @ b.astype(np.float64)
        S = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
        ratio = float(np.max(np.abs(c - exact) / S))
        assert ratio <= _umma_eps(k), (kind, ratio)


def test_batch_on_tensor_path_matches_oracle(eng, oracle):
    from tests.test_gpu_parity import REL_TOL, _oracle_batch, _rel, _setup

    wl = W.config_mlp_bab(seed=6, hidden=64, depth=4, n_in=196, eps=0.01, n_fix=8)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    splits, ns = W.draw_domains(wl, rl, ru, 200)
    glo, ghi, ginf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits, ns, 1)
    assert np.array_equal(ginf.astype(bool), oinf.astype(bool))
    f = ~oinf.astype(bool)
    both = np.concatenate([olo, ohi], axis=1)
    dev = _rel(np.concatenate([glo, ghi], axis=1)[f], both[f])
    print("max relative deviation on the tensor path:", dev)
    assert dev <= REL_TOL
    for d in range(0, 200, 25):
        if ginf[d]:
            continue
        mn = W.sample_min_margin(wl, 20000, 900 + d, splits[d][: ns[d]])
        ok = np.isfinite(mn)
        assert np.all(glo[d][ok] <= mn[ok])
    eng.release_network(nid)


def test_full_size_batch_on_tensor_path(eng, oracle):
    """Benchmark configuration (784 -> 8x256 -> 10, 4096 domains) on the tcgen05 path: parity with the
    oracle on a 32-domain sample, agreement with the binary64 device path, soundness on one domain."""
    from ny_b200 import B200Engine
    from tests.test_gpu_parity import REL_TOL, _oracle_batch, _rel

    wl = W.config_mlp_bab()
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = pl[0], pu[0]
    D = 4096
    splits, ns = W.draw_domains(wl, rl, ru, D)
    lo, hi, inf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    lo2, hi2, _ = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    assert np.array_equal(lo, lo2) and np.array_equal(hi, hi2)
    from ny_b200 import engine

    ref = B200Engine(0)
    ref.set_path(engine.PATH_F64)
    rid = ref.register_network(wl.net)
    flo, fhi, finf = ref.bab_bound_batch(rid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    ref.close()
    assert np.array_equal(inf, finf)
    feas = inf == 0
    dev64 = _rel(np.concatenate([lo, hi], 1)[feas], np.concatenate([flo, fhi], 1)[feas])
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    sel = np.arange(0, D, D // 32)
    olo, ohi, oinf, _ = _oracle_batch(oracle, onet.with_spec(wl.spec), wl, rl, ru, splits[sel], ns[sel], 1)
    f = ~oinf.astype(bool)
    dev = _rel(np.concatenate([lo, hi], 1)[sel][f], np.concatenate([olo, ohi], 1)[f])
    print("full-size tensor path: deviation vs binary64 device path", dev64, "vs oracle", dev)
    assert dev <= REL_TOL
    assert np.all(lo[feas] <= flo[feas] + 1e-6 * np.abs(flo[feas]).max(axis=1, keepdims=True))
    d = int(np.flatnonzero(feas)[0])
    mn = W.sample_min_margin(wl, 100000, 77, splits[d][: ns[d]])
    ok = np.isfinite(mn)
    assert np.all(lo[d][ok] <= mn[ok])
    eng.release_network(nid)


def test_narrow_box_triggers_binary64_rerun(eng, oracle):
    """A narrow input box makes every bound a small difference of large terms; the tensor path's rounding
    penalty is then visible at 1e-4, the engine notices it and re-evaluates the batch in binary64.  With the
    re-run disabled the bounds stay sound (never above the oracle's by more than fp32 noise) but looser."""
    from tests.test_gpu_parity import REL_TOL, _oracle_batch, _rel, _setup

    wl = W.config_mlp_bab(seed=21, hidden=64, depth=3, n_in=96, eps=0.01, n_fix=4)
    onet, ospec, nid, rl, ru = _setup(eng, oracle, wl)
    splits, ns = W.draw_domains(wl, rl, ru, 64)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits, ns, 1)
    f = ~oinf.astype(bool)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    eng.batch_run()
    glo, ghi, ginf = eng.batch_download()
    assert eng.batch_refined() > 0
    assert _rel(np.concatenate([glo, ghi], 1)[f], np.concatenate([olo, ohi], 1)[f]) <= REL_TOL
    eng.set_refine_tolerance(0.0)
    try:
        eng.batch_run()
        llo, lhi, _ = eng.batch_download()
        assert eng.batch_refined() == 0
        scale = np.abs(np.concatenate([olo, ohi], 1)).max(axis=1, keepdims=True)
        assert np.all(llo[f] <= olo[f] + 1e-6 * scale[f]) and np.all(lhi[f] >= ohi[f] - 1e-6 * scale[f])
        assert np.all(llo[f] <= glo[f] + 1e-6 * scale[f])
    finally:
        eng.set_refine_tolerance(5e-5)
    eng.release_network(nid)


def test_partial_rerun_touches_only_flagged_domains(eng, oracle):
    """A batch with a shared wide box where only some domains are narrow enough... is not constructible with one
    box, so the mix is built with per-domain boxes: a few cells of a wide box shrunk to slivers.  Only those are
    re-evaluated with binary64 contractions; every domain must agree with the oracle, and the ones that were not
    flagged must be bit-identical to a run with the re-evaluation switched off."""
    wl = W.config_mlp_bab(seed=72, hidden=96, depth=3, n_in=48, eps=0.05, n_fix=0)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    lo, hi = W.draw_input_cells(wl, 7)          # 128 cells
    D = lo.shape[0]
    narrow = np.arange(0, D, 9)
    mid = (lo[narrow].astype(np.float64) + hi[narrow]) / 2
    lo[narrow] = (mid - 1e-5 * (hi[narrow] - lo[narrow])).astype(np.float32)
    hi[narrow] = (mid + 1e-5 * (hi[narrow] - mid)).astype(np.float32)
    from ny_b200 import SPLIT_DTYPE
    sp0, ns = np.zeros((D, 0), SPLIT_DTYPE), np.zeros(D, np.int32)
    eng.batch_upload(nid, wl.spec, lo, hi, rl, ru, sp0, ns, mode=1)
    eng.set_refine_tolerance(0.0)
    try:
        eng.batch_run()
        flo, fhi, _ = eng.batch_download()
    finally:
        eng.set_refine_tolerance(5e-5)
    eng.batch_run()
    glo, ghi, ginf = eng.batch_download()
    refined = eng.batch_refined()
    assert 0 < refined < D // 2, refined
    changed = np.any(glo != flo, axis=1) | np.any(ghi != fhi, axis=1)
    assert 0 < changed.sum() <= refined
    assert np.all(np.isin(np.flatnonzero(changed), narrow))       # only slivers were re-evaluated
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    for d in list(narrow[:6]) + [1, 2, D - 1]:
        pl, pu, bad = oracle.domain_bounds(ospec, lo[d], hi[d], rl2, ru2, sp0[d], 1)
        olo, ohi = oracle.beta_crown_bound(ospec, lo[d], hi[d], pl, pu, sp0[d])
        both = np.concatenate([olo, ohi])
        den = np.maximum(np.abs(both), 1e-2 * np.abs(both).max())
        assert np.max(np.abs(np.concatenate([glo[d], ghi[d]]) - both) / den) <= 1e-4, d
    pl_all, pu_all = eng.batch_download_pre_bounds()
    assert np.all(pl_all <= pu_all)
    assert np.isclose(eng.batch_min_lower(), glo[ginf == 0].min())
    eng.release_network(nid)


def test_staged_operand_matches_direct_loads_bit_for_bit():
    """The fp32 A operand reaches the split either through the TMA staging ring (rows of K contiguous values whose
    base and stride are multiples of 16 bytes) or through direct global loads (anything else).  Padding A with one
    zero column and B with one zero row gives the same product through the other route (row stride K + 1 is not a
    multiple of 4 floats): the extra stage adds zeros, so the results must be identical bit for bit, and identical
    from call to call: at this size every CTA walks four tiles with the tensor core pacing the pipeline, the regime
    in which a missing proxy fence on the staging ring showed up as wrong later tiles."""
    from ny_b200 import B200Engine

    eng = B200Engine(0)
    g = np.random.Generator(np.random.PCG64(3))
    for (m, k, n) in [(73728, 256, 256), (20000, 256, 784), (9000, 100, 40)]:
        a = g.standard_normal((m, k), dtype=np.float32)
        b = g.standard_normal((k, n), dtype=np.float32)
        c = eng.gemm_f32(m, k, n, a, b)
        for rep in range(2):
            assert np.array_equal(c, eng.gemm_f32(m, k, n, a, b)), "call-to-call difference"
        a1 = np.concatenate([a, np.zeros((m, 1), np.float32)], axis=1)
        b1 = np.concatenate([b, np.zeros((1, n), np.float32)], axis=0)
        c1 = eng.gemm_f32(m, k + 1, n, a1, b1)
        assert np.array_equal(c, c1), (m, k, n)
    eng.close()
