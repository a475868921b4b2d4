"""The fused backward chain (all hidden layers' contractions and relaxations in one kernel, rows kept on the SM)
against the per-layer launches and against the CPU oracle, through the C ABI.  Both device routes apply the same
per-coefficient relaxation arithmetic; they differ in the accumulation order of the tensor-core sums, so their bounds
agree to within their certified rounding charges (a few 1e-5 of the domain's scale, asserted at 1e-4), and each
agrees with the oracle to the 1e-4 bar."""
import numpy as np
import pytest

from ny_b200 import workloads as W
from test_gpu_parity import _rel, REL_TOL, _oracle_batch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from ny_b200 import B200Engine

    e = B200Engine(0)
    yield e
    e.close()


def _both(eng, nid, wl, rl, ru, splits, ns, mode, alpha=None):
    """Both routes on the tensor path alone (no binary64 re-evaluation of domains whose rounding charge shows: the two
    routes certify different charges, so they would send different domains there)."""
    eng.set_refine_tolerance(0.0)
    try:
        return _both_raw(eng, nid, wl, rl, ru, splits, ns, mode, alpha)
    finally:
        eng.set_refine_tolerance(5e-5)


def _both_raw(eng, nid, wl, rl, ru, splits, ns, mode, alpha=None):
    eng.set_fusion(True)
    l0 = eng.launch_count()
    f = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=mode, alpha=alpha)
    n_fused = eng.launch_count() - l0
    eng.set_fusion(False)
    try:
        l0 = eng.launch_count()
        u = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=mode, alpha=alpha)
        n_unfused = eng.launch_count() - l0
    finally:
        eng.set_fusion(True)
    return f, u, n_fused, n_unfused


@pytest.mark.parametrize("hidden,depth,n_in,D", [(256, 4, 196, 300), (100, 3, 64, 130), (36, 5, 50, 71), (256, 8, 784, 512)])
def test_fused_chain_matches_per_layer_launches_and_oracle(eng, oracle, hidden, depth, n_in, D):
    wl = W.config_mlp_bab(seed=hidden + depth, hidden=hidden, depth=depth, n_in=n_in, eps=0.01, n_fix=6)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    ospec = onet.with_spec(wl.spec)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    splits, ns = W.draw_domains(wl, rl, ru, D)
    ns = ns.copy()
    ns[0] = 0
    ns[1] = 1
    (flo, fhi, finf), (ulo, uhi, uinf), n_fused, n_unfused = _both(eng, nid, wl, rl, ru, splits, ns, 1)
    assert np.array_equal(finf, uinf)
    feas = finf == 0
    scale = np.maximum(np.abs(ulo[feas]).max(axis=1, keepdims=True), np.abs(uhi[feas]).max(axis=1, keepdims=True))
    assert np.all(np.abs(flo[feas] - ulo[feas]) <= 1e-4 * scale) and np.all(np.abs(fhi[feas] - uhi[feas]) <= 1e-4 * scale)
    # with the default refinement on, the fused route against the oracle
    flo, fhi, finf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    n_or = min(D, 96)
    olo, ohi, oinf, _ = _oracle_batch(oracle, ospec, wl, rl, ru, splits[:n_or], ns[:n_or], 1)
    assert np.array_equal(finf[:n_or].astype(bool), oinf.astype(bool))
    f2 = ~oinf.astype(bool)
    both = np.concatenate([olo, ohi], axis=1)
    assert _rel(np.concatenate([flo[:n_or], fhi[:n_or]], axis=1)[f2], both[f2]) <= REL_TOL
    # sound against sampled executions of the unsplit domain
    mn = W.sample_min_margin(wl, 20000, 5)
    assert np.all(flo[0] <= mn)
    eng.release_network(nid)


def test_fused_chain_with_explicit_alpha_and_clamp_only_mode(eng, oracle):
    wl = W.config_mlp_bab(seed=77, hidden=128, depth=4, n_in=100, eps=0.02, n_fix=5)
    onet = oracle.Net(wl.net.weights, wl.net.biases)
    nid = eng.register_network(wl.net)
    rl, ru = oracle.ibp_forward(onet, wl.in_lo, wl.in_hi)
    D = 140
    splits, ns = W.draw_domains(wl, rl, ru, D)
    rng = np.random.default_rng(1)
    alpha = rng.uniform(0, 1, size=(D, wl.net.n_pre)).astype(np.float32)
    for mode in (0, 1):
        (flo, fhi, finf), (ulo, uhi, uinf), _, _ = _both(eng, nid, wl, rl, ru, splits, ns, mode, alpha)
        assert np.array_equal(finf, uinf)
        feas = finf == 0
        scale = np.maximum(np.abs(ulo[feas]).max(axis=1, keepdims=True), np.abs(uhi[feas]).max(axis=1, keepdims=True))
        assert np.all(np.abs(flo[feas] - ulo[feas]) <= 1e-4 * scale) and np.all(np.abs(fhi[feas] - uhi[feas]) <= 1e-4 * scale)
    eng.release_network(nid)


def test_fused_partial_passes_in_the_crown_pipeline(eng, oracle):
    """nyb200_crown_bounds seeds identity rows at every hidden layer (2 n_k rows per box): those partial passes go
    through the fused chain too."""
    wl = W.config_mlp_bab(seed=91, hidden=64, depth=4, n_in=40, eps=0.01)
    nid = eng.register_network(wl.net)
    lo, hi = W.draw_input_cells(wl, 3)
    eng.set_refine_tolerance(0.0)   # compare the two routes on the tensor path alone
    eng.set_fusion(True)
    flo, fhi, fil, fiu = eng.crown_bounds(nid, wl.spec, lo, hi)
    eng.set_fusion(False)
    try:
        ulo, uhi, uil, uiu = eng.crown_bounds(nid, wl.spec, lo, hi)
    finally:
        eng.set_fusion(True)
        eng.set_refine_tolerance(5e-5)
    flo2, fhi2, _, _ = eng.crown_bounds(nid, wl.spec, lo, hi)   # default settings for the oracle comparison below
    scale = np.abs(ulo).max(axis=1, keepdims=True)
    assert np.all(np.abs(flo - ulo) <= 1e-4 * scale) and np.all(np.abs(fhi - uhi) <= 1e-4 * scale)
    iscale = np.maximum(np.abs(uil), np.abs(uiu)).max(axis=1, keepdims=True)
    assert np.all(np.abs(fil - uil) <= 1e-4 * iscale) and np.all(np.abs(fiu - uiu) <= 1e-4 * iscale)
    onet = oracle.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    for d in range(0, lo.shape[0], 3):
        # against the oracle without its carried error matrices (the default convention discharges roundings layer by
        # layer and is tighter than the reference's carried channel on a depth-4 net by more than 1e-4)
        olo, ohi = oracle.crown(onet, lo[d], hi[d], error_channel=False)
        sc = max(np.abs(olo).max(), np.abs(ohi).max())
        assert np.all(np.abs(flo2[d] - olo) <= 2e-4 * sc) and np.all(np.abs(fhi2[d] - ohi) <= 2e-4 * sc), d
    eng.release_network(nid)
