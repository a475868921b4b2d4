"""GPU tests of the PGD attack batched over restarts against the numpy restatement in the oracle, on the same
starting points.  The step is a sign step, so a coordinate whose gradient is numerically zero may move the other
way on the device (3xTF32 or binary64 from fp32 operands) than in the binary64 restatement; the trajectories are
therefore compared through what the attack returns (objective values, monotone improvement, validity of the
reported points), the first step coordinate by coordinate where the gradient is not negligible."""
import numpy as np
import pytest

from ny_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["tf32x3", "f64"])
def eng(request):
    from ny_b200 import B200Engine, engine

    e = B200Engine(0)
    e.set_path(engine.PATH_TF32X3 if request.param == "tf32x3" else engine.PATH_F64)
    e.path_name = request.param
    yield e
    e.close()


def _starts(wl, K, seed):
    g = np.random.Generator(np.random.PCG64(seed))
    return (wl.in_lo + g.random((K, len(wl.in_lo)), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)


def _margin(wl, x):
    return (W.forward(wl.net, x) @ wl.spec.astype(np.float64).T).min(axis=1)


@pytest.mark.parametrize("kind", ["mlp", "cnn"])
def test_zero_steps_is_the_forward_pass(eng, oracle, kind):
    wl = (W.config_mlp_bab(seed=41, hidden=64, depth=3, n_in=48, eps=0.05) if kind == "mlp" else
          W.config_cnn(seed=42, eps=0.05, in_chw=(2, 8, 8), convs=((4, 3, 1, 1), (6, 4, 2, 1)), fcs=(24, 5)))
    nid = eng.register_network(wl.net)
    x0 = _starts(wl, 64, 1)
    best, bx, ce = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, 0, 0.01)
    want = _margin(wl, x0)
    assert np.array_equal(bx, x0)
    assert np.allclose(best, want, rtol=1e-5, atol=1e-6)
    assert ce == (int(np.argmin(best)) if best.min() <= 0 else -1)
    eng.release_network(nid)


@pytest.mark.parametrize("kind", ["mlp", "cnn"])
def test_first_step_follows_the_exact_gradient(eng, oracle, kind):
    wl = (W.config_mlp_bab(seed=43, hidden=64, depth=3, n_in=48, eps=0.05) if kind == "mlp" else
          W.config_cnn(seed=44, eps=0.05, in_chw=(2, 8, 8), convs=((4, 3, 1, 1), (6, 4, 2, 1)), fcs=(24, 5)))
    nid = eng.register_network(wl.net)
    K = 32
    # start in the middle of the box so that no coordinate is clipped by the first step
    x0 = np.repeat(((wl.in_lo.astype(np.float64) + wl.in_hi) / 2).astype(np.float32)[None, :], K, axis=0)
    x0 += (_starts(wl, K, 2) - x0) * np.float32(0.2)
    step = 0.1 * float((wl.in_hi - wl.in_lo).max()) / 2
    _, bx, _ = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, 1, step)
    ws, bs = oracle.lower_network(wl.net.weights, wl.net.biases)
    # exact gradient of the worst row at x0
    acts, z = [], x0.astype(np.float64)
    for k, w in enumerate(ws):
        z = z @ np.asarray(w, np.float64).T + (0 if bs[k] is None else np.asarray(bs[k], np.float64))
        if k + 1 < len(ws):
            z = np.maximum(z, 0)
        acts.append(z)
    marg = acts[-1] @ wl.spec.astype(np.float64).T
    g = wl.spec.astype(np.float64)[np.argmin(marg, axis=1)]
    for k in range(len(ws) - 1, -1, -1):
        if k + 1 < len(ws):
            g = g * (acts[k] > 0)
        g = g @ np.asarray(ws[k], np.float64)
    # the point kept after one step is x0 or x1, whichever has the smaller objective; recover x1 from both cases
    moved = np.any(bx != x0, axis=1)
    assert moved.sum() > K // 2
    clear = np.abs(g) > 1e-4 * np.abs(g).max(axis=1, keepdims=True)
    want = x0 - np.sign(g).astype(np.float32) * np.float32(step / (1 - 0.9))  # bias correction 1 - beta1 at t = 1
    want = np.clip(want, wl.in_lo, wl.in_hi)
    sel = moved[:, None] & clear
    assert np.allclose(bx[sel], want[sel], atol=1e-6)
    eng.release_network(nid)


@pytest.mark.parametrize("kind", ["mlp", "cnn"])
def test_attack_matches_restatement_and_reports_valid_points(eng, oracle, kind):
    wl = (W.config_mlp_bab(seed=45, hidden=64, depth=3, n_in=48, eps=0.08) if kind == "mlp" else
          W.config_cnn(seed=46, eps=0.08, in_chw=(2, 8, 8), convs=((4, 3, 1, 1), (6, 4, 2, 1)), fcs=(24, 5)))
    nid = eng.register_network(wl.net)
    K, steps = 96, 30
    x0 = _starts(wl, K, 3)
    eps = float((wl.in_hi - wl.in_lo).max()) / 2
    best, bx, ce = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, steps, 0.25 * eps)
    # reported points are inside the box and the reported values are their true objectives
    assert np.all(bx >= wl.in_lo) and np.all(bx <= wl.in_hi)
    true = _margin(wl, bx)
    assert np.allclose(best, true, rtol=1e-5, atol=1e-6)
    start = _margin(wl, x0)
    assert np.all(best <= start + 1e-6) and best.mean() < start.mean()
    assert ce == (int(np.argmin(best)) if best.min() <= 0 else -1)
    ws, bs = oracle.lower_network(wl.net.weights, wl.net.biases)
    obest, obx = oracle.pgd_attack(ws, bs, wl.spec, wl.in_lo, wl.in_hi, x0, steps, 0.25 * eps)
    scale = np.abs(start).mean()
    # same attack strength: per restart within a few percent of the objective scale, on average much closer
    assert np.abs(best - obest).max() <= 0.05 * scale
    assert np.abs(best - obest).mean() <= 0.005 * scale
    assert (best.min() <= 0) == (obest.min() <= 0) or abs(best.min() - obest.min()) <= 0.01 * scale
    eng.release_network(nid)
