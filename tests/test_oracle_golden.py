"""Pins the CPU oracle against the known answers held by the reference's own tests.

Sources (paths inside the ny project):
  crates/ny-propagate/src/tests/crown/reference.rs:22-158   toy 2-2-1 net (IBP [-6,4], CROWN [-3,3])
  crates/ny-propagate/src/tests/crown/reference.rs:160-380  3-4-4-2 MLP, eps 0.1 (8-digit IBP/CROWN values)
  crates/ny-propagate/src/tests/crown/reference.rs:382-467  tiny 2-2-2 net, CROWN after IBP intersection
  crates/ny-propagate/src/beta_crown/config/tests.rs        verdict predicates (strictness, NaN, inf)
The reference asserts |ny - value| < 1e-4 (1e-5 for the tiny net); the same tolerances are used here.
"""
import math

import numpy as np
import pytest

import json
import os

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "crown_reference.json")) as _f:
    GOLDEN = json.load(_f)
FC1, FC2, FC3 = GOLDEN["deep_3_4_4_2"]["weights"]
B1, B2, B3 = GOLDEN["deep_3_4_4_2"]["biases"]


def test_toy_model(oracle):
    g = GOLDEN["toy_2_2_1"]
    net = oracle.Net(g["weights"])
    lo, hi = g["in_lo"], g["in_hi"]
    pl, pu = oracle.ibp_forward(net, lo, hi)
    assert abs(pl[-1] - g["ibp"][0]) < g["tolerance"] and abs(pu[-1] - g["ibp"][1]) < g["tolerance"]
    cl, cu = oracle.crown(net, lo, hi)
    assert abs(cl[0] - g["crown"][0]) < g["tolerance"] and abs(cu[0] - g["crown"][1]) < g["tolerance"]
    for x in ([-1, -2], [2, 1], [0.5, -0.5]):
        y = net.forward(x)[0]
        assert pl[-1] - 1e-5 <= y <= pu[-1] + 1e-5
        assert cl[0] - 1e-5 <= y <= cu[0] + 1e-5


def test_deep_model(oracle):
    net = oracle.Net([FC1, FC2, FC3], [B1, B2, B3])
    lo, hi = [0.4] * 3, [0.6] * 3
    pl, pu = oracle.ibp_forward(net, lo, hi)
    g = GOLDEN["deep_3_4_4_2"]
    np.testing.assert_allclose(pl[-2:], g["ibp_lo"], atol=g["tolerance"], rtol=0)
    np.testing.assert_allclose(pu[-2:], g["ibp_hi"], atol=g["tolerance"], rtol=0)
    cl, cu = oracle.crown(net, lo, hi)
    np.testing.assert_allclose(cl, g["crown_lo"], atol=g["tolerance"], rtol=0)
    np.testing.assert_allclose(cu, g["crown_hi"], atol=g["tolerance"], rtol=0)
    # the published values carry 8 digits; the restatement agrees far inside the reference's tolerance
    np.testing.assert_allclose(cl, g["crown_lo"], atol=5e-8, rtol=0)
    np.testing.assert_allclose(cu, g["crown_hi"], atol=5e-8, rtol=0)
    assert np.all(cu - cl <= pu[-2:] - pl[-2:] + 1e-5)
    y = net.forward([0.5] * 3)
    assert np.all(y >= cl - 1e-5) and np.all(y <= cu + 1e-5)


def test_tiny_model_intersection(oracle):
    g = GOLDEN["tiny_2_2_2"]
    net = oracle.Net(g["weights"], g["biases"])
    pl, pu = oracle.ibp_forward(net, g["in_lo"], g["in_hi"])
    np.testing.assert_allclose(np.maximum(pl[:2], 0), [0, 0], atol=1e-5)
    np.testing.assert_allclose(pl[2:], [0, 0], atol=1e-5)
    np.testing.assert_allclose(pu[2:], [1.5, 1.0], atol=1e-5)
    cl, cu = oracle.crown(net, g["in_lo"], g["in_hi"])
    np.testing.assert_allclose(cl, g["crown_lo"], atol=g["tolerance"])
    np.testing.assert_allclose(cu, g["crown_hi"], atol=g["tolerance"])


def test_directed_rounding_steps(oracle):
    L = oracle.lib()
    assert L.nyo_next_up_f32(0.0) == np.float32(1e-45)
    assert L.nyo_next_down_f32(0.0) == -np.float32(1e-45)
    assert L.nyo_next_up_f32(1.0) == np.nextafter(np.float32(1), np.float32(2))
    assert L.nyo_next_down_f32(-1.0) == np.nextafter(np.float32(-1), np.float32(-2))
    assert math.isinf(L.nyo_next_up_f32(float("inf"))) and math.isnan(L.nyo_next_up_f32(float("nan")))


def test_certified_reduction_known_answers(oracle):
    # crates/ny-propagate/src/bounds/certified_reduction.rs `mod tests`
    big = np.float32(2.0 ** 30)
    coef = np.array([big, 1.0, -big], np.float32)
    val = np.array([big, 1.0, big], np.float32)
    lo = oracle.lib().nyo_certified_affine_sum(0.0, oracle._fp(coef), oracle._fp(val), 3, 0)
    hi = oracle.lib().nyo_certified_affine_sum(0.0, oracle._fp(coef), oracle._fp(val), 3, 1)
    assert lo <= 1.0 <= hi and lo > 0.99 and hi < 1.01
    coef = np.array([0.0, -0.0, 5.0, 0.0, -np.inf], np.float32)
    val = np.array([3.0, -7.0, 0.0, np.inf, -0.0], np.float32)
    assert oracle.lib().nyo_certified_affine_sum(0.0, oracle._fp(coef), oracle._fp(val), 5, 0) == 0.0
    assert oracle.lib().nyo_certified_affine_sum(-0.0, oracle._fp(coef), oracle._fp(val), 5, 1) == 0.0
    tiny = np.array([np.float32(1e-45)], np.float32)
    one = np.array([1.0], np.float32)
    lo = oracle.lib().nyo_certified_affine_sum(0.0, oracle._fp(tiny), oracle._fp(one), 1, 0)
    hi = oracle.lib().nyo_certified_affine_sum(0.0, oracle._fp(tiny), oracle._fp(one), 1, 1)
    assert 0.0 < lo <= float(tiny[0]) <= hi


def test_verdict_predicates(oracle):
    L = oracle.lib()
    assert L.nyo_domain_verified(0.1, 1.0, 0.0) == 1
    assert L.nyo_domain_verified(0.0, 1.0, 0.0) == 0  # strict
    assert L.nyo_domain_verified(float("nan"), 1.0, 0.0) == 0
    assert L.nyo_domain_verified(0.5, float("inf"), 0.0) == 0
    assert L.nyo_domain_verified(2.0, 1.0, 0.0) == 0  # inverted
    assert L.nyo_domain_violated(-2.0, -1.0, 0.0) == 1
    assert L.nyo_domain_violated(-2.0, 0.0, 0.0) == 0
    assert L.nyo_domain_violated(-1.0, -2.0, 0.0) == 0


# ---- Conv2d known answers (crates/ny-propagate/src/layers/convolution/conv2d/tests.rs) -------------------
def _conv_net(oracle, weight, bias, in_hw, stride=(1, 1), pad=(0, 0)):
    W, b = oracle.conv2d_dense(np.asarray(weight, np.float32), bias, stride, pad, in_hw)
    n_out = W.shape[0]
    # one conv layer followed by an identity read-out, so the conv's own interval is a pre-activation block
    return oracle.Net([W, np.eye(n_out, dtype=np.float32)], [b, None], [0, 0]), W, b


def test_conv2d_ibp_positive_and_negative_kernels(oracle):
    """tests.rs:46-66 (y = 2x + 0.5) and :561-584 (y = -2x + 1: the bounds swap)."""
    lo = np.array([1, 2, 3, 4], np.float32)
    hi = np.array([5, 6, 7, 8], np.float32)
    net, _, _ = _conv_net(oracle, [[[[2.0]]]], np.array([0.5], np.float32), (2, 2))
    pl, pu = oracle.ibp_forward(net, lo, hi)
    assert np.allclose(pl[:4], [2.5, 4.5, 6.5, 8.5], atol=1e-5) and np.allclose(pu[:4], [10.5, 12.5, 14.5, 16.5], atol=1e-5)
    assert np.all(pl[:4] <= [2.5, 4.5, 6.5, 8.5]) and np.all(pu[:4] >= [10.5, 12.5, 14.5, 16.5])
    net, _, _ = _conv_net(oracle, [[[[-2.0]]]], np.array([1.0], np.float32), (2, 2))
    pl, pu = oracle.ibp_forward(net, lo, hi)
    assert np.allclose(pl[:4], [-9, -11, -13, -15], atol=1e-5) and np.allclose(pu[:4], [-1, -3, -5, -7], atol=1e-5)


def test_conv2d_backward_identity_and_2x2_kernel(oracle):
    """tests.rs:287-306: identity coefficients through a 1x1 kernel of 2 give 2*I and bias 0.5;
    tests.rs:620-654: a 2x2 kernel on a 2x2 input gives the kernel weights as coefficients."""
    _, W, b = _conv_net(oracle, [[[[2.0]]]], np.array([0.5], np.float32), (2, 2))
    assert np.array_equal(np.eye(4, dtype=np.float32) @ W, 2 * np.eye(4, dtype=np.float32))
    assert np.array_equal(b, np.full(4, 0.5, np.float32))
    _, W, b = _conv_net(oracle, [[[[1.0, 2.0], [3.0, 4.0]]]], None, (2, 2))
    assert W.shape == (1, 4) and np.array_equal(W[0], [1, 2, 3, 4]) and b is None


def test_conv2d_strided_padded_matches_direct_convolution(oracle):
    """The dense lowering against a direct NCHW convolution loop, stride 2, pad 1, several channels."""
    g = np.random.Generator(np.random.PCG64(5))
    w = g.standard_normal((3, 2, 4, 4)).astype(np.float32)
    bias = g.standard_normal(3).astype(np.float32)
    ih = iw = 6
    W, b = oracle.conv2d_dense(w, bias, (2, 2), (1, 1), (ih, iw))
    oh = ow = (ih + 2 - 4) // 2 + 1
    x = g.standard_normal((2, ih, iw))
    want = np.zeros((3, oh, ow))
    for co in range(3):
        for oy in range(oh):
            for ox in range(ow):
                acc = float(bias[co])
                for ci in range(2):
                    for ky in range(4):
                        for kx in range(4):
                            iy, ix = oy * 2 - 1 + ky, ox * 2 - 1 + kx
                            if 0 <= iy < ih and 0 <= ix < iw:
                                acc += float(w[co, ci, ky, kx]) * x[ci, iy, ix]
                want[co, oy, ox] = acc
    got = W.astype(np.float64) @ x.ravel() + b
    assert np.allclose(got, want.ravel(), atol=1e-12)
    with pytest.raises(ValueError):
        oracle.conv2d_dense(w, None, (0, 1), (0, 0), (6, 6))       # tests.rs:874-897: zero stride rejected
    with pytest.raises(ValueError):
        oracle.conv2d_dense(w, None, (1, 1), (0, 0), (2, 2))       # tests.rs:913-927: output size underflow


# ---- the oracle's native Conv2d (kernel taps, no dense lowering) on the same known answers ----------------
def _native(weight, bias, in_hw, stride=(1, 1), pad=(0, 0)):
    from ny_b200.engine import Conv2d

    return Conv2d(np.asarray(weight, np.float32), None if bias is None else np.asarray(bias, np.float32),
                  stride=stride, pad=pad, in_hw=in_hw)


def test_native_conv2d_known_answers(oracle):
    """The same known answers of conv2d/tests.rs (:46-66, :561-584 interval pass; :287-306, :620-654 backward) through
    the native convolution of the oracle: interval pass values, and the backward coefficients read off plain CROWN
    of a single stable layer (on a box where every output is positive the bound is exactly the affine map)."""
    lo = np.array([1, 2, 3, 4], np.float32)
    hi = np.array([5, 6, 7, 8], np.float32)
    for k, want_lo, want_hi in ((2.0, [2.5, 4.5, 6.5, 8.5], [10.5, 12.5, 14.5, 16.5]),):
        c = _native([[[[k]]]], [0.5], (2, 2))
        net = oracle.Net([c, np.eye(4, dtype=np.float32)], [None, None], [0, 0])
        pl, pu = oracle.ibp_forward(net, lo, hi)
        assert np.allclose(pl[:4], want_lo, atol=1e-5) and np.allclose(pu[:4], want_hi, atol=1e-5)
        assert np.all(pl[:4] <= want_lo) and np.all(pu[:4] >= want_hi)
    c = _native([[[[-2.0]]]], [1.0], (2, 2))
    net = oracle.Net([c, np.eye(4, dtype=np.float32)], [None, None], [0, 0])
    pl, pu = oracle.ibp_forward(net, lo, hi)
    assert np.allclose(pl[:4], [-9, -11, -13, -15], atol=1e-5) and np.allclose(pu[:4], [-1, -3, -5, -7], atol=1e-5)
    # backward: CROWN through [conv 1x1 (2x + 0.5)] then identity read-out equals the interval of 2x + 0.5 exactly
    c = _native([[[[2.0]]]], [0.5], (2, 2))
    net = oracle.Net([c, np.eye(4, dtype=np.float32)], [None, None], [0, 0])
    ol, ou = oracle.crown(net, lo, hi)
    assert np.allclose(ol, [2.5, 4.5, 6.5, 8.5], atol=1e-5) and np.allclose(ou, [10.5, 12.5, 14.5, 16.5], atol=1e-5)
    # 2x2 kernel on a 2x2 input: one output = 1 x00 + 2 x01 + 3 x10 + 4 x11
    c = _native([[[[1.0, 2.0], [3.0, 4.0]]]], None, (2, 2))
    net = oracle.Net([c, np.eye(1, dtype=np.float32)], [None, None], [0, 0])
    ol, ou = oracle.crown(net, lo, hi)
    assert np.allclose(ol, [1 * 1 + 2 * 2 + 3 * 3 + 4 * 4], atol=1e-4) and np.allclose(ou, [1 * 5 + 2 * 6 + 3 * 7 + 4 * 8], atol=1e-4)


def test_native_conv2d_equals_dense_lowering(oracle):
    """Strided, padded, multi-channel CNN: interval pass, plain CROWN and the beta-CROWN bound of split domains through
    the native convolution agree with the dense lowering of the same network (same exact products; the sums differ
    only in the zeros the lowering adds)."""
    from ny_b200.engine import SPLIT_DTYPE

    g = np.random.Generator(np.random.PCG64(8))
    c1 = _native(g.standard_normal((4, 2, 4, 4)) * 0.3, g.standard_normal(4) * 0.1, (8, 8), (2, 2), (1, 1))
    c2 = _native(g.standard_normal((3, 4, 3, 3)) * 0.3, None, (c1.oh, c1.ow), (1, 1), (1, 1))
    fc = (g.standard_normal((6, c2.out_features)) * 0.3).astype(np.float32)
    fb = (g.standard_normal(6) * 0.1).astype(np.float32)
    spec = (np.eye(6, dtype=np.float32)[:1] - np.eye(6, dtype=np.float32)[1:]).astype(np.float32)
    ws, bs = oracle.lower_network([c1, c2, fc], [c1.bias, None, fb])
    dense, native = oracle.Net(ws, bs), oracle.Net([c1, c2, fc], [None, None, fb])
    assert np.array_equal(dense.dims, native.dims)
    x0 = g.uniform(0, 1, c1.in_features).astype(np.float32)
    lo, hi = x0 - np.float32(0.03), x0 + np.float32(0.03)
    dl, du = oracle.ibp_forward(dense, lo, hi)
    nl, nu = oracle.ibp_forward(native, lo, hi)
    assert np.array_equal(dl, nl) and np.array_equal(du, nu)
    a = oracle.crown(dense.with_spec(spec), lo, hi)
    b = oracle.crown(native.with_spec(spec), lo, hi)
    assert np.allclose(a[0], b[0], rtol=1e-6, atol=1e-7) and np.allclose(a[1], b[1], rtol=1e-6, atol=1e-7)
    # a split domain through the batch entry point
    unstable = np.flatnonzero((dl[: c1.out_features] < 0) & (du[: c1.out_features] > 0))
    sp = np.zeros((2, 2), SPLIT_DTYPE)
    sp[0, 0] = (0, int(unstable[0]), 1, 0.3)
    sp[0, 1] = (0, int(unstable[1]), -1, 0.1)
    sp[1, 0] = (0, int(unstable[2]), -1, 0.0)
    ns = np.array([2, 1], np.int32)
    S = spec.shape[0]
    rl = np.concatenate([dl, np.full(S, -np.inf, np.float32)])
    ru = np.concatenate([du, np.full(S, np.inf, np.float32)])
    r1 = oracle.bab_bound_batch(dense.with_spec(spec), lo, hi, rl, ru, sp, ns, 1)
    r2 = oracle.bab_bound_batch(native.with_spec(spec), lo, hi, rl, ru, sp, ns, 1)
    assert np.array_equal(r1[2], r2[2])
    assert np.allclose(r1[0], r2[0], rtol=1e-6, atol=1e-7) and np.allclose(r1[1], r2[1], rtol=1e-6, atol=1e-7)
    # sampled soundness of the native path
    xs = lo + g.random((20000, lo.shape[0])).astype(np.float32) * (hi - lo)
    ys = native.forward(xs) @ spec.astype(np.float64).T
    assert np.all(b[0] <= ys.min(axis=0)) and np.all(b[1] >= ys.max(axis=0))


def test_native_residual_network_equals_its_sequential_lowering(oracle):
    """A small residual CNN (conv stem + two residual blocks + pooled read-out): the oracle's native evaluation
    (kernel taps, identity branches joined in place) against the dense sequential lowering that carries the skipped
    activation as extra neurons.  Same function, same interval bounds on the original neurons, same beta-CROWN bounds
    of split domains."""
    from ny_b200 import workloads as W

    wl = W.config_resnet(seed=61, eps=0.02, n_fix=3, in_chw=(2, 8, 8), channels=4, blocks=2, n_out=5)
    ws, bs = oracle.lower_network(wl.net.weights, wl.net.biases)
    lw, lb, widths = oracle.lower_residual(ws, bs, wl.net.skips)
    low = oracle.Net(lw, lb)
    nat = oracle.Net(wl.net.weights, wl.net.biases, skips=wl.net.skips)
    idx, off = [], 0
    for k, n in enumerate(widths):
        idx.append(off + np.arange(n))
        off += lw[k].shape[0]
    idx = np.concatenate(idx)
    g = np.random.Generator(np.random.PCG64(2))
    x = wl.in_lo + g.random((8, len(wl.in_lo))) * (wl.in_hi - wl.in_lo)
    assert np.abs(nat.forward(x) - low.forward(x)).max() < 1e-10
    ll, lu = oracle.ibp_forward(low, wl.in_lo, wl.in_hi)
    nl, nu = oracle.ibp_forward(nat, wl.in_lo, wl.in_hi)
    tol = 1e-6 * np.maximum(np.abs(nl), np.abs(nu)) + 1e-7
    assert np.all(np.abs(ll[idx] - nl) <= tol) and np.all(np.abs(lu[idx] - nu) <= tol)
    D = 12
    splits, ns = W.draw_domains(wl, nl, nu, D)
    S = wl.spec.shape[0]
    ext = lambda a, v: np.concatenate([a, np.full(S, v, np.float32)])
    n_lo, n_hi, n_inf, _ = oracle.bab_bound_batch(nat.with_spec(wl.spec), wl.in_lo, wl.in_hi, ext(nl, -np.inf), ext(nu, np.inf), splits, ns, 1)
    # the lowered network's neuron indices differ: map the split neurons of layer r through idx
    lsp = splits.copy()
    l_lo, l_hi, l_inf, _ = oracle.bab_bound_batch(low.with_spec(wl.spec), wl.in_lo, wl.in_hi, ext(ll, -np.inf), ext(lu, np.inf), lsp, ns, 1)
    assert np.array_equal(n_inf, l_inf)
    f = n_inf == 0
    scale = np.abs(l_lo[f]).max(axis=1, keepdims=True)
    assert np.all(np.abs(n_lo[f] - l_lo[f]) <= 2e-6 * scale) and np.all(np.abs(n_hi[f] - l_hi[f]) <= 2e-6 * scale)
