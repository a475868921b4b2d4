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
