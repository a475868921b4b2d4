"""NNet and VNN-LIB readers (CPU only)."""
import numpy as np
import pytest

from ny_b200 import EngineError, formats

# The |x| network of the reference's quick-start (tests/models/crossing_relu.nnet: 1 -> 2 -> 1, weights (1, -1) then
# (1, 1), no biases), written out in the NNet layout.
ABS_NNET = """// NNet format - f(x) = |x|
2,1,1,2,
1,2,1,
0,
0.0,
1.0,
0.0,
1.0,
1.0,
-1.0,
0.0,
0.0,
1.0,1.0,
0.0,
"""


def test_nnet_abs_network():
    n = formats.parse_nnet(ABS_NNET)
    assert n.layer_sizes == [1, 2, 1]
    assert np.array_equal(n.weights[0], [[1.0], [-1.0]]) and np.array_equal(n.weights[1], [[1.0, 1.0]])
    assert np.array_equal(n.biases[0], [0.0, 0.0]) and np.array_equal(n.biases[1], [0.0])
    assert n.output_mean == 0.0 and n.output_range == 1.0      # means / ranges lines without the output entry
    net = n.to_network()
    assert net.dims.tolist() == [1, 2, 1]


def test_nnet_round_trip_and_errors():
    g = np.random.Generator(np.random.PCG64(1))
    ws = [g.standard_normal((7, 5)).astype(np.float32), g.standard_normal((3, 7)).astype(np.float32)]
    bs = [g.standard_normal(7).astype(np.float32), g.standard_normal(3).astype(np.float32)]
    n = formats.parse_nnet(formats.write_nnet(ws, bs))
    assert all(np.array_equal(a, b) for a, b in zip(n.weights, ws)) and all(np.array_equal(a, b) for a, b in zip(n.biases, bs))
    with pytest.raises(EngineError):
        formats.parse_nnet("2,1,1,\n")                                  # short header
    with pytest.raises(EngineError):
        formats.parse_nnet("1,2,1,2,\n2,1,\n0,\n0,0,\n1,1,\n0,0,0,\n1,1,1,\n1.0,\n0.0,\n")   # short weight row
    with pytest.raises(EngineError):
        formats.parse_nnet(ABS_NNET.rsplit("\n", 2)[0])                    # missing last bias


def test_vnnlib_box_and_single_atom():
    text = """; violation: the output reaches 2.0 or above
(declare-const X_0 Real)
(declare-const Y_0 Real)
(assert (>= X_0 -1.0))
(assert (<= X_0 1.0))
(assert (>= Y_0 2.0))
"""
    p = formats.parse_vnnlib(text, 1, 1)
    assert p.in_lo.tolist() == [-1.0] and p.in_hi.tolist() == [1.0]
    assert len(p.violation) == 1 and len(p.violation[0]) == 1
    a = p.violation[0][0]
    assert a.c.tolist() == [1.0] and a.d == -2.0                       # Y_0 - 2 >= 0


def test_vnnlib_and_or_relations():
    text = """(declare-const X_0 Real)(declare-const X_1 Real)(declare-const Y_0 Real)(declare-const Y_1 Real)(declare-const Y_2 Real)
(assert (and (>= X_0 0.1) (<= X_0 0.2)))
(assert (<= 0.3 X_1)) (assert (>= 0.4 X_1))
(assert (or (and (>= Y_0 Y_1) (>= Y_0 Y_2)) (<= Y_1 -1.5)))
"""
    p = formats.parse_vnnlib(text, 2, 3)
    assert np.allclose(p.in_lo, [0.1, 0.3]) and np.allclose(p.in_hi, [0.2, 0.4])
    assert np.all(p.in_lo.astype(np.float64) <= [0.1, 0.3]) and np.all(p.in_hi.astype(np.float64) >= [0.2, 0.4])  # outward
    assert len(p.violation) == 2 and len(p.violation[0]) == 2 and len(p.violation[1]) == 1
    assert p.violation[0][0].c.tolist() == [1, -1, 0] and p.violation[0][1].c.tolist() == [1, 0, -1]
    assert p.violation[1][0].c.tolist() == [0, -1, 0] and p.violation[1][0].d == -1.5      # -Y_1 - 1.5 >= 0


def test_vnnlib_rejections():
    decl = "(declare-const X_0 Real)(declare-const Y_0 Real)"
    with pytest.raises(EngineError):
        formats.parse_vnnlib(decl + "(assert (>= X_0 0.0))(assert (>= Y_0 1.0))", 1, 1)       # no upper bound on X_0
    with pytest.raises(EngineError):
        formats.parse_vnnlib(decl + "(assert (>= X_0 1.0))(assert (<= X_0 0.0))", 1, 1)       # empty box
    with pytest.raises(EngineError) as ei:
        formats.parse_vnnlib(decl + "(assert (>= X_0 0))(assert (<= X_0 1))(assert (>= (+ Y_0 1.0) 2.0))", 1, 1)
    assert ei.value.code == 1                                                                   # declined, not mis-read
    with pytest.raises(EngineError):
        formats.parse_vnnlib(decl + "(assert (>= X_0 0))(assert (<= X_0 1))(assert (>= Y_3 2.0))", 1, 1)
    with pytest.raises(EngineError):
        formats.parse_vnnlib("(assert (>= X_0 0)", 1, 1)


def test_vnnlib_union_of_boxes_and_empty_disjuncts_are_declined():
    """Input atoms below an `or` describe a union of boxes (one box per disjunct in the reference's parser);
    folding them into one box would intersect the disjuncts.  Declined, as is a disjunct or a whole property
    without output atoms (its violation set would be everything, not nothing)."""
    decl = "(declare-const X_0 Real)(declare-const Y_0 Real)"
    union = decl + """(assert (or (and (>= X_0 0.0) (<= X_0 0.5) (>= Y_0 1.0))
                                 (and (>= X_0 0.5) (<= X_0 1.0) (>= Y_0 2.0))))"""
    with pytest.raises(EngineError) as ei:
        formats.parse_vnnlib(union, 1, 1)
    assert ei.value.code == 1
    box = "(assert (>= X_0 0))(assert (<= X_0 1))"
    with pytest.raises(EngineError) as ei:
        formats.parse_vnnlib(decl + box + "(assert (or (and (<= X_0 1)) (>= Y_0 5)))", 1, 1)
    assert ei.value.code == 1
    with pytest.raises(EngineError) as ei:
        formats.parse_vnnlib(decl + box + "(assert (or (and) (>= Y_0 5)))", 1, 1)
    assert ei.value.code == 1
    with pytest.raises(EngineError) as ei:
        formats.parse_vnnlib(decl + box, 1, 1)                     # input box only: nothing to refute
    assert ei.value.code == 1


def test_threshold_of_a_clause_rounds_upwards():
    from ny_b200 import bab

    d = 0.1  # not representable: float32(0.1) > 0.1, float32(0.3) < 0.3 ...
    for d in (0.1, 0.3, -0.7, 1.0, 1e-9):
        prop = formats.Property(np.zeros(1, np.float32), np.ones(1, np.float32),
                                [[formats.Atom(np.array([1.0], np.float32), d)]])
        _, thr, _ = bab._rows(prop)
        assert float(thr[0]) >= d and float(np.nextafter(thr[0], np.float32(-np.inf))) < d


def test_input_split_scores_known_answers():
    """The smart-branching score of the input-split driver, on hand-computed cases."""
    from ny_b200 import bab

    lo, hi = np.array([0, 0, 1], np.float32), np.array([1, 2, 1], np.float32)
    dims, sc = bab.input_split_scores(lo, hi)                       # no coefficients: width, zero-width dims dropped
    assert dims.tolist() == [0, 1] and sc.tolist() == [1.0, 2.0]
    assert bab.select_input_dimension(lo, hi) == 1
    a = np.array([[1.0, 0.1, 5.0], [0.0, 0.0, 9.0]], np.float32)
    assert bab.select_input_dimension(lo, hi, a) == 0                # max(1 * .5, thresh * .5) > max(.1 * 1, thresh * 1)
    dims, sc = bab.input_split_scores(lo, hi, a, lower=np.array([0.5, 2.0]), thr=np.array([0.0, 0.0]))
    assert np.allclose(sc, [2.0005, 2.001])                          # row 1: clamped coefficient * width / 2 + margin 2
    assert bab.select_input_dimension(lo, hi, a, np.array([0.5, 2.0]), np.array([0.0, 0.0])) == 1
    assert bab.select_input_dimension(lo, hi, np.zeros((2, 3), np.float32)) == 1       # all-zero rows: width rule
    assert bab.select_input_dimension(lo, lo) == -1                                     # nothing to split
    nan_a = np.array([[np.nan, 1.0, 0.0]], np.float32)
    assert bab.select_input_dimension(lo, hi, nan_a) == 1                               # a NaN score never wins
    eq = np.array([[2.0, 1.0, 0.0]], np.float32)
    assert bab.select_input_dimension(lo, hi, eq) == 0                                  # tie 1.0 == 1.0: first wins


def test_frontier_dump_round_trip(tmp_path):
    from ny_b200 import bab
    from ny_b200.engine import SPLIT_DTYPE

    prop = formats.Property(np.zeros(2, np.float32), np.ones(2, np.float32),
                            [[formats.Atom(np.array([1, -1], np.float32), 0.5)]])
    fr = [np.zeros(0, SPLIT_DTYPE), np.array([(0, 3, 1, 0.0), (1, 2, -1, 0.25)], SPLIT_DTYPE)]
    path = tmp_path / "frontier.npz"
    bab.save_frontier(path, fr, np.arange(4, dtype=np.float32), np.arange(4, dtype=np.float32) + 1, prop, 3, 17)
    f2, il, ih, rounds, bounded = bab.load_frontier(path, prop)
    assert len(f2) == 2 and len(f2[0]) == 0 and np.array_equal(f2[1], fr[1])
    assert il.tolist() == [0, 1, 2, 3] and ih.tolist() == [1, 2, 3, 4] and (rounds, bounded) == (3, 17)
    other = formats.Property(prop.in_lo, prop.in_hi, [[formats.Atom(np.array([1, -1], np.float32), 0.75)]])
    with pytest.raises(ValueError):
        bab.load_frontier(path, other)
    splits, ns = bab.frontier_to_arrays(fr)
    assert splits.shape == (2, 2) and ns.tolist() == [0, 2]


def test_onnx_round_trip_and_declines():
    from ny_b200 import onnx_reader as R
    from ny_b200 import workloads as W

    g = np.random.Generator(np.random.PCG64(4))
    mlp = W.make_mlp([7, 12, 9, 3], 5)
    n2, shape = R.parse_onnx(R.write_onnx(mlp, (7,)))
    assert shape == (7,) and n2.dims.tolist() == [7, 12, 9, 3]
    assert all(np.array_equal(a, b) for a, b in zip(n2.weights, mlp.weights))
    assert all(np.array_equal(a, b) for a, b in zip(n2.biases, mlp.biases))
    cnn = W.make_cnn(3, in_chw=(2, 8, 8), convs=((4, 3, 1, 1), (6, 4, 2, 1)), fcs=(20, 5))
    data = R.write_onnx(cnn, (2, 8, 8))
    n3, shape = R.parse_onnx(data)
    assert shape == (2, 8, 8) and n3.dims.tolist() == cnn.dims.tolist()
    x = g.standard_normal((4, 128)).astype(np.float32)
    assert np.array_equal(W.forward(cnn, x), W.forward(n3, x))
    c0 = n3.weights[0]
    assert (c0.sh, c0.ph, c0.kh, c0.oc) == (1, 1, 3, 4) and np.array_equal(c0.bias, cnn.weights[0].bias)
    # a model that ends in a Relu gets an identity output layer
    tail = R._enc_node("Relu", ["z2"], ["y"])
    body = R.write_onnx(mlp, (7,))
    graph = [v for num, wt, v in R._fields(memoryview(body)) if num == 7][0]
    ended = R._vi(1, 8) + R._ld(7, bytes(graph) + R._ld(1, tail))
    n4, _ = R.parse_onnx(ended)
    assert n4.dims.tolist() == [7, 12, 9, 3, 3] and np.array_equal(n4.weights[-1], np.eye(3, dtype=np.float32))
    # declines: an operator outside the subset, two affine layers in a row, damaged bytes
    pool = R._vi(1, 8) + R._ld(7, bytes(graph) + R._ld(1, R._enc_node("MaxPool", ["z2"], ["y"])))
    with pytest.raises(EngineError) as ei:
        R.parse_onnx(pool)
    assert ei.value.code == 1
    lin2 = R._ld(1, R._enc_node("Gemm", ["input", "W"], ["a"], [R._enc_attr_int("transB", 1)]))
    lin2 += R._ld(1, R._enc_node("Gemm", ["a", "W"], ["b"], [R._enc_attr_int("transB", 1)]))
    lin2 += R._ld(5, R._enc_tensor("W", np.eye(3, dtype=np.float32))) + R._ld(11, R._enc_value_info("input", [1, 3]))
    with pytest.raises(EngineError) as ei:
        R.parse_onnx(R._ld(7, lin2))
    assert ei.value.code == 1
    with pytest.raises(EngineError):
        R.parse_onnx(body[: len(body) // 2])
    with pytest.raises(EngineError):
        R.parse_onnx(b"")


def test_fsb_candidate_filter_and_margin():
    from ny_b200 import bab

    main = np.array([0.5, -1, 0.2, 0.9, 0.2, -1], np.float32)
    backup = np.array([-0.1, 1, -0.9, 0.0, -0.3, 1], np.float32)
    assert bab.fsb_candidates(main, backup, 2).tolist() == [3, 0, 2, 4]       # two best scores, two most negative intercepts
    assert bab.fsb_candidates(main, backup, 1).tolist() == [3, 2]
    assert bab.fsb_candidates(main, backup, 10).tolist() == [3, 0, 2, 4]      # k beyond the candidate count: all, once
    assert bab.fsb_candidates(np.full(4, -1, np.float32), np.ones(4, np.float32), 3).size == 0
    # clause 0 = atoms 0, 1 (any refutes it), clause 1 = atom 2: margin = min over clauses of the best atom's gap
    m = bab._margin(np.array([[1.0, 0.5, -2.0], [0.5, 3.0, 0.25]], np.float32), np.array([0.0, 1.0, 0.0], np.float32),
                    np.array([0, 0, 1]), 2)
    assert m.tolist() == [-2.0, 0.25]


def test_command_line_errors_exit_with_code_4(tmp_path):
    """Operational errors (missing model, malformed property, unknown format) leave with the reference's code 4 before any
    device is touched."""
    from ny_b200.__main__ import main

    model = tmp_path / "abs.nnet"
    model.write_text(ABS_NNET)
    bad_prop = tmp_path / "bad.vnnlib"
    bad_prop.write_text("(declare-const X_0 Real)(declare-const Y_0 Real)(assert (>= X_0 0.0))(assert (>= Y_0 1.0))")
    assert main(["beta-crown", str(tmp_path / "missing.nnet"), "-p", str(bad_prop)]) == 4
    assert main(["beta-crown", str(model), "-p", str(bad_prop)]) == 4            # no upper bound on X_0
    assert main(["verify", str(tmp_path / "model.pt"), "-p", str(bad_prop)]) == 4
    assert main(["beta-crown", str(model)]) == 4                                  # -p is required


def test_make_children_appends_the_split_and_keeps_histories():
    from ny_b200 import bab
    from ny_b200.engine import SPLIT_DTYPE

    sp = np.zeros((3, 2), SPLIT_DTYPE)
    ns = np.array([0, 1, 2], np.int32)
    sp[1, 0] = (1, 5, -1, 0.5)
    sp[1, 1] = (9, 9, 9, 9.0)                       # junk past the end of history 1 must not travel
    sp[2, 0], sp[2, 1] = (0, 3, 1, 0.25), (1, 7, -1, 0.75)
    beta = np.array([[0, 0], [0.125, 0], [1.5, 2.5]], np.float32)
    ch, cn = bab.make_children(sp, ns, np.array([0, 1, 2]), np.array([2, 0, 1]), np.array([4, 6, 8]), beta=beta)
    assert cn.tolist() == [1, 1, 2, 2, 3, 3] and ch.shape == (6, 3)
    assert ch[0, 0].tolist() == (2, 4, 1, 0.0) and ch[1, 0].tolist() == (2, 4, -1, 0.0)
    assert ch[2, 0].tolist() == (1, 5, -1, 0.125) and ch[2, 1].tolist() == (0, 6, 1, 0.0) and ch[2, 2].tolist() == (0, 0, 0, 0.0)
    assert ch[5, 0].tolist() == (0, 3, 1, 1.5) and ch[5, 1].tolist() == (1, 7, -1, 2.5) and ch[5, 2].tolist() == (1, 8, -1, 0.0)
    ch2, _ = bab.make_children(sp, ns, np.array([2]), np.array([2, 0, 1]), np.array([4, 6, 8]))     # multipliers kept
    assert ch2[0, 0].tolist() == (0, 3, 1, 0.25) and ch2[1, 1].tolist() == (1, 7, -1, 0.75)


def test_onnx_input_normalisation_and_constant_transpose_are_folded():
    from ny_b200 import onnx_reader as R
    from ny_b200 import workloads as W

    g = np.random.Generator(np.random.PCG64(8))
    w1 = g.standard_normal((5, 4)).astype(np.float32)
    b1 = g.standard_normal(5).astype(np.float32)
    w2 = g.standard_normal((3, 5)).astype(np.float32)
    mean = g.standard_normal(4).astype(np.float32)
    std = (0.5 + g.random(4)).astype(np.float32)
    nodes = [R._enc_node("Sub", ["input", "mean"], ["c"]), R._enc_node("Div", ["c", "std"], ["n"]),
             R._enc_node("Gemm", ["n", "W1", "B1"], ["z1"], [R._enc_attr_int("transB", 1)]), R._enc_node("Relu", ["z1"], ["a1"]),
             R._enc_node("Transpose", ["W2t"], ["W2"]), R._enc_node("MatMul", ["a1", "W2"], ["y"])]
    graph = b"".join(R._ld(1, n) for n in nodes)
    for name, arr in (("mean", mean), ("std", std), ("W1", w1), ("B1", b1), ("W2t", w2)):     # W2t is [out, in]: MatMul needs its transpose
        graph += R._ld(5, R._enc_tensor(name, arr))
    graph += R._ld(11, R._enc_value_info("input", [1, 4]))
    net, shape = R.parse_onnx(R._ld(7, graph))
    assert shape == (4,) and net.dims.tolist() == [4, 5, 3]
    x = g.standard_normal((6, 4)).astype(np.float32)
    want = np.maximum(((x.astype(np.float64) - mean) / std) @ w1.astype(np.float64).T + b1, 0) @ w2.astype(np.float64).T
    assert np.allclose(W.forward(net, x), want, rtol=1e-5, atol=1e-6)
    # a normalisation in front of a convolution is declined, not mis-folded
    conv = [R._enc_node("Sub", ["input", "m"], ["c"]), R._enc_node("Conv", ["c", "K"], ["y"])]
    gr = b"".join(R._ld(1, n) for n in conv) + R._ld(5, R._enc_tensor("m", np.zeros(1, np.float32)))
    gr += R._ld(5, R._enc_tensor("K", np.ones((1, 1, 1, 1), np.float32))) + R._ld(11, R._enc_value_info("input", [1, 1, 2, 2]))
    with pytest.raises(EngineError) as ei:
        R.parse_onnx(R._ld(7, gr))
    assert ei.value.code == 1


def test_onnx_residual_add_becomes_an_identity_skip():
    from ny_b200 import onnx_reader as R
    from ny_b200 import workloads as W

    g = np.random.Generator(np.random.PCG64(9))
    ws = [g.standard_normal(s).astype(np.float32) * 0.5 for s in ((6, 4), (6, 6), (6, 6), (3, 6))]
    bs = [g.standard_normal(w.shape[0]).astype(np.float32) for w in ws]
    # x -> L0 -> relu (a0) -> L1 -> relu -> L2 -> + a0 -> relu -> L3
    nodes = [R._enc_node("Gemm", ["input", "W0", "B0"], ["z0"], [R._enc_attr_int("transB", 1)]), R._enc_node("Relu", ["z0"], ["a0"]),
             R._enc_node("Gemm", ["a0", "W1", "B1"], ["z1"], [R._enc_attr_int("transB", 1)]), R._enc_node("Relu", ["z1"], ["a1"]),
             R._enc_node("Gemm", ["a1", "W2", "B2"], ["z2"], [R._enc_attr_int("transB", 1)]), R._enc_node("Add", ["z2", "a0"], ["s2"]),
             R._enc_node("Relu", ["s2"], ["a2"]), R._enc_node("Gemm", ["a2", "W3", "B3"], ["y"], [R._enc_attr_int("transB", 1)])]
    graph = b"".join(R._ld(1, n) for n in nodes)
    for k, (w, b) in enumerate(zip(ws, bs)):
        graph += R._ld(5, R._enc_tensor(f"W{k}", w)) + R._ld(5, R._enc_tensor(f"B{k}", b))
    graph += R._ld(11, R._enc_value_info("input", [1, 4]))
    net, _ = R.parse_onnx(R._ld(7, graph))
    assert net.skips == {2: 0} and net.dims.tolist() == [4, 6, 6, 6, 3]
    x = g.standard_normal((5, 4))
    a0 = np.maximum(x @ ws[0].astype(np.float64).T + bs[0], 0)
    a1 = np.maximum(a0 @ ws[1].astype(np.float64).T + bs[1], 0)
    a2 = np.maximum(a1 @ ws[2].astype(np.float64).T + bs[2] + a0, 0)
    want = a2 @ ws[3].astype(np.float64).T + bs[3]
    assert np.allclose(W.forward(net, x.astype(np.float32)), want, rtol=1e-5, atol=1e-5)
    # a skip around a single layer is outside what the engine's blocks express: declined
    bad = [R._enc_node("Gemm", ["input", "W0", "B0"], ["z0"], [R._enc_attr_int("transB", 1)]), R._enc_node("Relu", ["z0"], ["a0"]),
           R._enc_node("Gemm", ["a0", "W1", "B1"], ["z1"], [R._enc_attr_int("transB", 1)]), R._enc_node("Add", ["z1", "a0"], ["s1"]),
           R._enc_node("Relu", ["s1"], ["a1"]), R._enc_node("Gemm", ["a1", "W3", "B3"], ["y"], [R._enc_attr_int("transB", 1)])]
    gb = b"".join(R._ld(1, n) for n in bad)
    for k in (0, 1, 3):
        gb += R._ld(5, R._enc_tensor(f"W{k}", ws[k])) + R._ld(5, R._enc_tensor(f"B{k}", bs[k]))
    gb += R._ld(11, R._enc_value_info("input", [1, 4]))
    with pytest.raises(EngineError) as ei:
        R.parse_onnx(R._ld(7, gb))
    assert ei.value.code == 1


# ---- the reference's own ONNX fixtures (tests/golden/onnx: copies of its tests/models/*.onnx, data only) ----------
def _onnx_fixture(name):
    import os

    with open(os.path.join(os.path.dirname(__file__), "golden", "onnx", name), "rb") as f:
        return f.read()


def test_reader_on_the_reference_single_linear_known_answers(oracle):
    """crates/ny-onnx/src/tests/core/propagate.rs:12-66: single_linear.onnx is W = [[1,2],[3,-1],[-2,1]],
    b = [0.5,-0.5,1]; the point [1,1] maps to [3.5,1.5,0] and the box [0,1]^2 to [0.5,-1.5,-1] .. [3.5,2.5,2]."""
    from ny_b200 import onnx_reader as R

    net, shape = R.parse_onnx(_onnx_fixture("single_linear.onnx"))
    assert shape == (2,) and len(net.weights) == 1
    assert np.array_equal(net.weights[0], np.array([[1, 2], [3, -1], [-2, 1]], np.float32))
    assert np.array_equal(net.biases[0], np.array([0.5, -0.5, 1.0], np.float32))
    onet = oracle.Net(net.weights, net.biases)
    lo, hi = oracle.ibp_forward(onet, np.ones(2, np.float32), np.ones(2, np.float32))
    assert np.allclose(lo[:3], [3.5, 1.5, 0.0], atol=1e-5) and np.allclose(hi[:3], [3.5, 1.5, 0.0], atol=1e-5)
    lo, hi = oracle.ibp_forward(onet, np.zeros(2, np.float32), np.ones(2, np.float32))
    assert np.allclose(lo[:3], [0.5, -1.5, -1.0], atol=1e-5) and np.allclose(hi[:3], [3.5, 2.5, 2.0], atol=1e-5)


def test_reader_on_the_reference_sequential_fixtures(oracle):
    """The shapes the reference's differential-translation tests state for its fixtures
    (crates/ny-onnx/src/tests/core/differential_translation.rs:216-243: simple_mlp is Linear(2->4) + ReLU +
    Linear(4->2); conv_relu is Conv2d(1->2, 2x2) + ReLU on a 3-D input; mnist_conv is Conv -> ReLU -> Flatten -> Linear)
    and the soundness check of tests/core/graph.rs:13-66 on linear_relu: interval bounds of [0,1]^2 contain the
    network's value at the four corners and the centre."""
    from ny_b200 import onnx_reader as R
    from ny_b200 import workloads as W

    mlp, shape = R.parse_onnx(_onnx_fixture("simple_mlp.onnx"))
    assert shape == (2,) and [w.shape for w in mlp.weights] == [(4, 2), (2, 4)]
    conv, shape = R.parse_onnx(_onnx_fixture("conv_relu.onnx"))
    assert shape == (1, 4, 4) and (conv.weights[0].oc, conv.weights[0].ic, conv.weights[0].kh, conv.weights[0].kw) == (2, 1, 2, 2)
    assert int(conv.dims[1]) == 2 * 3 * 3                        # stride 1, no padding: 3x3 outputs per channel
    mn, shape = R.parse_onnx(_onnx_fixture("mnist_conv.onnx"))
    assert shape == (1, 8, 8) and hasattr(mn.weights[0], "kh") and mn.weights[1].shape == (5, 72)
    one, shape = R.parse_onnx(_onnx_fixture("single_conv2d.onnx"))
    assert shape == (1, 5, 5) and len(one.weights) == 1
    lr, shape = R.parse_onnx(_onnx_fixture("linear_relu.onnx"))
    onet = oracle.Net(lr.weights, lr.biases)
    lo, hi = oracle.ibp_forward(onet, np.zeros(2, np.float32), np.ones(2, np.float32))
    n_out = int(lr.dims[-1])
    for pt in ([0, 0], [1, 0], [0, 1], [1, 1], [0.5, 0.5]):
        y = W.forward(lr, np.array([pt], np.float32))[0]
        assert np.all(y >= lo[-n_out:] - 1e-5) and np.all(y <= hi[-n_out:] + 1e-5)
    # every fixture: the network evaluates, and the interval pass of its own box encloses a sample
    g = np.random.Generator(np.random.PCG64(3))
    for net, shp in ((mlp, (2,)), (conv, (1, 4, 4)), (mn, (1, 8, 8)), (one, (1, 5, 5))):
        n0 = int(np.prod(shp))
        x = g.random((4, n0), dtype=np.float32)
        on = oracle.Net(net.weights, net.biases)
        lo, hi = oracle.ibp_forward(on, np.zeros(n0, np.float32), np.ones(n0, np.float32))
        y = W.forward(net, x)
        k = y.shape[1]
        assert np.all(y >= lo[-k:] - 1e-5) and np.all(y <= hi[-k:] + 1e-5)


def test_reader_declines_the_reference_maxpool_fixture():
    """cnn_with_flatten.onnx contains a MaxPool, which the bound kernels do not cover: UnsupportedOp, not a guess."""
    from ny_b200 import onnx_reader as R
    from ny_b200.engine import EngineError

    with pytest.raises(EngineError) as ei:
        R.parse_onnx(_onnx_fixture("cnn_with_flatten.onnx"))
    assert "MaxPool" in str(ei.value)
