"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, the host
mirror validates shapes the way the reference's engine boundary does, workloads are reproducible."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib_path():
    from ny_b200 import build

    return build.build()


def test_library_exports_every_declared_symbol(lib_path):
    header = open(os.path.join(ROOT, "include", "nyb200.h")).read()
    declared = sorted(set(re.findall(r"\b(nyb200_\w+)\s*\(", header)))
    assert len(declared) >= 20
    L = ctypes.CDLL(lib_path)
    missing = [n for n in declared if not hasattr(L, n)]
    assert missing == []
    from ny_b200 import engine

    assert sorted(engine.EXPORTS) == declared


def test_provenance_string_needs_no_gpu(lib_path):
    L = ctypes.CDLL(lib_path)
    L.nyb200_backend_provenance.restype = ctypes.c_char_p
    assert b"sm_100a" in L.nyb200_backend_provenance()


def test_create_fails_loudly_without_a_device(lib_path):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from ny_b200 import B200Engine, EngineError

    with pytest.raises(EngineError) as ei:
        B200Engine(0)
    assert ei.value.code == 1  # UnsupportedOp: declined, and there is no CPU path to fall back to


def test_network_shape_validation():
    from ny_b200 import EngineError, Network

    Network([np.zeros((3, 2)), np.zeros((1, 3))])
    with pytest.raises(EngineError):
        Network([np.zeros((3, 2)), np.zeros((1, 4))])


def test_workloads_are_reproducible_and_well_formed():
    from ny_b200 import workloads as W

    a, b = W.config_mlp_bab(seed=2, hidden=32, depth=3), W.config_mlp_bab(seed=2, hidden=32, depth=3)
    assert all(np.array_equal(x, y) for x, y in zip(a.net.weights, b.net.weights))
    assert a.spec.shape == (9, 10) and np.all(a.in_lo >= 0) and np.all(a.in_hi <= 1)
    assert np.all(a.spec.sum(axis=1) == 0)
    rl = -np.ones(a.net.n_pre, np.float32)
    rh = np.ones(a.net.n_pre, np.float32)
    s1, n1 = W.draw_domains(a, rl, rh, 16)
    s2, n2 = W.draw_domains(a, rl, rh, 8, first=8)
    assert np.array_equal(s1[8:], s2) and np.all(n1 == 8)
    for d in range(16):  # drawn without replacement
        keys = set(zip(s1["relu"][d].tolist(), s1["neuron"][d].tolist()))
        assert len(keys) == 8
    assert set(np.unique(s1["sign"])) <= {-1, 1}


def test_projection_block_lowering_is_exact():
    """lower_projection_block (GpuResnetSegment::ResidualProj, crates/ny-core/src/gemm.rs:1658-1669): the widened
    sequential layers compute F(z) + P(z) for z >= 0 up to binary64 summation order, for Linear and Conv2d blocks, with
    P's bias carried on a constant neuron when both branches have one; blocks outside the supported form are declined."""
    from ny_b200 import Conv2d, EngineError, lower_projection_block

    g = np.random.Generator(np.random.PCG64(5))
    f32 = lambda *s: g.standard_normal(s).astype(np.float32)
    relu = lambda x: np.maximum(x, 0)
    nz, h, no = 6, 9, 7
    W1, b1, W2, W3, b3, Wp, bp = f32(h, nz), f32(h), f32(h, h), f32(no, h), f32(no), f32(no, nz), f32(no)
    low = lower_projection_block([(W1, b1), (W2, None), (W3, b3)], (Wp, bp))
    z = np.abs(g.standard_normal((5, nz)))
    ref = relu(relu(z @ W1.astype(np.float64).T + b1) @ W2.astype(np.float64).T) @ W3.astype(np.float64).T + b3 \
        + z @ Wp.astype(np.float64).T + bp
    x = z
    for k, (w, b) in enumerate(low):
        x = x @ w.astype(np.float64).T + (0 if b is None else b.astype(np.float64))
        if k < len(low) - 1:
            x = relu(x)
    assert np.abs(x - ref).max() < 1e-12
    assert low[0][0].shape == (h + nz + 1, nz) and low[-1][0].shape == (no, h + nz + 1)   # z and the constant ride along
    assert np.array_equal(low[-1][1], b3)                                              # no fp32 sum of two biases
    cz, c1, co = 3, 4, 5
    F1 = Conv2d(f32(c1, cz, 3, 3), f32(c1), (2, 2), (1, 1), (8, 8))
    F2 = Conv2d(f32(co, c1, 3, 3), f32(co), (1, 1), (1, 1), (4, 4))
    P = Conv2d(f32(co, cz, 1, 1), f32(co), (2, 2), (0, 0), (8, 8))
    lowc = lower_projection_block([(F1, None), (F2, None)], (P, None))
    z = np.abs(g.standard_normal((4, cz * 64)))
    ref = F2.apply(relu(F1.apply(z))) + P.apply(z)
    assert np.abs(lowc[1][0].apply(relu(lowc[0][0].apply(z))) - ref).max() < 1e-12
    with pytest.raises(EngineError):
        lower_projection_block([(W1, b1)], (Wp, bp))                                   # a one-layer F
    with pytest.raises(EngineError):
        lower_projection_block([(F1, None), (F2, None)], (Conv2d(f32(co, cz, 3, 3), None, (2, 2), (1, 1), (8, 8)), None))
    with pytest.raises(EngineError):
        lower_projection_block([(F1, None), (W3, None)], (P, None))                    # mixed layer kinds


def test_kfsb_reduce_operators_and_fallback():
    """select_fsb's combination of the two children's margins (KfsbReduceOp: min / max / mean,
    beta_crown/engine/branching/sequential.rs:482-507), its tie rule, NaN handling and the depth-keyed fallback
    (:535-552), against a stand-in engine that returns canned scores and child bounds."""
    from ny_b200 import SPLIT_DTYPE, bab, formats

    class FakeEngine:
        def __init__(self, lower):
            self.lower = lower

        def batch_branch_scores(self, with_backup=True):
            main = np.full((1, 6), -1.0, np.float32)
            main[0, [1, 3, 4]] = [0.5, 0.9, 0.7]          # three candidates, BaBSR order 3, 4, 1
            return main, np.zeros((1, 6), np.float32)

        def bab_bound_batch(self, net_id, spec, lo, hi, inh_lo, inh_hi, splits, ns, mode=1):
            assert len(ns) == 6 and np.all(ns == 1)
            self.asked = [(int(s[0]["neuron"]), int(s[0]["sign"])) for s in splits]
            return self.lower.reshape(6, 1), None, np.zeros(6, np.int32)

    class Net:
        dims = np.array([2, 6, 1])

    prop = formats.Property(np.zeros(2, np.float32), np.ones(2, np.float32), [[formats.Atom(np.array([-1.0], np.float32), 0.0)]])
    take = [np.zeros(0, SPLIT_DTYPE)]
    # children (active, inactive) of candidates 3, 4, 1 in that order
    lower = np.array([-1.0, -5.0, -2.0, -3.0, -4.0, -0.5], np.float32)
    picks = {}
    for op in ("min", "max", "mean"):
        eng = FakeEngine(lower)
        picks[op] = bab.select_fsb(eng, 0, Net, prop, None, None, take, [0], k=3, reduce=op)[0]
        assert eng.asked == [(3, 1), (3, -1), (4, 1), (4, -1), (1, 1), (1, -1)]
    assert picks == {"min": (0, 4), "max": (0, 1), "mean": (0, 1)}     # min: -5, -3, -4; max: -1, -2, -0.5; mean: -3, -2.5, -2.25
    # ties within 1e-6 go to the larger BaBSR score; NaN never wins
    eng = FakeEngine(np.array([-2.0, -2.0, -2.0, -2.0, np.nan, -1.0], np.float32))
    assert bab.select_fsb(eng, 0, Net, prop, None, None, take, [0], k=3)[0] == (0, 3)
    # every trial NaN: the depth-keyed fallback picks one of the candidates, the same one every time
    eng = FakeEngine(np.full(6, np.nan, np.float32))
    a = bab.select_fsb(eng, 0, Net, prop, None, None, take, [0], k=3)[0]
    b = bab.select_fsb(eng, 0, Net, prop, None, None, take, [0], k=3)[0]
    assert a == b and a in [(0, 3), (0, 4), (0, 1)]
    assert a == [(0, 3), (0, 4), (0, 1)][bab.kfsb_fallback_index(0, 3)]
    with pytest.raises(ValueError):
        bab.select_fsb(eng, 0, Net, prop, None, None, take, [0], k=3, reduce="median")
