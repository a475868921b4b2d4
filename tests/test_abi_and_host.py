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
