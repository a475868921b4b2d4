"""The allocation-free interval forward pass (nyb200_ibp_forward_noalloc) against the regular entry
point, through the C ABI, twice in a row: the second call reuses the library's fixed scratch with the
first call's leftovers in it and must still agree.  Collected last on purpose."""
import numpy as np
import pytest

from ny_b200 import workloads as W

pytestmark = pytest.mark.gpu


def test_noalloc_forward_matches_regular_entry_point_twice():
    import torch

    from ny_b200 import B200Engine, EngineError, Network

    eng = B200Engine(0, torch.cuda.current_stream().cuda_stream)
    wl_a = W.config_mlp_bab(seed=31, hidden=96, depth=4, n_in=200)   # first call: wide hidden layers
    wl_b = W.config_mlp_small(seed=5)                               # second call: narrower net, other box
    for wl in (wl_a, wl_b):
        nid = eng.register_network(wl.net)
        ref_lo, ref_hi = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)      # existing entry point (host buffers)
        lo = torch.from_numpy(wl.in_lo).cuda()
        hi = torch.from_numpy(wl.in_hi).cuda()
        out_lo = torch.full((wl.net.n_pre,), float("nan"), device="cuda")
        out_hi = torch.full((wl.net.n_pre,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        eng.ibp_forward_noalloc(nid, lo.data_ptr(), hi.data_ptr(), out_lo.data_ptr(), out_hi.data_ptr())
        got_lo, got_hi = out_lo.cpu().numpy(), out_hi.cpu().numpy()
        # same arithmetic, same reduction order: the two entry points agree bit for bit (the parity tests'
        # 1e-5 relative tolerance for interval bounds is therefore met with room to spare)
        assert np.array_equal(got_lo, ref_lo[0]) and np.array_equal(got_hi, ref_hi[0])
        assert np.all(got_lo <= got_hi)
        eng.release_network(nid)
    # widths beyond the fixed scratch are refused with a clear error, not truncated
    big = Network([np.zeros((4, 8200), np.float32), np.zeros((2, 4), np.float32)])
    nid = eng.register_network(big)
    x = torch.zeros(8200, device="cuda")
    o = torch.zeros(6, device="cuda")
    with pytest.raises(EngineError) as ei:
        eng.ibp_forward_noalloc(nid, x.data_ptr(), x.data_ptr(), o.data_ptr(), o.data_ptr())
    assert ei.value.code == 1 and "8192" in str(ei.value)
    eng.close()


def test_noalloc_refuses_conv_and_skip_networks_before_any_launch():
    """The allocation-free pass is a dense mat-vec per layer: a Conv2d layer (whose weights are a filter bank, not
    a dense matrix) and a residual connection are refused with UnsupportedOp.  The refusal happens on the host,
    so the launch counter does not move."""
    import torch

    from ny_b200 import B200Engine, EngineError, Network
    from ny_b200.engine import Conv2d

    eng = B200Engine(0, torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(3)
    conv = Conv2d(rng.standard_normal((4, 2, 3, 3)).astype(np.float32), None, stride=(1, 1), pad=(1, 1), in_hw=(6, 6))
    cnn = Network([conv, rng.standard_normal((3, conv.out_features)).astype(np.float32)])
    w = [rng.standard_normal((8, 5)).astype(np.float32), rng.standard_normal((8, 8)).astype(np.float32),
         rng.standard_normal((8, 8)).astype(np.float32), rng.standard_normal((2, 8)).astype(np.float32)]
    skipnet = Network(w, skips={2: 0})
    for net, word in ((cnn, "Conv2d"), (skipnet, "residual")):
        nid = eng.register_network(net)
        x = torch.zeros(int(net.dims[0]), device="cuda")
        o = torch.zeros(net.n_pre, device="cuda")
        before = eng.launch_count()
        with pytest.raises(EngineError) as ei:
            eng.ibp_forward_noalloc(nid, x.data_ptr(), x.data_ptr(), o.data_ptr(), o.data_ptr())
        assert ei.value.code == 1 and word in str(ei.value)
        assert eng.launch_count() == before
        eng.release_network(nid)
    eng.close()
