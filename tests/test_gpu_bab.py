"""The branch-and-bound driver over the device batch calls, end to end from model and property text."""
import numpy as np
import pytest

from ny_b200 import bab, formats
from ny_b200 import workloads as W
from test_formats import ABS_NNET

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from ny_b200 import B200Engine

    e = B200Engine(0)
    yield e
    e.close()


def _prop(y_op, value):
    return (f"(declare-const X_0 Real)(declare-const Y_0 Real)(assert (>= X_0 -1.0))(assert (<= X_0 1.0))"
            f"(assert ({y_op} Y_0 {value}))")


def test_abs_network_quick_start_verdicts(eng):
    """The reference's quick start (README.md:82-115): f(x) = |x| on [-1, 1].  "Y_0 >= 2.0" cannot be reached:
    VERIFIED; "Y_0 >= 0.5" can: VIOLATED, with a counterexample that the concrete network confirms."""
    net = formats.parse_nnet(ABS_NNET).to_network()
    nid = eng.register_network(net)
    safe = formats.parse_vnnlib(_prop(">=", 2.0), 1, 1)
    r = bab.verify(eng, nid, net, safe)
    assert r.status == "verified" and r.counterexample is None
    unsafe = formats.parse_vnnlib(_prop(">=", 0.5), 1, 1)
    r = bab.verify(eng, nid, net, unsafe)
    assert r.status == "violated"
    x = float(r.counterexample[0])
    assert -1.0 <= x <= 1.0 and abs(x) >= 0.5 and abs(float(r.output[0]) - abs(x)) < 1e-6
    # |x| <= 1 exactly: "Y_0 >= 1.0" is reached at the corners, "Y_0 >= 1.0001" is not
    assert bab.verify(eng, nid, net, formats.parse_vnnlib(_prop(">=", 1.0), 1, 1)).status == "violated"
    r = bab.verify(eng, nid, net, formats.parse_vnnlib(_prop(">=", 1.0001), 1, 1))
    assert r.status == "verified"                            # the two chords of the root relaxation sum to exactly 1
    eng.release_network(nid)


def test_bab_closes_the_gap_between_root_bound_and_true_minimum(eng, tmp_path):
    wl = W.config_mlp_bab(seed=81, hidden=12, depth=2, n_in=4, n_out=3, eps=0.4, n_fix=0)
    net = wl.net
    nid = eng.register_network(net)
    # true minimum of the margins, from dense sampling and the attack
    mn = W.sample_min_margin(wl, 400000, 3)
    g = np.random.Generator(np.random.PCG64(5))
    x0 = (wl.in_lo + g.random((512, 4), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)
    for s in range(wl.spec.shape[0]):
        best, _, _ = eng.pgd_attack(nid, wl.spec[s:s + 1], wl.in_lo, wl.in_hi, x0, 60, 0.1)
        mn[s] = min(mn[s], best.min())
    root_lo, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    s = int(np.argmax(mn - root_lo[0]))                 # the row with the widest gap
    assert mn[s] - root_lo[0][s] > 1e-3
    row = wl.spec[s]

    def prop(t):   # violation: margin_s <= t, i.e. -row . y + t >= 0
        return formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-row, float(t))]])

    t_safe = float(root_lo[0][s] + 0.6 * (mn[s] - root_lo[0][s]))   # above the root bound, below the true minimum
    # beta = 0 bounds ignore the split constraints' effect on the input region: sound but incomplete, so the plain
    # driver may stop at "unknown"; it must never claim a violation.  With the split multipliers optimised the
    # search closes.
    r = bab.verify(eng, nid, net, prop(t_safe), batch=256, max_rounds=200)
    assert r.status in ("verified", "unknown") and r.rounds >= 1 and r.domains_bounded > 1
    r2 = bab.verify(eng, nid, net, prop(t_safe), batch=256, max_rounds=200, optimize_iterations=20)
    assert r2.status == "verified" and r2.rounds >= 1 and r2.open_domains == 0
    assert r2.domains_bounded < r.domains_bounded            # optimised bounds prune earlier
    # children that inherit their parent's optimised slopes and multipliers need no more domains than cold starts
    r3 = bab.verify(eng, nid, net, prop(t_safe), batch=256, max_rounds=200, optimize_iterations=20, warm_start=False)
    assert r3.status == "verified" and r2.domains_bounded <= r3.domains_bounded
    # BaBSR and filtered smart branching drive the same search to the same verdict
    for kind in (2, 3):
        rk = bab.verify(eng, nid, net, prop(t_safe), batch=256, max_rounds=200, optimize_iterations=20, branching=kind)
        assert rk.status == "verified" and rk.open_domains == 0
    # stop after two rounds, dump the frontier, resume from the dump: same verdict, and the two legs together bound
    # exactly the domains of the uninterrupted run; one metrics record per round
    import json

    ck, mj = tmp_path / "frontier.npz", tmp_path / "rounds.jsonl"
    ra = bab.verify(eng, nid, net, prop(t_safe), batch=256, max_rounds=2, optimize_iterations=20, checkpoint=ck,
                    metrics_jsonl=mj)
    assert ra.status == "unknown" and ra.open_domains > 0 and ck.exists()
    rb = bab.verify(eng, nid, net, prop(t_safe), batch=256, max_rounds=200, optimize_iterations=20, resume=ck,
                    metrics_jsonl=mj)
    assert rb.status == "verified" and rb.domains_bounded == r2.domains_bounded and ra.rounds + rb.rounds == r2.rounds
    recs = [json.loads(line) for line in open(mj)]
    assert len(recs) == r2.rounds and recs[-1]["open"] == 0 and recs[-1]["explored"] == r2.domains_bounded
    assert all(rec["verified"] + rec["infeasible"] <= rec["batch"] for rec in recs)
    t_unsafe = float(mn[s] + 1e-3 * max(1.0, abs(mn[s])))
    r = bab.verify(eng, nid, net, prop(t_unsafe))
    assert r.status == "violated"
    y = W.forward(net, r.counterexample)
    assert float(row @ y) <= t_unsafe and np.all(r.counterexample >= wl.in_lo) and np.all(r.counterexample <= wl.in_hi)
    eng.release_network(nid)


def test_crown_input_coefficients(eng):
    """Linear network: the exported rows are spec . W exactly on both sides; they go stale with the next batch call."""
    from ny_b200 import EngineError, Network

    g = np.random.Generator(np.random.PCG64(12))
    w = g.standard_normal((4, 6)).astype(np.float32)
    b = g.standard_normal(4).astype(np.float32)
    net = Network([w], [b])
    nid = eng.register_network(net)
    spec = g.standard_normal((3, 4)).astype(np.float32)
    lo = g.standard_normal((5, 6)).astype(np.float32)
    hi = lo + 0.1
    lower, upper, _, _ = eng.crown_bounds(nid, spec, lo, hi)
    la, ua = eng.crown_input_coeffs(5, 3, 6)
    want = spec.astype(np.float64) @ w.astype(np.float64)
    assert np.allclose(la, want[None], rtol=1e-5, atol=1e-6) and np.allclose(ua, want[None], rtol=1e-5, atol=1e-6)
    conc = np.where(want > 0, lo[:, None, :], hi[:, None, :])
    assert np.allclose(lower, (want[None] * conc).sum(-1) + spec @ b, rtol=1e-4, atol=1e-4)
    eng.pgd_attack(nid, spec, lo[0], hi[0], lo[:1], 1, 0.01)
    with pytest.raises(EngineError):
        eng.crown_input_coeffs(5, 3, 6)
    eng.release_network(nid)


def test_input_split_on_an_acas_shaped_network(eng):
    wl = W.config_mlp_small(seed=7)                     # 5 -> 6 x 50 -> 5
    net = wl.net
    nid = eng.register_network(net)
    lo = (wl.x0 - np.float32(0.25)).astype(np.float32)
    hi = (wl.x0 + np.float32(0.25)).astype(np.float32)
    g = np.random.Generator(np.random.PCG64(2))
    xs = (lo + g.random((300000, 5), dtype=np.float32) * (hi - lo)).astype(np.float32)
    ys = W.forward(net, xs) @ wl.spec.astype(np.float64).T
    mn = ys.min(axis=0)
    for s in range(wl.spec.shape[0]):
        best, _, _ = eng.pgd_attack(nid, wl.spec[s:s + 1], lo, hi, xs[:512], 60, 0.05)
        mn[s] = min(mn[s], best.min())
    root, _, _, _ = eng.crown_bounds(nid, wl.spec, lo, hi)
    s = int(np.argmax(mn - root[0]))
    assert mn[s] - root[0][s] > 1e-3
    row = wl.spec[s]

    def prop(t):
        return formats.Property(lo, hi, [[formats.Atom(-row, float(t))]])

    t_safe = float(root[0][s] + 0.7 * (mn[s] - root[0][s]))
    r = bab.verify_input_split(eng, nid, net, prop(t_safe), batch=512)
    assert r.status == "verified" and r.rounds >= 2 and r.domains_bounded > 1 and r.open_domains == 0
    t_unsafe = float(mn[s] + 1e-3 * max(1.0, abs(mn[s])))
    r = bab.verify_input_split(eng, nid, net, prop(t_unsafe), batch=512)
    assert r.status == "violated"
    assert float(row @ W.forward(net, r.counterexample)) <= t_unsafe
    assert np.all(r.counterexample >= lo) and np.all(r.counterexample <= hi)
    eng.release_network(nid)


def test_command_line_surface_and_exit_codes(tmp_path):
    """`python -m ny_b200 beta-crown|verify MODEL -p PROPERTY`: the reference's result block and exit codes
    (0 proved, 1 falsified, 2 unknown, 4 operational error) on the quick-start network."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    model = tmp_path / "abs.nnet"
    model.write_text(ABS_NNET)
    safe, unsafe = tmp_path / "safe.vnnlib", tmp_path / "unsafe.vnnlib"
    safe.write_text(_prop(">=", 2.0))
    unsafe.write_text(_prop(">=", 0.5))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))

    def run(*args):
        r = subprocess.run([sys.executable, "-m", "ny_b200", *args], env=env, cwd=root, capture_output=True, text=True, timeout=300)
        return r.returncode, r.stdout

    rc, out = run("beta-crown", str(model), "-p", str(safe))
    assert rc == 0 and "Status: VERIFIED" in out
    rc, out = run("beta-crown", str(model), "-p", str(unsafe))
    assert rc == 1 and "Status: VIOLATED" in out and "Counterexample input" in out
    rc, out = run("beta-crown", str(model), "-p", str(safe), "--input-split")
    assert rc == 0 and "Status: VERIFIED" in out
    rc, out = run("beta-crown", str(model), "-p", str(safe), "--resident")      # the open set on the device
    assert rc == 0 and "Status: VERIFIED" in out
    rc, out = run("beta-crown", str(model), "-p", str(unsafe), "--resident", "--beta-iterations", "0")
    assert rc == 1 and "Status: VIOLATED" in out
    rc, out = run("beta-crown", str(model), "-p", str(safe), "--resident", "--branching", "fsb")
    assert rc == 4
    rc, out = run("verify", str(model), "-p", str(safe), "--method", "crown")
    assert rc == 0
    rc, out = run("verify", str(model), "-p", str(safe), "--method", "ibp")      # the interval pass only reaches y <= 2
    assert rc == 2 and "Status: UNKNOWN" in out
    rc, out = run("verify", str(model), "-p", str(safe), "--method", "ibp", "--allow-unknown")
    assert rc == 0
    rc, out = run("beta-crown", str(tmp_path / "missing.nnet"), "-p", str(safe))
    assert rc == 4


_SHARDED = r"""
import json, os, sys
import numpy as np
import torch
import torch.distributed as dist
from ny_b200 import B200Engine, bab, formats
from ny_b200 import workloads as W

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
eng = B200Engine(int(os.environ["LOCAL_RANK"]))
wl = W.config_mlp_bab(seed=83, hidden=24, depth=3, n_in=4, n_out=3, eps=0.2, n_fix=0)
nid = eng.register_network(wl.net)
mn = W.sample_min_margin(wl, 200000, 3)
root, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
s = int(np.argmax(mn - root[0]))
t = float(root[0][s] + 0.9 * (mn[s] - root[0][s]))
prop = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], t)]])
one = bab.verify(eng, nid, wl.net, prop, batch=32, max_rounds=400, optimize_iterations=20, warm_start=False)
many = bab.verify(eng, nid, wl.net, prop, batch=32, max_rounds=400, optimize_iterations=20, warm_start=False, dist=dist,
                  dist_device=f"cuda:{os.environ['LOCAL_RANK']}")
out = dict(rank=rank, one=[one.status, one.rounds, one.domains_bounded], many=[many.status, many.rounds, many.domains_bounded])
gathered = [None] * world
dist.all_gather_object(gathered, out)
if rank == 0:
    print("RESULT " + json.dumps(gathered))
dist.destroy_process_group()
"""


def test_sharded_search_over_nccl(tmp_path):
    """The same search on one GPU and sharded over two (one process per GPU, NCCL): same verdict, the same domains
    bounded in total (the order of a breadth-first search does not change what is explored without warm starts),
    fewer rounds."""
    import json
    import os
    import subprocess
    import sys

    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "sharded.py"
    script.write_text(_SHARDED)
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29577", str(script)], env=env, cwd=root, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    assert all(x["one"] == res[0]["one"] and x["many"] == res[0]["many"] for x in res)
    one, many = res[0]["one"], res[0]["many"]
    assert one[0] == many[0] == "verified"
    assert many[2] == one[2] and many[1] < one[1]


@pytest.mark.gpu
@pytest.mark.parametrize("branching", [0, 1, 2])
def test_device_resident_frontier_runs_the_host_loop_search(eng, branching):
    """The search with the open domain set kept on the device (nyb200_frontier_*: pop, bound, prune, branch, push
    children in one call per round) against the host loop with the same settings: the same domains in the same order,
    so the same verdict, the same number of rounds, the same number of domains bounded and left open - on a property
    the search closes, on one it cannot close in the given rounds, and with batches smaller than the frontier (the
    ring wraps)."""
    wl = W.config_mlp_bab(seed=83, hidden=16, depth=3, n_in=6, n_out=4, eps=0.25, n_fix=0)
    net = wl.net
    nid = eng.register_network(net)
    root_lo, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    mn = W.sample_min_margin(wl, 200000, 3)
    s = int(np.argmax(mn - root_lo[0]))
    row = wl.spec[s]

    def prop(t):
        return formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-row, float(t))]])

    cases = [(float(root_lo[0][s] + 0.25 * (mn[s] - root_lo[0][s])), 64, 40),     # an easy threshold
             (float(root_lo[0][s] + 0.9 * (mn[s] - root_lo[0][s])), 48, 12)]      # a hard one: runs out of rounds, ring wraps
    for t, batch, rounds in cases:
        a = bab.verify(eng, nid, net, prop(t), batch=batch, max_rounds=rounds, branching=branching)
        b = bab.verify_resident(eng, nid, net, prop(t), batch=batch, max_rounds=rounds, branching=branching)
        assert (a.status, a.rounds, a.domains_bounded, a.open_domains) == (b.status, b.rounds, b.domains_bounded, b.open_domains)
        assert a.domains_bounded > 3
    # a small capacity is refused cleanly, not overrun
    from ny_b200 import EngineError

    p = prop(cases[1][0])
    spec, thr, owner = bab._rows(p)
    _, _, il, iu = eng.crown_bounds(nid, spec, p.in_lo, p.in_hi)
    eng.frontier_create(nid, spec, thr, owner, 1, p.in_lo, p.in_hi, il[0], iu[0], max_depth=30, capacity=8)
    with pytest.raises(EngineError):
        for _ in range(20):
            eng.frontier_round(4, branching)
    eng.frontier_destroy()
    eng.release_network(nid)


@pytest.mark.gpu
def test_records_taken_from_the_device_frontier_and_given_back_leave_the_search_unchanged(eng):
    """nyb200_frontier_take / give (the levelling moves of the sharded search): records leave from the back of the
    ring into device arrays, keep their contents, and a search that gets them back bounds the same domains."""
    import torch

    wl = W.config_mlp_bab(seed=83, hidden=16, depth=3, n_in=6, n_out=4, eps=0.25, n_fix=0)
    nid = eng.register_network(wl.net)
    root_lo, _, il, iu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    mn = W.sample_min_margin(wl, 200000, 3)
    s = int(np.argmax(mn - root_lo[0]))
    p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root_lo[0][s] + 0.9 * (mn[s] - root_lo[0][s])))]])
    spec, thr, owner = bab._rows(p)
    depth, cap = 20, 64     # a small ring, so that the taken range wraps

    def run(interrupt):
        eng.frontier_create(nid, spec, thr, owner, 1, p.in_lo, p.in_hi, il[0], iu[0], max_depth=depth, capacity=cap)
        log = []
        for r in range(9):
            log.append(eng.frontier_round(6, 1))
            if interrupt and r in (3, 6):
                n = eng.frontier_count()
                k = n - 2
                sp = torch.full((k, 4 * depth), -7, dtype=torch.int32, device="cuda:0")
                ns = torch.full((k,), -7, dtype=torch.int32, device="cuda:0")
                assert eng.frontier_take(k, sp.data_ptr(), ns.data_ptr()) == k and eng.frontier_count() == 2
                hist = ns.cpu().numpy()
                assert hist.min() >= 1 and hist.max() <= r + 1
                rec = sp.cpu().numpy().reshape(k, depth, 4)
                for i in range(k):   # (relu, neuron, sign, beta) of every used slot
                    assert np.all(np.abs(rec[i, : hist[i], 2]) == 1) and np.all(rec[i, : hist[i], 0] >= 0)
                eng.frontier_give(k, sp.data_ptr(), ns.data_ptr())
                assert eng.frontier_count() == n
        eng.frontier_destroy()
        return log

    plain = run(False)
    assert run(True) == plain and plain[-1][0] > 0
    # asking for more than the ring holds hands over what is there
    eng.frontier_create(nid, spec, thr, owner, 1, p.in_lo, p.in_hi, il[0], iu[0], max_depth=depth, capacity=cap)
    sp = torch.zeros((5, 4 * depth), dtype=torch.int32, device="cuda:0")
    ns = torch.zeros((5,), dtype=torch.int32, device="cuda:0")
    assert eng.frontier_take(5, sp.data_ptr(), ns.data_ptr()) == 1 and eng.frontier_count() == 0    # only the root is there
    assert eng.frontier_round(6, 1)[0] == 0                                                        # nothing to bound
    eng.frontier_give(1, sp.data_ptr(), ns.data_ptr())
    assert eng.frontier_count() == 1
    eng.frontier_destroy()

    eng.release_network(nid)


_SHARDED_RESIDENT = r"""
import json, os, sys
import numpy as np
import torch
import torch.distributed as dist
from ny_b200 import B200Engine, bab, formats
from ny_b200 import workloads as W

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
lr = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(lr)
dist.init_process_group("nccl")
eng = B200Engine(lr)
wl = W.config_mlp_bab(seed=83, hidden=24, depth=3, n_in=4, n_out=3, eps=0.2, n_fix=0)
nid = eng.register_network(wl.net)
mn = W.sample_min_margin(wl, 200000, 3)
root, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
s = int(np.argmax(mn - root[0]))
out = dict(rank=rank)
for name, frac, rounds, batch in (("closes", 0.5, 200, 2), ("open", 0.97, 9, 16)):
    t = float(root[0][s] + frac * (mn[s] - root[0][s]))
    prop = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], t)]])
    one = bab.verify_resident(eng, nid, wl.net, prop, batch=batch, max_rounds=rounds)
    many = bab.verify_resident(eng, nid, wl.net, prop, batch=batch, max_rounds=rounds, dist=dist, dist_device=f"cuda:{lr}")
    out[name] = dict(one=[one.status, one.rounds, one.domains_bounded, one.open_domains],
                     many=[many.status, many.rounds, many.domains_bounded, many.open_domains], exchange=many.exchange)
gathered = [None] * world
dist.all_gather_object(gathered, out)
if rank == 0:
    print("RESULT " + json.dumps(gathered))
dist.destroy_process_group()
"""


def test_sharded_search_on_device_resident_frontiers_over_nccl(tmp_path):
    """Every rank keeps its own device frontier; records move between the GPUs' rings over NCCL, device to device.
    Against the single-GPU resident search: the same verdict and, when the search closes, the same domains bounded in
    fewer rounds (two domains per rank and round); on a search that runs out of rounds, at least as many domains bounded
    in the same rounds."""
    import json
    import os
    import subprocess
    import sys

    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "sharded_resident.py"
    script.write_text(_SHARDED_RESIDENT)
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29578", str(script)], env=env, cwd=root, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    for name in ("closes", "open"):
        assert all(x[name]["one"] == res[0][name]["one"] and x[name]["many"] == res[0][name]["many"] for x in res)
    one, many = res[0]["closes"]["one"], res[0]["closes"]["many"]
    assert one[0] == many[0] == "verified" and many[2] == one[2] and many[1] < one[1]
    one, many = res[0]["open"]["one"], res[0]["open"]["many"]
    assert one[0] == many[0] == "unknown" and many[1] == one[1] and many[2] >= one[2]
    moved = sum(x["closes"]["exchange"]["records_moved"] for x in res)
    assert moved > 0 and moved % 2 == 0   # every move is counted by its sender and by its receiver


@pytest.mark.gpu
def test_device_resident_search_dumps_its_frontier_and_resumes(eng, tmp_path):
    """A resident search stopped by its round limit writes the open records (front first) in the host loop's dump
    format; resumed from there, by either loop, it ends where the uninterrupted search ends."""
    wl = W.config_mlp_bab(seed=83, hidden=24, depth=3, n_in=4, n_out=3, eps=0.2, n_fix=0)
    net = wl.net
    nid = eng.register_network(net)
    root_lo, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    mn = W.sample_min_margin(wl, 200000, 3)
    s = int(np.argmax(mn - root_lo[0]))
    p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root_lo[0][s] + 0.5 * (mn[s] - root_lo[0][s])))]])
    whole = bab.verify_resident(eng, nid, net, p, batch=2, max_rounds=200)
    assert whole.status == "verified" and whole.rounds > 4
    dump = tmp_path / "frontier.npz"
    first = bab.verify_resident(eng, nid, net, p, batch=2, max_rounds=3, checkpoint=dump)
    assert first.status == "unknown" and first.open_domains > 0 and dump.exists()
    hist, _, _, rounds, bounded = bab.load_frontier(dump, p)
    assert len(hist) == first.open_domains and rounds == 3 and bounded == first.domains_bounded
    rest = bab.verify_resident(eng, nid, net, p, batch=2, max_rounds=200, resume=dump)
    assert rest.status == "verified" and rest.domains_bounded == whole.domains_bounded and rest.rounds == whole.rounds - 3
    host = bab.verify(eng, nid, net, p, batch=2, max_rounds=200, resume=dump)
    assert host.status == "verified" and host.domains_bounded == whole.domains_bounded and host.rounds == rest.rounds
    other = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root_lo[0][s]) - 1.0)]])
    with pytest.raises(ValueError):
        bab.verify_resident(eng, nid, net, other, batch=2, max_rounds=3, resume=dump)
    eng.release_network(nid)


@pytest.mark.gpu
@pytest.mark.parametrize("branching", [1, 2])
def test_device_resident_optimising_search_with_warm_starts_runs_the_host_loop_search(eng, branching):
    """nyb200_frontier_round_optimized: every domain's slopes and multipliers optimised on the device, children
    starting from their parent's (slopes in a device ring, multipliers in the split records).  Against the host loop
    with the same settings (which downloads the parameters and uploads them with the children): the same domains with
    the same starting points in the same order, so the same verdict, rounds and domain counts - on a threshold that
    one bound per domain does not close in these rounds."""
    wl = W.config_mlp_bab(seed=83, hidden=24, depth=3, n_in=4, n_out=3, eps=0.2, n_fix=0)
    net = wl.net
    nid = eng.register_network(net)
    root_lo, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    mn = W.sample_min_margin(wl, 200000, 3)
    s = int(np.argmax(mn - root_lo[0]))
    p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root_lo[0][s] + 0.9 * (mn[s] - root_lo[0][s])))]])
    for batch, rounds in ((32, 400), (5, 7)):    # closes; stops early with a frontier larger than the batch (ring wraps)
        a = bab.verify(eng, nid, net, p, batch=batch, max_rounds=rounds, branching=branching, optimize_iterations=6, warm_start=True)
        b = bab.verify_resident(eng, nid, net, p, batch=batch, max_rounds=rounds, branching=branching, optimize_iterations=6)
        assert (a.status, a.rounds, a.domains_bounded, a.open_domains) == (b.status, b.rounds, b.domains_bounded, b.open_domains)
    assert a.domains_bounded > 3
    plain = bab.verify_resident(eng, nid, net, p, batch=32, max_rounds=400, branching=branching)
    full = bab.verify_resident(eng, nid, net, p, batch=32, max_rounds=400, branching=branching, optimize_iterations=6)
    assert full.status == "verified" and (plain.status != "verified" or full.domains_bounded <= plain.domains_bounded)
    eng.release_network(nid)


@pytest.mark.gpu
def test_device_frontier_refuses_what_it_cannot_hold(eng):
    """Capacity, depth and argument checks of the frontier's transfer calls: refused with a status, nothing overrun."""
    import torch

    from ny_b200 import SPLIT_DTYPE, EngineError

    wl = W.config_mlp_bab(seed=83, hidden=16, depth=3, n_in=6, n_out=4, eps=0.25, n_fix=0)
    nid = eng.register_network(wl.net)
    root_lo, _, il, iu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[0], float(root_lo[0][0]) + 1.0)]])
    spec, thr, owner = bab._rows(p)
    with pytest.raises(EngineError):
        eng.frontier_count()                       # no frontier yet
    eng.frontier_create(nid, spec, thr, owner, 1, p.in_lo, p.in_hi, il[0], iu[0], max_depth=4, capacity=6)
    sp = torch.zeros((8, 16), dtype=torch.int32, device="cuda:0")
    ns = torch.ones((8,), dtype=torch.int32, device="cuda:0")
    with pytest.raises(EngineError):
        eng.frontier_give(6, sp.data_ptr(), ns.data_ptr())          # 1 + 6 > capacity
    eng.frontier_give(5, sp.data_ptr(), ns.data_ptr())
    assert eng.frontier_count() == 6
    with pytest.raises(EngineError):
        eng.frontier_upload(np.zeros((2, 5), SPLIT_DTYPE), np.array([1, 5], np.int32))     # deeper than max_depth
    with pytest.raises(EngineError):
        eng.frontier_upload(np.zeros((2, 3), SPLIT_DTYPE), np.array([1, 4], np.int32))     # length beyond the row
    with pytest.raises(EngineError):
        eng.frontier_upload(np.zeros((7, 2), SPLIT_DTYPE), np.ones(7, np.int32))           # more than capacity
    assert eng.frontier_count() == 6               # refused calls left the contents alone
    eng.frontier_upload(np.zeros((0, 1), SPLIT_DTYPE), np.zeros(0, np.int32))
    assert eng.frontier_count() == 0 and eng.frontier_download(4)[1].shape == (0,)
    eng.frontier_destroy()
    eng.release_network(nid)


@pytest.mark.gpu
def test_search_shared_by_the_engines_of_a_pool(eng):
    """verify_resident_pool: one device frontier per engine of an EnginePool on the same GPU, rounds on their own
    streams and threads, shards levelled ring to ring.  Against the single-frontier search: the same verdict and, when
    the search closes, the same domains bounded in fewer rounds; plain and optimising."""
    from ny_b200.pool import EnginePool

    wl = W.config_mlp_bab(seed=83, hidden=24, depth=3, n_in=4, n_out=3, eps=0.2, n_fix=0)
    nid = eng.register_network(wl.net)
    root_lo, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    mn = W.sample_min_margin(wl, 200000, 3)
    s = int(np.argmax(mn - root_lo[0]))
    pool = EnginePool(0, 3)
    h = pool.register_network(wl.net)
    for frac, it in ((0.5, 0), (0.9, 6)):
        p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root_lo[0][s] + frac * (mn[s] - root_lo[0][s])))]])
        one = bab.verify_resident(eng, nid, wl.net, p, batch=2, max_rounds=300, optimize_iterations=it)
        many = bab.verify_resident_pool(pool, h, wl.net, p, batch=2, max_rounds=300, optimize_iterations=it)
        assert one.status == many.status == "verified"
        assert many.rounds < one.rounds and many.exchange["records_moved"] > 0
        if it == 0:   # without warm starts the order of a complete search does not change what it bounds
            assert many.domains_bounded == one.domains_bounded
    # a search that runs out of rounds reports what is left on all engines
    p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root_lo[0][s] + 0.97 * (mn[s] - root_lo[0][s])))]])
    cut = bab.verify_resident_pool(pool, h, wl.net, p, batch=4, max_rounds=6)
    assert cut.status == "unknown" and cut.open_domains > 0 and cut.rounds == 6
    pool.close()
    eng.release_network(nid)


@pytest.mark.gpu
def test_verdict_only_refinement_re_evaluates_only_what_could_change_a_verdict(eng):
    """nyb200_frontier_set_refinement(1): a round re-evaluates in binary64 only the domains whose lower bound misses
    its threshold by less than twice the row's rounding charge.  Far from the threshold nothing is re-evaluated although
    the parity rule flags the domains; the search reaches the same verdict either way, and a verified verdict is
    confirmed by sampling."""
    wl = W.config_mlp_bab(seed=83, hidden=24, depth=3, n_in=4, n_out=3, eps=0.2, n_fix=0)
    net = wl.net
    nid = eng.register_network(net)
    root_lo, _, il, iu = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    mn = W.sample_min_margin(wl, 200000, 3)
    s = int(np.argmax(mn - root_lo[0]))
    for frac in (0.5, 0.9):
        t = float(root_lo[0][s] + frac * (mn[s] - root_lo[0][s]))
        p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], t)]])
        a = bab.verify_resident(eng, nid, net, p, batch=16, max_rounds=300, optimize_iterations=6 if frac > 0.6 else 0)
        b = bab.verify_resident(eng, nid, net, p, batch=16, max_rounds=300, optimize_iterations=6 if frac > 0.6 else 0,
                                refinement="verdict")
        assert a.status == b.status == "verified" and t < mn[s]
        assert b.domains_bounded >= a.domains_bounded - 2 and b.domains_bounded <= 2 * a.domains_bounded + 8
        # the host loop with per-batch thresholds (nyb200_batch_set_thresholds) bounds the same domains
        h = bab.verify(eng, nid, net, p, batch=16, max_rounds=300, optimize_iterations=6 if frac > 0.6 else 0, refinement="verdict")
        assert (h.status, h.rounds, h.domains_bounded) == (b.status, b.rounds, b.domains_bounded)
    # rounds far from the threshold: the parity rule sends domains to binary64, the verdict rule none
    p = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(mn[s]) + 5.0)]])      # cannot be verified
    spec, thr, owner = bab._rows(p)
    counts = {}
    for mode in (False, True):
        eng.set_refine_tolerance(1e-9)        # the parity rule at a tolerance that flags everything
        eng.frontier_create(nid, spec, thr, owner, 1, p.in_lo, p.in_hi, il[0], iu[0], max_depth=12, capacity=4096)
        eng.frontier_set_refinement(mode)
        n = 0
        for _ in range(6):
            eng.frontier_round(64, 1)
            n += eng.batch_refined()
        counts[mode] = (n, eng.frontier_count())
        eng.frontier_destroy()
    eng.set_refine_tolerance(5e-5)
    assert counts[False][0] > 0 and counts[True][0] == 0 and counts[False][1] == counts[True][1]
    eng.release_network(nid)
