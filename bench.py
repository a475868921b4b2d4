"""Benchmark of the hot path: beta-CROWN bounding of a batch of BaB domains.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the hot path over one batch: for every domain the interval forward pass
under its splits, the CROWN backward pass with alpha slopes / beta multipliers for both bound
directions of every specification row, and concretisation.  Workload: ReLU MLP 784 -> 8x256 -> 10,
9 specification rows, 4096 domains per GPU each fixing 8 seeded unstable neurons (synthetic, seeded).
With N > 1 (launched by torch.distributed.run) every rank bounds its own shard of N*4096 domains
(weak scaling); the only exchange is the per-round min-reduce of the global lower bound over NCCL.

Prints ONE JSON line (rank 0).  `value` is timed with inputs resident in HBM; `e2e` is the same metric
through the host-buffer C-ABI call (host->device copy of the step's inputs from pinned memory,
device->host read of the bounds, inside the timed region).  By default three batches are in flight per GPU
(`--in-flight 3`: one engine, stream and workspace per batch, the batches taking turns step by step, one host
thread per batch in the e2e leg), because independent batches overlap on the device; the kernel timings of the
roofline come from a region with a single batch in flight, and its step time is reported next to the other.  `--impl reference` times the CPU
restatement of the reference's own path (oracle/, a thread pool over domains) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_PER_GPU = 4096
_emit = lambda obj: print(json.dumps(obj))
METRIC = "BaB domains bounded/sec (beta-CROWN)"
UNIT = "domains/s"
# Algorithmic work per domain for this network (fp32 coefficients, both bound directions carried):
# contraction FLOPs 2*S*2*(10*256 + 7*256^2 + 256*784) and layer-by-layer bytes (each coefficient tile
# written once and read once per layer, per-neuron relaxation inputs, 2*S outputs).
S_ROWS = 9
FLOPS_PER_DOMAIN = 2 * (2 * S_ROWS) * (10 * 256 + 7 * 256 * 256 + 256 * 784)
BYTES_PER_DOMAIN = 2 * (2 * S_ROWS * 8 * 256 * 4) + 2 * S_ROWS * 784 * 4 + 8 * 256 * 3 * 4 + 2 * S_ROWS * 4


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def measure_tf32_peak(device):
    """Dense TF32 GEMM rate of this GPU, measured the way the bf16 figure of MEASURED_PEAKS.json was: torch.matmul
    (a library GEMM is fine for a peak) on 8192^3 fp32 operands with TF32 allowed, best of 10 after warm-up."""
    import torch

    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device=device)
        b = torch.randn(n, n, device=device)
        for _ in range(3):
            a @ b
        torch.cuda.synchronize(device)
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            a @ b
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        del a, b
        torch.cuda.empty_cache()
        return 2.0 * n ** 3 / (best / 1e3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def committed_traffic(kernel: str, domains: int):
    """DRAM bytes per launch of `kernel` at `domains` domains from the committed ncu captures (profiles/traffic.json:
    dram__bytes_read.sum + dram__bytes_write.sum of one launch at the listed batch sizes), or None when no capture at
    this size is on record."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return None
    rec = json.load(open(p)).get(kernel, {})
    v = rec.get(str(domains))
    return None if v is None else float(v)


def oracle_parity(eng, nid, wl, rl, ru, splits, ns, lo, hi, inf, n=32):
    """Outside the timed region: the device bounds of the first n domains against the CPU oracle, with the rule the
    parity tests use (relative to max(|oracle bound|, floor * the domain's largest bound))."""
    from oracle import ny_oracle as O

    onet = O.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    olo, ohi, oinf, _ = O.bab_bound_batch(onet, wl.in_lo, wl.in_hi, rl2, ru2, splits[:n], ns[:n], 1)
    same_inf = bool(np.array_equal(oinf.astype(bool), inf[:n].astype(bool)))
    f = ~oinf.astype(bool)
    floor = 1e-2
    dev = np.concatenate([lo[:n], hi[:n]], axis=1)[f].astype(np.float64)
    ref = np.concatenate([olo, ohi], axis=1)[f].astype(np.float64)
    den = np.maximum(np.abs(ref), floor * np.abs(ref).max(axis=1, keepdims=True))
    rel = np.abs(dev - ref) / den
    unfloored = np.abs(dev - ref) / np.maximum(np.abs(ref), 1e-30)
    verdict_same = bool(np.array_equal((lo[:n][f] > 0).all(axis=1), (olo[f] > 0).all(axis=1)))
    return {"max_rel": float(rel.max()), "max_rel_unfloored": float(unfloored.max()), "n_domains_checked": int(f.sum()),
            "tolerance": 1e-4, "floor": "denominator max(|oracle bound|, 1e-2 * the domain's largest |bound|)",
            "infeasible_flags_identical": same_inf, "verdicts_at_threshold_0_identical": verdict_same,
            "never_above_oracle_lower_by_more_than_1e-6_scale": bool(np.all(lo[:n][f] <= olo[f] + 1e-6 * np.abs(ref).max(axis=1, keepdims=True)))}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self, keep_busy=None):
        """keep_busy: a callable that runs a little more of the same GPU work; used (untimed) while waiting for a
        first sample when nvidia-smi was slower to start than the whole measurement."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        deadline = time.time() + 5.0
        while keep_busy is not None and len(self.rows) < 2 and time.time() < deadline and self.proc.poll() is None:
            keep_busy()
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(wl, rl, ru, sample_domains: int, repeats: int = 1):
    """Times the oracle (CPU restatement of the reference path) on `sample_domains` domains of the same
    workload with all host threads.  Returns (domains/s, threads)."""
    from oracle import ny_oracle as O
    from ny_b200 import workloads as W

    onet = O.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
    S = wl.spec.shape[0]
    rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
    ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
    splits, ns = W.draw_domains(wl, rl, ru, sample_domains)
    best = None
    used = 1
    for _ in range(repeats):
        t0 = time.perf_counter()
        _, _, _, used = O.bab_bound_batch(onet, wl.in_lo, wl.in_hi, rl2, ru2, splits, ns, 1, 0)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_domains / best, used


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU path (restated in oracle/) on the host cores."""
    if rank != 0:
        return
    from oracle import ny_oracle as O
    from ny_b200 import workloads as W

    wl = W.config_mlp_bab()
    onet = O.Net(wl.net.weights, wl.net.biases)
    rl, ru = O.ibp_forward(onet, wl.in_lo, wl.in_hi)
    sample = args.ref_sample
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(wl, rl, ru, max(8, sample // 8))
    times = []
    threads = 1
    for _ in range(args.steps):
        t0 = time.perf_counter()
        _, threads = cpu_baseline(wl, rl, ru, sample)
        times.append(time.perf_counter() - t0)
    ms = 1e3 * float(np.mean(times))
    value = sample / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic",
        "config": {"workload": "beta-CROWN bound of BaB domains, ReLU MLP 784->8x256->10, 9 spec rows, 8 splits/domain",
                   "domains_per_step": sample, "same_config": sample == D_PER_GPU,
                   "note": "CPU restatement of the reference path (naive binary64 loops over a thread pool; the Rust reference "
                           "with its faer SIMD GEMMs cannot be built here)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample} domains per step of the {D_PER_GPU}-domain workload"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


class _DevPtr:
    """Exposes a raw device pointer to torch through __cuda_array_interface__."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 3}


def run_ours(args, rank, world, local_rank):
    import torch

    from ny_b200 import B200Engine
    from ny_b200 import workloads as W

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    stream = torch.cuda.current_stream()
    tf32_peak = None
    if rank == 0 and not args.no_peak:
        tf32_peak = measure_tf32_peak(f"cuda:{local_rank}")   # roofline denominator; well before the timed region
    eng = B200Engine(local_rank, stream.cuda_stream)
    from ny_b200 import engine as E

    eng.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
    eng.set_fusion(bool(args.fusion))
    reserve = args.reserve_sms if args.reserve_sms >= 0 else (2 if world > 1 else 0)   # room for the min-reduce beside the kernels
    eng.set_reserved_sms(reserve)
    eng._path_name = args.path
    wl = W.config_mlp_bab()
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)  # root interval bounds, computed on the device
    rl, ru = pl[0].copy(), pu[0].copy()
    D = args.domains
    splits, ns = W.draw_domains(wl, rl, ru, D, first=rank * D)
    S = wl.spec.shape[0]

    # ---- resident timing ------------------------------------------------------------------
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    min_t = torch.as_tensor(_DevPtr(eng.batch_min_lower_device(), 1), device=f"cuda:{local_rank}")

    from ny_b200 import sharding

    # The round's only exchange, the min-reduce of the global lower bound, runs on a second stream: the main stream
    # copies the round's minimum into one of two slots, the side stream reduces that slot across ranks while the main
    # stream is already in the next round's forward pass.  A slot is reused two rounds later, after the side stream's
    # event of its previous use.
    side = torch.cuda.Stream(device=local_rank) if dist is not None else None
    lb_slot = [torch.empty(1, device=f"cuda:{local_rank}") for _ in range(2)]
    lb_done = [None, None]
    counter = {"round": 0, "late_reruns": 0}

    def step():
        eng.batch_run()
        # No host synchronisation per round: the run's last kernel publishes its status words to mapped host memory
        # and the host looks at them without waiting.  A round that flagged domains for the binary64 re-evaluation
        # (none on this workload) is seen a round or two late and re-evaluated then, inside the timed region.
        _, attention = eng.batch_poll()
        if attention:
            eng.batch_refined()
            counter["late_reruns"] += 1
        if dist is not None:
            i = counter["round"] & 1
            if lb_done[i] is not None:
                stream.wait_event(lb_done[i])
            lb_slot[i].copy_(min_t)
            ready = torch.cuda.Event()
            ready.record(stream)
            with torch.cuda.stream(side):
                side.wait_event(ready)
                sharding.allreduce_min(lb_slot[i], dist)
                lb_done[i] = torch.cuda.Event()
                lb_done[i].record(side)
        counter["round"] += 1

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()   # before the warm-up, so that nvidia-smi is already reporting when the timed region runs
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    eng.timing_enable(True)
    eng.timing_reset()
    l0 = eng.launch_count()
    # The timed region is args.steps steps between two events; it is repeated back to back (`blocks` times, 30 by
    # default) and the reported step time is the median block's, with the spread next to it: one block of 20 steps
    # lasts well under 40 ms, too short for a single sample to be a stable number.
    blocks = max(1, args.blocks)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    barrier()
    t0 = time.perf_counter()
    evs[0].record(stream)
    for b in range(blocks):
        for _ in range(args.steps):
            step()
        if b == blocks - 1:
            eng.batch_refined()   # the last rounds' status, with a synchronisation: the region ends with final bounds
        evs[b + 1].record(stream)
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    block_ms = np.array([evs[b].elapsed_time(evs[b + 1]) for b in range(blocks)])
    launches = (eng.launch_count() - l0) // blocks
    gemm_ms, _ = eng.timing_read("gemm")
    chain_ms, _ = eng.timing_read("chain")
    fwd_ms, _ = eng.timing_read("forward")
    bwd_ms, _ = eng.timing_read("backward")
    eng.timing_enable(False)
    lo, hi, inf = eng.batch_download()
    refined = eng.batch_refined()

    # ---- resident timing with several batches in flight -------------------------------------
    # One engine per batch (own stream, own workspace, own resident domains); a step is still one batch, the engines
    # take turns.  Kernels of different batches are independent, so the latency-bound interval pass of one overlaps the
    # tensor-bound chain of another and the launch gaps and tails of both fill up.  The block's end event is recorded
    # on the first stream after it has waited for the others.
    B = max(1, args.in_flight)
    engs, nids, streams, dom = [eng], [nid], [stream], [(splits, ns)]
    for i in range(1, B):
        st_i = torch.cuda.Stream(device=local_rank)
        e_i = B200Engine(local_rank, st_i.cuda_stream)
        e_i.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
        e_i.set_fusion(bool(args.fusion))
        e_i.set_reserved_sms(reserve)
        e_i.set_launch_overlap(False)
        n_i = e_i.register_network(wl.net)
        d_i = W.draw_domains(wl, rl, ru, D, first=(world * i + rank) * D)
        e_i.batch_upload(n_i, wl.spec, wl.in_lo, wl.in_hi, rl, ru, d_i[0], d_i[1], mode=1)
        engs.append(e_i); nids.append(n_i); streams.append(st_i); dom.append(d_i)
    block_ms_multi = None
    launches_multi = 0
    if B > 1:
        eng.set_launch_overlap(False)   # dependent launches pay with one batch in flight only (nyb200_set_launch_overlap)
        mins = [min_t] + [torch.as_tensor(_DevPtr(e.batch_min_lower_device(), 1), device=f"cuda:{local_rank}") for e in engs[1:]]
        slots = [[torch.empty(1, device=f"cuda:{local_rank}") for _ in range(2)] for _ in range(B)]
        done = [[None, None] for _ in range(B)]
        turn = {"k": 0}

        def step_multi():
            i = turn["k"] % B
            r = (turn["k"] // B) & 1
            e, st = engs[i], streams[i]
            e.batch_run()
            _, attention = e.batch_poll()
            if attention:
                e.batch_refined()
                counter["late_reruns"] += 1
            if dist is not None:
                if done[i][r] is not None:
                    st.wait_event(done[i][r])
                with torch.cuda.stream(st):
                    slots[i][r].copy_(mins[i])
                ready = torch.cuda.Event()
                ready.record(st)
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    sharding.allreduce_min(slots[i][r], dist)
                    done[i][r] = torch.cuda.Event()
                    done[i][r].record(side)
            turn["k"] += 1

        def join_streams():
            for st in streams[1:]:
                ev = torch.cuda.Event()
                ev.record(st)
                stream.wait_event(ev)

        for _ in range(max(args.warmup, 3) * B):
            step_multi()
        barrier()
        l0 = sum(e.launch_count() for e in engs)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
        t0 = time.perf_counter()
        evs[0].record(stream)
        for st in streams[1:]:
            st.wait_event(evs[0])
        for b in range(blocks):
            for _ in range(args.steps):
                step_multi()
            if b == blocks - 1:
                for e in engs:
                    e.batch_refined()
            join_streams()
            evs[b + 1].record(stream)
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        block_ms_multi = np.array([evs[b].elapsed_time(evs[b + 1]) for b in range(blocks)])
        launches_multi = (sum(e.launch_count() for e in engs) - l0) // blocks
        lo_again = eng.batch_download()[0]
        assert np.array_equal(lo_again, lo), "a batch's bounds changed with other batches in flight"
        eng.set_launch_overlap(True)

    # ---- end-to-end: host buffers in pinned memory through the C-ABI call ------------------
    def pinned(a):
        t = torch.empty(a.nbytes, dtype=torch.uint8, pin_memory=True)
        v = t.numpy().view(a.dtype).reshape(a.shape)
        v[...] = a
        return v, t

    sp_p, _k1 = pinned(splits)
    ns_p, _k2 = pinned(ns)
    e2e_calls = max(2, min(args.steps, 10)) * (3 if blocks > 1 else 1)
    for _ in range(2):
        eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, sp_p, ns_p, mode=1)
    barrier()
    e2e_times = []
    for _ in range(e2e_calls):
        t1 = time.perf_counter()
        elo, ehi, einf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, sp_p, ns_p, mode=1)
        e2e_times.append((time.perf_counter() - t1) * 1e3)   # the call returns with the bounds on the host
    barrier()

    # ---- the same calls with `in_flight` batches in flight (ny_b200.pool.EnginePool: one engine, stream, workspace and
    # host thread per batch, the batches handed out in turn), so that one batch's transfers and host work overlap
    # another's kernels; every batch still travels host -> device -> host inside its call
    pair_ms = None
    for e in engs[1:]:
        e.close()
    if B > 1:
        from ny_b200.pool import EnginePool

        def configure(e):
            e.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
            e.set_fusion(bool(args.fusion))

        pool = EnginePool(local_rank, B, configure)
        handle = pool.register_network(wl.net)
        pinned_dom = [(pinned(x[0])[0], pinned(x[1])[0]) for x in dom]
        pool_calls = B * max(4, e2e_calls // 2)
        work = [(wl.spec, wl.in_lo, wl.in_hi, rl, ru, pinned_dom[k % B][0], pinned_dom[k % B][1], 1) for k in range(pool_calls)]
        pool.bound_batches(handle, work[: 2 * B])
        barrier()
        t1 = time.perf_counter()
        results = pool.bound_batches(handle, work)
        pair_ms = (time.perf_counter() - t1) * 1e3 / pool_calls    # the calls return with the bounds on the host
        barrier()
        assert np.array_equal(results[0][0], lo) and np.array_equal(results[B][0], lo), "the batches in flight disturbed each other"
        pool.close()

    def busy():
        for _ in range(20):
            eng.batch_run()
        torch.cuda.synchronize()

    clocks = sampler.stop(busy)
    assert np.array_equal(elo, lo), "resident and host-buffer paths disagree"
    h2d = splits.nbytes + ns.nbytes + wl.spec.nbytes + wl.in_lo.nbytes + wl.in_hi.nbytes + rl.nbytes + ru.nbytes
    d2h = lo.nbytes + hi.nbytes + inf.nbytes

    rebalance = rebalance_exercise(dist, rank, world, f"cuda:{local_rank}", int(wl.net.n_pre)) if dist is not None else None
    def over_ranks(block_times):
        per = block_times / args.steps
        if dist is not None:  # max over ranks, block by block
            t = torch.tensor(per, device=f"cuda:{local_rank}", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per = t.cpu().numpy()
        return per

    per_step_one = over_ranks(block_ms)
    ms_one = float(np.median(per_step_one))
    per_step = over_ranks(block_ms_multi) if block_ms_multi is not None else per_step_one
    ms_per_step = float(np.median(per_step))
    e2e_single_ms = float(np.median(e2e_times))
    e2e_ms = pair_ms if pair_ms is not None else e2e_single_ms
    if dist is not None:
        t = torch.tensor([e2e_ms, e2e_single_ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, e2e_single_ms = float(t[0]), float(t[1])
    e2e_val = D * world / (e2e_ms / 1e3)
    value = D * world / (ms_per_step / 1e3)
    if B > 1:
        launches = launches_multi

    if rank == 0:
        peaks = load_peaks()
        dims = [int(x) for x in wl.net.dims]
        S2 = 2 * S
        fused = chain_ms > 0
        if eng_path_name(eng) == "f64":
            kernel, k_ms, k_flops = "k_gemm_f64", gemm_ms, FLOPS_PER_DOMAIN * D
        elif fused:
            # the dominant kernel: the fused chain carries the contractions of every layer but the first (wide) one
            kernel, k_ms = "k_chain", chain_ms
            k_flops = 2.0 * S2 * (dims[-1] * dims[-2] + sum(dims[k] * dims[k + 1] for k in range(1, len(dims) - 2))) * D
        else:
            kernel, k_ms, k_flops = "k_umma_tf32x3", gemm_ms, FLOPS_PER_DOMAIN * D
        achieved = k_flops / (k_ms / 1e3) / 1e12 if k_ms > 0 else None
        if tf32_peak:
            peak_tf, peak_src = tf32_peak, "measured tf32 (torch.matmul with TF32 allowed, 8192^3, best of 10, this run)"
        else:
            peak_tf, peak_src = peaks["bf16_tflops"] / 2.0, f"{peaks['source']} bf16 GEMM / 2 (TF32 not measured in this run)"
        traffic = committed_traffic(kernel, D)
        roofline = {
            "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
            "frac": (achieved / peak_tf) if achieved else None,
            "frac_step": FLOPS_PER_DOMAIN * D / (ms_per_step / 1e3) / 1e12 / peak_tf,
            "traffic": traffic,
            "traffic_source": ("dram__bytes_read.sum + dram__bytes_write.sum of one launch at this batch size, committed ncu "
                               "capture (profiles/traffic.json)") if traffic is not None else "no capture at this batch size on record",
            "kernel": kernel, "kernel_ms": k_ms, "kernel_algorithmic_gflop": k_flops / 1e9,
            "peak_source": peak_src,
            "kernel_timing": "CUDA events around each launch in the timed region with one batch in flight (with several in "
                             "flight other batches' kernels run inside a launch's event pair); frac_step uses the reported step",
            "hbm_view": {"achieved_gbs": BYTES_PER_DOMAIN * D / ((fwd_ms + bwd_ms) / 1e3) / 1e9 if (fwd_ms + bwd_ms) > 0 else None,
                         "peak_gbs": peaks["hbm_gbs"]},
            # every algorithmic product is issued as three TF32 products (Ah*Wh + Ah*Wl + Al*Wh): what the tensor pipe does
            "tensor_view": ({"issued_tflops": 3.0 * achieved, "frac_of_peak": 3.0 * achieved / peak_tf}
                            if achieved and eng_path_name(eng) != "f64" else None),
            "phase_ms": {"forward": fwd_ms, "backward": bwd_ms, "fused_chain": chain_ms, "per_layer_contractions": gemm_ms},
        }
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "ms_per_step_spread": {"blocks": int(blocks), "min": float(per_step.min()), "p10": float(np.percentile(per_step, 10)),
                                   "median": ms_per_step, "p90": float(np.percentile(per_step, 90)), "max": float(per_step.max())},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64" if eng_path_name(eng) == "f64" else "tf32x3", "data": "synthetic",
            "config": {"workload": "beta-CROWN bound of BaB domains, ReLU MLP 784->8x256->10, 9 spec rows (both bound "
                                   "directions), 8 splits/domain, constrained forward re-propagation",
                       "domains_per_gpu": D, "global_batch": D * world, "parallelism": f"domain-sharded x{world}",
                       "batches_in_flight": B,
                       "in_flight": (f"{B} resident batches of {D} domains per GPU, one engine and stream each, taking turns: a step is "
                                     "one batch; kernels of different batches overlap") if B > 1 else "one batch",
                       "ms_per_step_one_batch_in_flight": ms_one,
                       "l2": "per-step working set (per-domain tables 200 MB, coefficient rows 2 x 231 MB) exceeds the 126 MB L2",
                       "backward": "fused chain" if fused else "one launch per layer",
                       "feasible_domains": int((inf == 0).sum()),
                       "domains_sent_to_binary64_rerun": int(refined),
                       "rounds_rerun_after_a_late_status": int(counter["late_reruns"]),
                       "host_sync": "none per round (status words polled from mapped host memory); one at the end of the timed region",
                       "exchange": ("1-float MIN all-reduce of the global lower bound per round on a second stream, "
                                    "overlapping the next round") if world > 1 else "none (single rank)"},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": e2e_ms, "calls": len(e2e_times), "batches_in_flight": B if pair_ms is not None else 1,
                    "single_call_ms": e2e_single_ms,
                    "single_call_ms_spread": {"min": float(np.min(e2e_times)), "max": float(np.max(e2e_times))}},
            "gpu_launches": int(launches) * int(blocks), "gpu_launches_per_block": int(launches), "clocks": clocks, "roofline": roofline,
            "wall_ms_per_step": wall_ms / (args.steps * blocks),
        }
        if rebalance is not None:
            line["rebalance"] = rebalance
        if world == 1 and not args.no_parity:
            line["parity"] = oracle_parity(eng, nid, wl, rl, ru, splits, ns, lo, hi, inf)
        if world == 1 and not args.no_cpu_baseline:
            sample = args.cpu_sample
            v, threads = cpu_baseline(wl, rl, ru, sample)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{sample} domains of the same workload, one pass, all host threads"}
        _emit(line)
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


def run_alpha_crown(args, rank, world, local_rank):
    """Secondary workload (--workload alpha-crown): alpha-CROWN optimisation, MLP 784 -> 9x512 -> 10, box
    x0 +- 0.015, 9 spec rows, 20 projected-Adam iterations at lr 0.1 over 2048 input-split cells per GPU.
    One step = the whole 20-iteration optimisation of the batch; value = domains optimised per second."""
    import torch

    from ny_b200 import B200Engine
    from ny_b200 import engine as E
    from ny_b200 import workloads as W
    from oracle import ny_oracle as O  # cpu_baseline leg only (below)

    torch.cuda.set_device(local_rank)
    stream = torch.cuda.current_stream()
    eng = B200Engine(local_rank, stream.cuda_stream)
    eng.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
    wl = W.config_alpha_crown()
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = pl[0].copy(), pu[0].copy()
    D, iters = (args.domains if args.domains != D_PER_GPU else 2048), 20
    lo, hi = W.draw_input_cells(wl, 11, first=rank * D, count=D)
    sp0, ns = np.zeros((D, 0), E.SPLIT_DTYPE), np.zeros(D, np.int32)
    eng.batch_upload(nid, wl.spec, lo, hi, rl, ru, sp0, ns, mode=1)
    for _ in range(max(args.warmup, 3)):
        eng.batch_optimize(iters, 0.1, 0.0)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        eng.batch_optimize(iters, 0.1, 0.0)
    ev1.record(stream)
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = eng.launch_count() - l0
    glo, ghi, ginf = eng.batch_download()
    # end to end: upload of the cells from host memory, optimisation, download of the bounds
    t1 = time.perf_counter()
    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(e2e_steps):
        eng.batch_upload(nid, wl.spec, lo, hi, rl, ru, sp0, ns, mode=1)
        eng.batch_optimize(iters, 0.1, 0.0)
        elo, ehi, einf = eng.batch_download()
    e2e_ms = (time.perf_counter() - t1) * 1e3 / e2e_steps
    clocks = sampler.stop()
    assert np.array_equal(elo, glo)
    dims = [int(x) for x in wl.net.dims]
    S = wl.spec.shape[0]
    mac_bwd = dims[-1] * dims[-2] + sum(dims[k] * dims[k + 1] for k in range(len(dims) - 2))
    mac_adj = sum(dims[k] * dims[k + 1] for k in range(len(dims) - 2))
    flops = 2.0 * D * (iters * 2 * S * mac_bwd + (iters - 1) * S * mac_adj)
    peaks = load_peaks()
    peak_tf = peaks["bf16_tflops"] / 2.0
    line = {
        "metric": "alpha-CROWN domains optimised/sec (20 projected-Adam iterations)", "value": D / (ms / 1e3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.path, "data": "synthetic",
        "config": {"workload": "alpha-CROWN optimisation, ReLU MLP 784->9x512->10, box x0+-0.015, 9 spec rows, 20 "
                               "projected-Adam iterations (lr 0.1) on per-neuron alpha, 2048 input-split cells",
                   "domains_per_gpu": D, "iterations": iters,
                   "l2": "coefficient buffers and checkpoints (about 1 GB) exceed the 126 MB L2"},
        "e2e": {"value": D / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": int(lo.nbytes + hi.nbytes + rl.nbytes + ru.nbytes + wl.spec.nbytes),
                "d2h_bytes_per_step": int(glo.nbytes + ghi.nbytes + ginf.nbytes), "ms_per_step": e2e_ms},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": flops / (ms / 1e3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": flops / (ms / 1e3) / 1e12 / peak_tf, "traffic": None, "kernel": "whole optimisation step",
                     "peak_source": f"{peaks['source']} bf16 GEMM / 2 (TF32 operand rate)"},
    }
    if not args.no_cpu_baseline:
        onet = O.Net(wl.net.weights, wl.net.biases).with_spec(wl.spec)
        rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
        ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
        n = 8
        t0 = time.perf_counter()
        for d in range(n):
            opl, opu, _ = O.domain_bounds(onet, lo[d], hi[d], rl2, ru2, sp0[d], 1)
            O.optimize(onet, lo[d], hi[d], opl, opu, sp0[d], O.heuristic_alpha(onet, opl, opu), iters, 0.1, 0.0)
        line["cpu_baseline"] = {"value": n / (time.perf_counter() - t0), "unit": UNIT, "cores": 1, "kind": "port",
                                "sample": f"{n} cells of the same workload, one thread"}
    _emit(line)
    eng.close()


def run_cnn(args, local_rank, kind="cnn"):
    """Secondary workload (--workload cnn): beta-CROWN bound of 1024 BaB domains (8 splits each) of the CNN
    3x32x32 -> conv(16,k4,s2,p1) -> conv(32,k4,s2,p1) -> FC 2048->100 -> FC 100->10, box x0 +- 2/255, 9 spec rows.
    One step = one bound evaluation of the whole batch (interval convolutions forward, transposed convolutions
    backward)."""
    import torch

    from ny_b200 import B200Engine
    from ny_b200 import engine as E
    from ny_b200 import workloads as W
    from oracle import ny_oracle as O  # cpu_baseline leg only (below)

    torch.cuda.set_device(local_rank)
    stream = torch.cuda.current_stream()
    eng = B200Engine(local_rank, stream.cuda_stream)
    eng.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
    wl = W.config_cnn() if kind == "cnn" else W.config_resnet()
    nid = eng.register_network(wl.net)
    pl, pu = eng.ibp_forward_gpu(nid, wl.in_lo, wl.in_hi)
    rl, ru = pl[0].copy(), pu[0].copy()
    D = args.domains if args.domains != D_PER_GPU else (1024 if kind == "cnn" else 256)
    splits, ns = W.draw_domains(wl, rl, ru, D)
    eng.batch_upload(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    for _ in range(max(args.warmup, 3)):
        eng.batch_run()
    torch.cuda.synchronize()
    eng.timing_enable(True)
    eng.timing_reset()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # a step is the bound evaluation AND the check that sends domains with a visible rounding charge through the
    # binary64 contractions once more (what a download would trigger): the bounds are final when the step ends
    ev0.record(stream)
    for _ in range(args.steps):
        eng.batch_run()
        eng.batch_refined()
    ev1.record(stream)
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = eng.launch_count() - l0
    gemm_ms, _ = eng.timing_read("gemm")
    fwd_ms, _ = eng.timing_read("forward")
    bwd_ms, _ = eng.timing_read("backward")
    eng.timing_enable(False)
    glo, ghi, ginf = eng.batch_download()
    refined = eng.batch_refined()
    e2e_steps = max(2, min(args.steps, 5))
    t1 = time.perf_counter()
    for _ in range(e2e_steps):
        elo, ehi, einf = eng.bab_bound_batch(nid, wl.spec, wl.in_lo, wl.in_hi, rl, ru, splits, ns, mode=1)
    e2e_ms = (time.perf_counter() - t1) * 1e3 / e2e_steps
    clocks = sampler.stop()
    assert np.array_equal(elo, glo)
    S = wl.spec.shape[0]
    # algorithmic work per domain: backward MACs per coefficient row through each layer (a convolution costs
    # out_features * in_channels * kh * kw), both bound directions; bytes = every coefficient tile written and
    # read once per layer (fp32)
    macs = 0
    for w in wl.net.weights:
        macs += w.out_features * w.ic * w.kh * w.kw if hasattr(w, "kh") else w.shape[0] * w.shape[1]
    flops = 2.0 * D * 2 * S * macs
    dims = [int(x) for x in wl.net.dims]
    bytes_alg = D * 2 * S * 4.0 * (2 * sum(dims[1:-1]) + dims[0] + dims[-1])
    peaks = load_peaks()
    line = {
        "metric": METRIC, "value": D / (ms / 1e3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64 convolutions, " + args.path + " fully connected", "data": "synthetic",
        "config": {"workload": ("beta-CROWN bound of BaB domains, CNN 3x32x32 conv(16,k4,s2,p1)-conv(32,k4,s2,p1)-FC100-FC10, "
                                "box x0+-2/255, 9 spec rows (both directions), 8 splits/domain, transposed-convolution backward")
                               if kind == "cnn" else
                               ("beta-CROWN bound of BaB domains, residual CNN 3x32x32: conv stem (64,k3) + 4 residual blocks "
                                "(two 3x3 convs, 64 ch) + avgpool + FC 64->10, box x0+-1/255, 9 spec rows, 8 splits/domain"),
                   "domains_per_gpu": D, "feasible_domains": int((ginf == 0).sum()),
                   "domains_sent_to_binary64_rerun": int(refined),
                   "l2": "coefficient ping-pong buffers (2 x 302 MB) exceed the 126 MB L2"},
        "e2e": {"value": D / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": int(splits.nbytes + ns.nbytes + rl.nbytes * 2 + wl.in_lo.nbytes * 2 + wl.spec.nbytes),
                "d2h_bytes_per_step": int(glo.nbytes + ghi.nbytes + ginf.nbytes), "ms_per_step": e2e_ms},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": bytes_alg / (bwd_ms / 1e3) / 1e9 if bwd_ms > 0 else None, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": (bytes_alg / (bwd_ms / 1e3) / 1e9 / peaks["hbm_gbs"]) if bwd_ms > 0 else None,
                     "traffic": None, "kernel": "backward pass (tcgen05 im2col-space contraction + col2im gather for the convolutions)",
                     "peak_source": peaks["source"] + " copy bandwidth",
                     "flops_view": {"achieved_tflops": flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else None},
                     "phase_ms": {"forward": fwd_ms, "backward": bwd_ms, "contraction": gemm_ms}},
    }
    if not args.no_cpu_baseline:
        # the oracle's native convolution (kernel taps, transposed convolution of the coefficient rows) and, for the
        # residual network, identity branches joined in place: the reference's algorithm, not a dense lowering
        onet = O.Net(wl.net.weights, wl.net.biases, skips=getattr(wl.net, "skips", None) or None).with_spec(wl.spec)
        rl2 = np.concatenate([rl, np.full(S, -np.inf, np.float32)])
        ru2 = np.concatenate([ru, np.full(S, np.inf, np.float32)])
        n = 64 if kind == "cnn" else 16
        t0 = time.perf_counter()
        _, _, _, threads = O.bab_bound_batch(onet, wl.in_lo, wl.in_hi, rl2, ru2, splits[:n], ns[:n], 1)
        line["cpu_baseline"] = {"value": n / (time.perf_counter() - t0), "unit": UNIT, "cores": int(threads), "kind": "port",
                                "sample": f"{n} domains of the same workload, native convolutions, all host threads"}
    _emit(line)
    eng.close()



def run_search(args, rank, world, local_rank):
    """Secondary workload (--workload bab-search): the whole branch-and-bound loop (ny_b200/bab.py) on a seeded MLP
    64 -> 4x256 -> 10 with a property it cannot close in the given rounds, so that every round bounds a full batch:
    with --resident 1 (default) the open domain set lives on the device and a round is one call (pop, bound or
    optimise with warm starts, prune, branch, push); with --resident 0 the host loop runs: upload of the children's split
    lists, bound, download, branching choice, child creation on the host.  One step = one search of `rounds` rounds;
    value = domains bounded per second of wall clock, host work included.
    With N > 1 ranks (one process per GPU) every rank bounds its own shard of the frontier, `batch` domains per rank
    and round; the root starts on rank 0, so the first rounds exercise the point-to-point rebalancing (split records
    from one GPU's frontier to another's, device to device; in the host loop also the warm-start slopes when the
    search optimises), whose traffic the line reports."""
    import torch

    from ny_b200 import B200Engine, bab, formats
    from ny_b200 import engine as E
    from ny_b200 import workloads as W

    torch.cuda.set_device(local_rank)
    dist = None
    dev = f"cuda:{local_rank}"
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    eng = B200Engine(local_rank, torch.cuda.current_stream().cuda_stream)
    eng.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
    wl = W.config_mlp_bab(seed=7, hidden=256, depth=4, n_in=64, n_out=10, eps=0.05, n_fix=0)
    nid = eng.register_network(wl.net)
    root, _, _, _ = eng.crown_bounds(nid, wl.spec, wl.in_lo, wl.in_hi)
    s = int(np.argmin(root[0]))
    prop = formats.Property(wl.in_lo, wl.in_hi, [[formats.Atom(-wl.spec[s], float(root[0][s] + 0.5 * abs(root[0][s]) + 0.5))]])
    batch = args.domains if args.domains != D_PER_GPU else 4096
    rounds = 40
    opt_it = args.search_iterations

    resident = bool(args.resident)

    pool = handle = None
    if resident and dist is None and args.search_engines > 1:
        from ny_b200.pool import EnginePool

        pool = EnginePool(local_rank, args.search_engines, lambda e: e.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64))
        handle = pool.register_network(wl.net)

    def search():
        if pool is not None:   # one device frontier per engine of the pool, their rounds overlapping on the GPU
            return bab.verify_resident_pool(pool, handle, wl.net, prop, batch=batch, max_rounds=rounds, branching=1, pgd_restarts=64,
                                            pgd_steps=10, optimize_iterations=opt_it, max_domains=1 << 18,
                                            refinement=args.search_refinement)
        if resident:   # the open domain set stays on the device: one call per round
            return bab.verify_resident(eng, nid, wl.net, prop, batch=batch, max_rounds=rounds, branching=1, pgd_restarts=64,
                                       pgd_steps=10, optimize_iterations=opt_it, max_domains=1 << 18,
                                       refinement=args.search_refinement, dist=dist, dist_device=dev)
        return bab.verify(eng, nid, wl.net, prop, batch=batch, max_rounds=rounds, optimize_iterations=opt_it, branching=1,
                          pgd_restarts=64, pgd_steps=10, dist=dist, dist_device=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        r = search()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = eng.launch_count()
    l0_pool = sum(e.launch_count() for e in pool.engines) if pool is not None else 0
    barrier()
    t0 = time.perf_counter()
    bounded = 0
    moved = {"exchanges": 0, "records_moved": 0, "bytes_moved": 0}
    for _ in range(args.steps):
        r = search()
        bounded += r.domains_bounded          # already the sum over ranks
        for k in moved:
            moved[k] += (r.exchange or {}).get(k, 0)
    barrier()
    dt = time.perf_counter() - t0
    launches = eng.launch_count() - l0
    if pool is not None:
        launches = sum(e.launch_count() for e in pool.engines) - l0_pool
    clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t[0])
        t = torch.tensor([moved["exchanges"], moved["records_moved"], moved["bytes_moved"], launches], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        # every move is counted by its sender and by its receiver; an exchange by every rank
        moved = {"exchanges": int(t[0]) // world, "records_moved": int(t[1]) // 2, "bytes_moved": int(t[2]) // 2}
        launches = int(t[3])
    value = bounded / dt
    if rank == 0:
        _emit({
            "metric": "BaB domains bounded/sec (beta-CROWN), whole search loop", "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dt * 1e3 / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.path, "data": "synthetic",
            "config": {"workload": f"branch and bound on a ReLU MLP 64->4x256->10, box x0+-0.05, one property row, {rounds} rounds "
                                   f"of up to {batch} domains per GPU, intercept branching, "
                                   + (f"{opt_it} optimisation iterations per domain with warm start" if opt_it > 1 else "one bound per domain")
                                   + ", attack and root bound included",
                       "parallelism": f"frontier sharded x{world}",
                       "frontier": (f"device-resident, {args.search_engines} engines on the GPU with a frontier each, up to {batch} domains "
                                    "per engine and round, levelled ring to ring") if pool is not None
                                   else "device-resident (nyb200_frontier_round: pop, bound, prune, branch, push per call)" if resident
                                   else "host (numpy blocks; upload of the children's split lists every round)",
                       "refinement": ("binary64 re-evaluation of the domains whose verdict the rounding charge could change"
                                      if (resident and args.search_refinement == "verdict") else
                                      "binary64 re-evaluation of every domain whose rounding charge is visible at the engine's tolerance"),
                       "timing": "wall clock around the search calls, max over ranks", "status": r.status,
                       "domains_per_search": r.domains_bounded, "open_at_stop": r.open_domains},
            "rebalance": moved if (world > 1 or pool is not None) else None,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None, "ms_per_step": dt * 1e3 / args.steps},
            "gpu_launches": int(launches), "clocks": clocks,
        })
    if pool is not None:
        pool.close()
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


def rebalance_exercise(dist, rank, world, device, n_pre):
    """Untimed proof that the exchange runs on this hardware: rank r holds 64 * (r + 1) synthetic domain records with
    their slopes, the ranks level them point to point over NCCL, and every rank checks that the slopes it ends up
    with still belong to their records."""
    import torch

    from ny_b200 import SPLIT_DTYPE, sharding

    n_local, depth = 64 * (rank + 1), 8
    splits = np.zeros((n_local, depth), SPLIT_DTYPE)
    splits["neuron"] = (rank << 20) + np.arange(n_local)[:, None]
    ns = np.full(n_local, depth, np.int32)
    alpha = np.tile(((rank << 20) + np.arange(n_local)).astype(np.float32)[:, None], (1, n_pre))
    stats = {}
    before = sharding.gather_counts(n_local, dist, device)
    splits, ns, alpha = sharding.exchange_domains(splits, ns, dist, device, alpha=alpha, stats=stats, counts=before)
    after = sharding.gather_counts(len(ns), dist, device)
    intact = bool(np.array_equal(splits["neuron"][:, 0].astype(np.float32), alpha[:, 0]) and np.all(alpha == alpha[:, :1]))
    t = torch.tensor([stats.get("records_moved", 0), stats.get("bytes_moved", 0), 1 if intact else 0], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return {"counts_before": before, "counts_after": after, "records_moved": int(t[0]) // 2, "bytes_moved": int(t[1]) // 2,
            "slopes_travel_with_records": int(t[2]) == world, "transport": "torch.distributed send/recv over NCCL, untimed"}


def run_pgd(args, local_rank, kind="cnn"):
    """Secondary workload (--workload pgd): PGD attack, 100 steps x 1024 restarts, step 0.25 * eps, margin loss,
    on the CNN 3x32x32 conv(16,k4,s2,p1)-conv(32,k4,s2,p1)-FC100-FC10 with box x0 +- 2/255.  One step of this bench =
    one whole attack (101 forward passes, 100 gradients, the binary64 re-validation); value = restart-steps/s."""
    import torch

    from ny_b200 import B200Engine
    from ny_b200 import engine as E
    from ny_b200 import workloads as W
    from oracle import ny_oracle as O  # cpu_baseline leg only (below)

    torch.cuda.set_device(local_rank)
    eng = B200Engine(local_rank, torch.cuda.current_stream().cuda_stream)
    eng.set_path(E.PATH_TF32X3 if args.path == "tf32x3" else E.PATH_F64)
    wl = W.config_cnn() if kind == "cnn" else W.config_resnet()
    nid = eng.register_network(wl.net)
    K, steps = 1024, 100
    g = np.random.Generator(np.random.PCG64(7))
    x0 = (wl.in_lo + g.random((K, len(wl.in_lo)), dtype=np.float32) * (wl.in_hi - wl.in_lo)).astype(np.float32)
    eps = float((wl.in_hi - wl.in_lo).max()) / 2
    for _ in range(2):
        eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, steps, 0.25 * eps)
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = eng.launch_count()
    n = max(2, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(n):
        best, bx, ce = eng.pgd_attack(nid, wl.spec, wl.in_lo, wl.in_hi, x0, steps, 0.25 * eps)
    ms = (time.perf_counter() - t0) * 1e3 / n   # host buffers in and out: this is the end-to-end call
    launches = (eng.launch_count() - l0) // n
    clocks = sampler.stop()
    start = (W.forward(wl.net, x0[:16]) @ wl.spec.astype(np.float64).T).min(axis=1)
    line = {
        "metric": "PGD restart-steps/sec", "value": K * steps / (ms / 1e3), "unit": "restart-steps/s", "n_gpus": 1,
        "steps": n, "warmup": 2, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": args.path, "data": "synthetic",
        "config": {"workload": ("PGD attack, 1024 restarts x 100 steps, step 0.25*eps, margin loss, CNN 3x32x32 "
                                "conv(16,k4,s2,p1)-conv(32,k4,s2,p1)-FC100-FC10, box x0+-2/255") if kind == "cnn" else
                               ("PGD attack, 1024 restarts x 100 steps, step 0.25*eps, margin loss, residual CNN 3x32x32 "
                                "(conv stem 64,k3 + 4 residual blocks + avgpool + FC 64->10), box x0+-1/255"),
                   "restarts": K, "pgd_steps": steps, "timing": "wall clock around the host-buffer C-ABI call",
                   "mean_objective_start": float(start.mean()), "mean_objective_end": float(best.mean()),
                   "counterexample": int(ce)},
        "e2e": {"value": K * steps / (ms / 1e3), "unit": "restart-steps/s", "h2d_bytes_per_step": int(x0.nbytes + wl.in_lo.nbytes * 2 + wl.spec.nbytes),
                "d2h_bytes_per_step": int(best.nbytes + bx.nbytes), "ms_per_step": ms},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if not args.no_cpu_baseline and kind == "cnn":
        ws, bs = O.lower_network(wl.net.weights, wl.net.biases)
        kk, ss = 64, 10
        t0 = time.perf_counter()
        O.pgd_attack(ws, bs, wl.spec, wl.in_lo, wl.in_hi, x0[:kk], ss, 0.25 * eps)
        line["cpu_baseline"] = {"value": kk * ss / (time.perf_counter() - t0), "unit": "restart-steps/s", "cores": "numpy BLAS threads",
                                "kind": "port", "sample": f"{kk} restarts x {ss} steps on the dense lowering"}
    _emit(line)
    eng.close()


def eng_path_name(eng):
    return getattr(eng, "_path_name", "tf32x3")


def main():
    # Libraries (NCCL's version banner, for one) may write to stdout; the contract is ONE JSON line there.
    # Keep the real stdout aside, send everything else to stderr, and print the result line on the real one.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    global _emit
    _emit = lambda obj: (real_stdout.write(json.dumps(obj) + "\n"), real_stdout.flush())
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default=os.environ.get("NYB200_PATH", "tf32x3"), choices=["f64", "tf32x3"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the 32-domain oracle comparison after the timed region")
    ap.add_argument("--no-peak", action="store_true", help="skip the TF32 GEMM peak measurement (profiling runs)")
    ap.add_argument("--blocks", type=int, default=30, help="back-to-back repetitions of the timed --steps block")
    ap.add_argument("--ref-sample", type=int, default=D_PER_GPU, help="domains per step of the reference arm")
    ap.add_argument("--cpu-sample", type=int, default=D_PER_GPU, help="domains of the cpu_baseline leg")
    ap.add_argument("--fusion", type=int, default=1, help="0: one launch per layer; 1: fused backward chain (default)")
    ap.add_argument("--workload", default="bab", choices=["bab", "alpha-crown", "cnn", "resnet", "pgd", "pgd-resnet", "bab-search"],
                    help="bab: the headline beta-CROWN batch (default); alpha-crown: the alpha optimisation case; "
                         "cnn: the convolutional case (both 1 GPU)")
    ap.add_argument("--resident", type=int, default=1,
                    help="bab-search on one GPU: 1 keeps the frontier on the device (default), 0 runs the host loop")
    ap.add_argument("--search-engines", type=int, default=2,
                    help="bab-search on one GPU: engines (device frontiers) sharing the search, their rounds overlapping (1: a single frontier)")
    ap.add_argument("--search-refinement", default="verdict", choices=["verdict", "parity"],
                    help="bab-search on the device frontier: which domains are re-evaluated in binary64 (see bab.verify_resident)")
    ap.add_argument("--search-iterations", type=int, default=0,
                    help="bab-search: optimisation iterations per domain (0 = one bound per domain, the reference's throughput default)")
    ap.add_argument("--in-flight", type=int, default=3,
                    help="resident batches in flight per GPU (one engine and stream each; 1: a single batch, as the kernel profiles use)")
    ap.add_argument("--reserve-sms", type=int, default=-1,
                    help="SMs the persistent kernels leave to the min-reduce on the side stream (-1: 2 when N > 1, else 0)")
    ap.add_argument("--domains", type=int, default=D_PER_GPU, help="domains per GPU (profiling runs use a smaller batch)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "alpha-crown":
        if rank == 0:
            run_alpha_crown(args, 0, 1, local_rank)
        return
    if args.workload == "bab-search":
        run_search(args, rank, world, local_rank)
        return
    if args.workload in ("pgd", "pgd-resnet"):
        if rank == 0:
            run_pgd(args, local_rank, "cnn" if args.workload == "pgd" else "resnet")
        return
    if args.workload in ("cnn", "resnet"):
        if rank == 0:
            run_cnn(args, local_rank, args.workload)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
