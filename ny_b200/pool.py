"""Several batches in flight on one GPU.

Batches of BaB domains are independent, and one batch alone leaves the GPU partly idle: its interval pass is a chain
of short, latency-bound launches, its transfers and the host side of the call run while no kernel does.  An
EnginePool holds `n` engines on the same device, each with a stream, a workspace and a host thread of its own, and
hands batches to them in turn: one batch's interval pass overlaps another's tensor-bound backward chain, one's
host-to-device copy another's kernels.  Results are bit-identical to a single engine's (every batch runs the same
kernels on its own memory).  The reference's counterpart is one engine handle per worker thread
(crates/ny-core/src/gemm.rs:568-578 caches device weights per handle).
"""
from __future__ import annotations

import threading

from .engine import B200Engine


class EnginePool:
    def __init__(self, device: int = 0, n: int = 3, configure=None):
        """configure(engine): optional per-engine set-up (path, tolerances, fusion)."""
        if n < 1:
            raise ValueError("at least one engine")
        self.engines = []
        for _ in range(n):
            e = B200Engine(device)
            e.use_own_stream()
            if n > 1:
                e.set_launch_overlap(False)   # early-scheduled CTAs of one engine would hold SMs another engine can use
            if configure is not None:
                configure(e)
            self.engines.append(e)
        self._nets = []

    def __len__(self):
        return len(self.engines)

    def register_network(self, net) -> int:
        """Registers the network on every engine; returns the pool's handle for it."""
        self._nets.append([e.register_network(net) for e in self.engines])
        return len(self._nets) - 1

    def bound_batches(self, net: int, batches):
        """batches: iterable of argument tuples for B200Engine.bab_bound_batch after the network id, i.e.
        (spec, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits[, mode[, alpha]]).  Batch k runs on engine k mod n, each
        engine's batches in order on its own thread.  Returns the results in the order of `batches`.  An engine's
        error is raised after all threads have ended."""
        batches = list(batches)
        out = [None] * len(batches)
        errors = []
        n = len(self.engines)

        def work(i):
            e, nid = self.engines[i], self._nets[net][i]
            try:
                for k in range(i, len(batches), n):
                    out[k] = e.bab_bound_batch(nid, *batches[k])
            except Exception as exc:  # noqa: BLE001 - handed to the caller below
                errors.append(exc)

        threads = [threading.Thread(target=work, args=(i,)) for i in range(min(n, len(batches)))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        return out

    def close(self):
        for e in self.engines:
            e.close()
        self.engines = []
