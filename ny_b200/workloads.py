"""Seeded synthetic workloads with the shapes of the benchmark configurations.

They stand in for ACAS-Xu / MNIST / CIFAR style verification instances (no benchmark-suite item
is used): random He-initialised networks, a random nominal input, an L-inf box, specification
rows y_c - y_j, and BaB domains that fix seeded unstable neurons.  Everything is derived from
numpy's PCG64 streams so the same arrays are produced on every machine.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .engine import SPLIT_DTYPE, Conv2d, Network


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def make_mlp(dims, seed: int) -> Network:
    """Weights N(0, 2/fan_in), biases N(0, 0.01) (variances), fp32."""
    g = _rng(seed)
    ws, bs = [], []
    for k in range(len(dims) - 1):
        fan_in = dims[k]
        ws.append((g.standard_normal((dims[k + 1], dims[k])) * np.sqrt(2.0 / fan_in)).astype(np.float32))
        bs.append((g.standard_normal(dims[k + 1]) * 0.1).astype(np.float32))
    return Network(ws, bs)


def forward(net: Network, x) -> np.ndarray:
    z = np.asarray(x, np.float64)
    one = z.ndim == 1
    if one:
        z = z[None, :]
    posts = []
    for k in range(len(net.weights)):
        z = net.layer_forward(k, z)
        if k in net.skips:
            z = z + posts[net.skips[k]]
        if k + 1 < len(net.weights):
            z = np.maximum(z, 0.0)
        posts.append(z)
    return z[0] if one else z


def margin_spec(n_out: int, c: int) -> np.ndarray:
    """Rows e_c - e_j for every j != c."""
    rows = []
    for j in range(n_out):
        if j == c:
            continue
        r = np.zeros(n_out, np.float32)
        r[c] = 1.0
        r[j] = -1.0
        rows.append(r)
    return np.stack(rows)


@dataclass
class Workload:
    name: str
    net: Network
    x0: np.ndarray
    in_lo: np.ndarray
    in_hi: np.ndarray
    spec: np.ndarray
    n_fix: int = 0
    seed: int = 0
    meta: dict = field(default_factory=dict)


def config_mlp_small(seed: int = 1) -> Workload:
    """MLP 5 -> 6x50 -> 5, box x0 +- 0.05 with x0 ~ U(-1,1)^5, 4 rows y0 - yj."""
    net = make_mlp([5] + [50] * 6 + [5], seed)
    g = _rng(seed + 1000)
    x0 = g.uniform(-1, 1, 5).astype(np.float32)
    return Workload("mlp_5_6x50_5", net, x0, x0 - np.float32(0.05), x0 + np.float32(0.05), margin_spec(5, 0), 0, seed)


def config_mlp_bab(seed: int = 2, hidden: int = 256, depth: int = 8, n_in: int = 784, n_out: int = 10,
                   eps: float = 0.02, n_fix: int = 8) -> Workload:
    """MLP 784 -> 8x256 -> 10, box x0 +- 0.02 clipped to [0,1], 9 rows y_c - y_j (c = argmax f(x0))."""
    net = make_mlp([n_in] + [hidden] * depth + [n_out], seed)
    g = _rng(seed + 1000)
    x0 = g.uniform(0, 1, n_in).astype(np.float32)
    lo = np.clip(x0 - np.float32(eps), 0, 1).astype(np.float32)
    hi = np.clip(x0 + np.float32(eps), 0, 1).astype(np.float32)
    c = int(np.argmax(forward(net, x0)))
    return Workload(f"mlp_{n_in}_{depth}x{hidden}_{n_out}", net, x0, lo, hi, margin_spec(n_out, c), n_fix, seed,
                    {"eps": eps, "label": c})


def make_cnn(seed: int, in_chw=(3, 32, 32), convs=((16, 4, 2, 1), (32, 4, 2, 1)), fcs=(100, 10)) -> Network:
    """Conv layers (out_channels, kernel, stride, pad) then fully connected widths; He-initialised fp32
    (weights N(0, 2/fan_in), biases N(0, 0.01))."""
    g = _rng(seed)
    c, h, w = in_chw
    layers = []
    for (oc, k, s, p) in convs:
        fan_in = c * k * k
        wt = (g.standard_normal((oc, c, k, k)) * np.sqrt(2.0 / fan_in)).astype(np.float32)
        b = (g.standard_normal(oc) * 0.1).astype(np.float32)
        conv = Conv2d(wt, b, (s, s), (p, p), (h, w))
        layers.append(conv)
        c, h, w = oc, conv.oh, conv.ow
    n = c * h * w
    ws, bs = list(layers), [None] * len(layers)
    for width in fcs:
        ws.append((g.standard_normal((width, n)) * np.sqrt(2.0 / n)).astype(np.float32))
        bs.append((g.standard_normal(width) * 0.1).astype(np.float32))
        n = width
    return Network(ws, bs)


def make_resnet(seed: int, in_chw=(3, 32, 32), channels: int = 64, blocks: int = 4, n_out: int = 10) -> Network:
    """conv stem (channels, k3, s1, p1) + `blocks` residual blocks (two 3x3 convs, ReLU, identity skip) + global
    average pool + FC channels -> n_out, He-initialised.  The pool and the FC are one Linear layer (the pool folded
    into its weights: W[i][c] / (H*W) over the pixels, exact in fp32 for power-of-two H*W)."""
    g = _rng(seed)
    c, h, w = in_chw
    layers, skips = [], {}
    def conv(ci, co):
        wt = (g.standard_normal((co, ci, 3, 3)) * np.sqrt(2.0 / (ci * 9))).astype(np.float32)
        b = (g.standard_normal(co) * 0.1).astype(np.float32)
        return Conv2d(wt, b, (1, 1), (1, 1), (h, w))
    layers.append(conv(c, channels))
    for _ in range(blocks):
        layers.append(conv(channels, channels))
        layers.append(conv(channels, channels))
        skips[len(layers) - 1] = len(layers) - 3
    fc = (g.standard_normal((n_out, channels)) * np.sqrt(2.0 / channels)).astype(np.float32)
    fb = (g.standard_normal(n_out) * 0.1).astype(np.float32)
    pooled = np.repeat(fc / np.float32(h * w), h * w, axis=1).astype(np.float32)
    return Network(layers + [pooled], [None] * len(layers) + [fb], skips)


def config_resnet(seed: int = 5, eps: float = 1.0 / 255.0, n_fix: int = 8, **kw) -> Workload:
    """Residual CNN on 3x32x32 (stem + 4 blocks of two 3x3 convs, 64 channels, avgpool, FC 64->10), box x0 +- 1/255
    clipped to [0,1], 9 margin rows."""
    net = make_resnet(seed, **kw)
    g = _rng(seed + 1000)
    n_in = int(net.dims[0])
    x0 = g.uniform(0, 1, n_in).astype(np.float32)
    lo = np.clip(x0 - np.float32(eps), 0, 1).astype(np.float32)
    hi = np.clip(x0 + np.float32(eps), 0, 1).astype(np.float32)
    c = int(np.argmax(forward(net, x0)))
    return Workload("resnet_" + "_".join(str(int(d)) for d in net.dims[:3]), net, x0, lo, hi,
                    margin_spec(int(net.dims[-1]), c), n_fix, seed, {"eps": eps, "label": c})


def config_cnn(seed: int = 3, eps: float = 2.0 / 255.0, n_fix: int = 8, **kw) -> Workload:
    """CNN on 3x32x32: conv(16,k4,s2,p1)-ReLU, conv(32,k4,s2,p1)-ReLU, FC 2048->100-ReLU, FC 100->10; box
    x0 +- 2/255 with x0 ~ U(0,1) clipped to [0,1]; 9 margin rows."""
    net = make_cnn(seed, **kw)
    g = _rng(seed + 1000)
    n_in = int(net.dims[0])
    x0 = g.uniform(0, 1, n_in).astype(np.float32)
    lo = np.clip(x0 - np.float32(eps), 0, 1).astype(np.float32)
    hi = np.clip(x0 + np.float32(eps), 0, 1).astype(np.float32)
    c = int(np.argmax(forward(net, x0)))
    n_out = int(net.dims[-1])
    return Workload("cnn_" + "_".join(str(int(d)) for d in net.dims), net, x0, lo, hi, margin_spec(n_out, c), n_fix, seed,
                    {"eps": eps, "label": c})


def config_alpha_crown(seed: int = 4, hidden: int = 512, depth: int = 9, n_in: int = 784, n_out: int = 10,
                       eps: float = 0.015) -> Workload:
    """MLP 784 -> 9x512 -> 10, box x0 +- 0.015 clipped to [0,1], 9 margin rows: the alpha-CROWN optimisation case."""
    wl = config_mlp_bab(seed=seed, hidden=hidden, depth=depth, n_in=n_in, n_out=n_out, eps=eps, n_fix=0)
    wl.name = f"alpha_crown_mlp_{n_in}_{depth}x{hidden}_{n_out}"
    return wl


def draw_input_cells(wl: Workload, n_bits: int, first: int = 0, count: int | None = None):
    """Input-split BaB domains: the root box halved along n_bits seeded coordinates gives 2^n_bits cells;
    returns the boxes (lo [D, n_in], hi [D, n_in]) of cells first .. first+count-1 (cell index bit b selects the
    lower or upper half of coordinate dims[b])."""
    g = _rng(wl.seed * 7919 + 17)
    n_in = wl.in_lo.shape[0]
    wide = np.flatnonzero(wl.in_hi > wl.in_lo)
    dims = g.choice(wide, size=n_bits, replace=False)
    total = 1 << n_bits
    count = total - first if count is None else count
    idx = (np.arange(first, first + count) % total).astype(np.int64)
    lo = np.repeat(wl.in_lo[None, :], count, axis=0).astype(np.float32)
    hi = np.repeat(wl.in_hi[None, :], count, axis=0).astype(np.float32)
    mid = ((wl.in_lo.astype(np.float64) + wl.in_hi.astype(np.float64)) * 0.5).astype(np.float32)
    for b, j in enumerate(dims):
        upper = ((idx >> b) & 1).astype(bool)
        lo[upper, j] = mid[j]
        hi[~upper, j] = mid[j]
    return lo, hi


def draw_domains(wl: Workload, root_lo: np.ndarray, root_hi: np.ndarray, D: int, first: int = 0):
    """D BaB domains: domain d fixes n_fix neurons drawn without replacement (stream seed+d) from the
    root-unstable set, sign ~ Bernoulli(1/2), beta ~ U(0,1).  Returns (splits [D, n_fix], n_splits [D]).
    `first` offsets the domain index so that ranks can draw disjoint shards of one global batch."""
    net = wl.net
    n_hidden = int(net.dims[1:-1].sum())
    unstable = np.flatnonzero((root_lo[:n_hidden] < 0) & (root_hi[:n_hidden] > 0))
    offs = np.concatenate([[0], np.cumsum(net.dims[1:-1])])
    n_fix = min(wl.n_fix, len(unstable))
    splits = np.zeros((D, max(n_fix, 1)), SPLIT_DTYPE)
    n_splits = np.full(D, n_fix, np.int32)
    for d in range(D):
        g = _rng(wl.seed * 1_000_003 + first + d)
        pick = g.choice(unstable, size=n_fix, replace=False) if n_fix else np.zeros(0, np.int64)
        sign = np.where(g.random(n_fix) < 0.5, 1, -1)
        beta = g.random(n_fix).astype(np.float32)
        relu = np.searchsorted(offs, pick, side="right") - 1
        splits["relu"][d, :n_fix] = relu
        splits["neuron"][d, :n_fix] = pick - offs[relu]
        splits["sign"][d, :n_fix] = sign
        splits["beta"][d, :n_fix] = beta
    return splits, n_splits


def sample_min_margin(wl: Workload, n_samples: int, seed: int, splits=None, chunk: int = 8192) -> np.ndarray:
    """Empirical minimum of the specification rows over seeded concrete points of the box that also
    satisfy the domain's split constraints (points violating a split are discarded).  Used by the
    soundness check: a valid lower bound must not exceed it."""
    g = _rng(seed)
    net = wl.net
    S = wl.spec.shape[0]
    best = np.full(S, np.inf)
    offs = np.concatenate([[0], np.cumsum(net.dims[1:-1])])
    done = 0
    while done < n_samples:
        n = min(chunk, n_samples - done)
        done += n
        x = wl.in_lo.astype(np.float64) + g.random((n, len(wl.in_lo))) * (wl.in_hi.astype(np.float64) - wl.in_lo)
        z = x
        ok = np.ones(n, bool)
        posts = []
        for k in range(len(net.weights)):
            z = net.layer_forward(k, z)
            if k in net.skips:
                z = z + posts[net.skips[k]]
            posts.append(None)
            if k + 1 < len(net.weights):
                if splits is not None:
                    for s in splits:
                        if s["relu"] == k:
                            v = z[:, s["neuron"]]
                            ok &= (v >= 0) if s["sign"] > 0 else (v <= 0)
                z = np.maximum(z, 0.0)
            posts[k] = z
        m = z @ wl.spec.astype(np.float64).T
        if ok.any():
            best = np.minimum(best, m[ok].min(axis=0))
    return best
