"""ctypes binding of the CPU oracle (libny_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline legs.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libny_oracle.so")


class _Net(C.Structure):
    _fields_ = [
        ("n_linear", C.c_int32),
        ("dims", C.POINTER(C.c_int32)),
        ("wflat", C.POINTER(C.c_float)),
        ("bflat", C.POINTER(C.c_float)),
        ("has_bias", C.POINTER(C.c_int32)),
        ("relu_after", C.POINTER(C.c_int32)),
        ("conv_geom", C.POINTER(C.c_int32)),
        ("skip_from", C.POINTER(C.c_int32)),
    ]


SPLIT_DTYPE = np.dtype([("relu", "<i4"), ("neuron", "<i4"), ("sign", "<i4"), ("beta", "<f4")])


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file; returns the library path."""
    src = os.path.join(_HERE, "ny_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        fp = C.POINTER(C.c_float)
        ip = C.POINTER(C.c_int32)
        np_ = C.POINTER(_Net)
        L.nyo_next_up_f32.restype = C.c_float
        L.nyo_next_up_f32.argtypes = [C.c_float]
        L.nyo_next_down_f32.restype = C.c_float
        L.nyo_next_down_f32.argtypes = [C.c_float]
        L.nyo_certified_affine_sum.restype = C.c_double
        L.nyo_certified_affine_sum.argtypes = [C.c_float, fp, fp, C.c_int, C.c_int]
        L.nyo_ibp_forward.argtypes = [np_, fp, fp, fp, fp]
        L.nyo_crown.argtypes = [np_, fp, fp, fp, fp, fp, fp]
        L.nyo_crown_split.argtypes = [np_, fp, fp, C.c_void_p, C.c_int, fp, fp, fp, fp]
        L.nyo_beta_crown_bound.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, fp, fp]
        L.nyo_domain_bounds.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, C.c_int, fp, fp]
        L.nyo_bab_bound_batch.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, ip, C.c_int, C.c_int, C.c_int,
                                          fp, fp, ip, C.c_int]
        dp = C.POINTER(C.c_double)
        L.nyo_joint_gradient.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, dp, fp, fp]
        L.nyo_optimize.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, C.c_int, C.c_float, C.c_float,
                                   C.c_float, C.c_float, fp, fp]
        L.nyo_optimize_objective.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, C.c_int, C.c_float, C.c_float,
                                             C.c_float, C.c_float, C.c_int, fp, fp]
        L.nyo_joint_gradient_rows.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, dp, fp, fp, C.c_int]
        L.nyo_select_largest_width.argtypes = [np_, fp, fp, C.c_void_p, C.c_int, ip, ip, fp]
        L.nyo_beta_crown_bound_dual.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, fp, fp, fp]
        L.nyo_upper_gradient.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, fp, dp, fp]
        L.nyo_optimize_dual.argtypes = [np_, fp, fp, fp, fp, C.c_void_p, C.c_int, fp, C.c_int, C.c_float, C.c_float,
                                        C.c_float, C.c_float, C.c_int, fp, fp, fp]
        L.nyo_set_error_channel.argtypes = [C.c_int]
        L.nyo_set_error_channel.restype = None
        L.nyo_select_intercept.argtypes = [np_, fp, fp, C.c_void_p, C.c_int, ip, ip, fp]
        L.nyo_domain_verified.argtypes = [C.c_float, C.c_float, C.c_float]
        L.nyo_domain_violated.argtypes = [C.c_float, C.c_float, C.c_float]
        _lib = L
    return _lib


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


def _ip(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32)) if a is not None else None


class Net:
    """Sequential ReLU network: weights[k] is a dense [out, in] matrix (row-major) or a Conv2d description (any
    object with weight [oc, ic, kh, kw], sh, sw, ph, pw, ih, iw, oh, ow attributes, e.g. ny_b200.engine.Conv2d);
    biases[k] is [out] ([oc] for a convolution) or None.  Convolutions are evaluated natively (kernel taps), not
    through a dense lowering."""

    def __init__(self, weights, biases=None, relu_after=None, skips=None):
        """skips: optional {k: j}: the post-activation output of layer j joins layer k's output before its ReLU."""
        L = len(weights)
        self.skips = dict(skips or {})
        self._skip = None
        if self.skips:
            self._skip = np.full(L, -1, np.int32)
            for k, j in self.skips.items():
                self._skip[k] = j
        self.weights = [w if hasattr(w, "kh") else np.ascontiguousarray(w, dtype=np.float32) for w in weights]
        self.relu_after = None if relu_after is None else np.ascontiguousarray(relu_after, np.int32)
        biases = biases if biases is not None else [None] * L
        biases = [(w.bias if hasattr(w, "kh") and b is None else b) for w, b in zip(self.weights, biases)]
        self.biases = [None if b is None else np.ascontiguousarray(b, dtype=np.float32) for b in biases]
        dims, flat, geom = [], [], np.zeros((L, 12), np.int32)
        for k, w in enumerate(self.weights):
            if hasattr(w, "kh"):
                if k == 0:
                    dims.append(w.ic * w.ih * w.iw)
                dims.append(w.oc * w.oh * w.ow)
                geom[k] = (w.ic, w.ih, w.iw, w.oc, w.oh, w.ow, w.kh, w.kw, w.sh, w.sw, w.ph, w.pw)
                flat.append(np.ascontiguousarray(w.weight, np.float32).ravel())
            else:
                if k == 0:
                    dims.append(w.shape[1])
                dims.append(w.shape[0])
                flat.append(w.ravel())
        self.dims = np.array(dims, dtype=np.int32)
        self._w = np.concatenate(flat).astype(np.float32)
        bl = [b for b in self.biases if b is not None]
        self._b = np.concatenate(bl).astype(np.float32) if bl else np.zeros(1, np.float32)
        self._hb = np.array([0 if b is None else 1 for b in self.biases], dtype=np.int32)
        self._geom = np.ascontiguousarray(geom) if geom.any() else None
        self.c = _Net(L, _ip(self.dims), _fp(self._w), _fp(self._b), _ip(self._hb), _ip(self.relu_after), _ip(self._geom), _ip(self._skip))

    @property
    def n_pre(self) -> int:
        return int(self.dims[1:].sum())

    def with_spec(self, spec) -> "Net":
        """Append the specification rows as a bias-free Linear layer, the way ny's CLI does
        (ny-cli commands/beta_crown/constraint_eval.rs:80-91)."""
        L = len(self.weights)
        ra = [1] * (L - 1) + [0, 0] if self.relu_after is None else list(self.relu_after[: L - 1]) + [0, 0]
        return Net(self.weights + [np.asarray(spec, np.float32)], self.biases + [None], ra, self.skips)

    def forward(self, x):
        """Concrete forward pass in binary64 (rows of x are points)."""
        one = np.asarray(x).ndim == 1
        z = np.asarray(x, np.float64).reshape(1, -1) if one else np.asarray(x, np.float64)
        posts = []
        for k, w in enumerate(self.weights):
            if hasattr(w, "kh"):
                z = w.apply(z)   # the description's own concrete convolution, its bias included
                if w.bias is None and self.biases[k] is not None:
                    z = z + np.repeat(self.biases[k].astype(np.float64), w.oh * w.ow)[None, :]
            else:
                z = z @ w.astype(np.float64).T
                if self.biases[k] is not None:
                    z = z + self.biases[k].astype(np.float64)
            if k in self.skips:
                z = z + posts[self.skips[k]]
            if k + 1 < len(self.weights) and (self.relu_after is None or self.relu_after[k]):
                z = np.maximum(z, 0.0)
            posts.append(z)
        return z[0] if one else z


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def conv2d_dense(weight, bias, stride, pad, in_hw):
    """The linear map of a Conv2d layer as a dense matrix over NCHW-flattened tensors.

    weight [oc, ic, kh, kw], bias [oc] or None, dilation 1, one group.  Returns (W [oc*oh*ow, ic*ih*iw],
    b [oc*oh*ow] or None) with W[(co,oy,ox), (ci,iy,ix)] = weight[co,ci,ky,kx] for iy = oy*sh - ph + ky,
    ix = ox*sw - pw + kx inside the input.  With this matrix the interval pass W+ l + W- u + b is the
    reference's interval convolution (layers/convolution/conv2d/bound.rs:86-268) and the CROWN backward
    A * W is its transposed convolution (conv2d/bound.rs:601-900, conv2d/ops_transpose_gemm.rs): the same
    products, summed per output element; the bias is expanded per channel (GpuCrownLayer::Conv2d::bias_expanded,
    ny-core/src/gemm.rs:1566)."""
    weight = np.asarray(weight, np.float32)
    oc, ic, kh, kw = weight.shape
    sh, sw = stride
    ph, pw = pad
    ih, iw = in_hw
    if sh <= 0 or sw <= 0 or kh <= 0 or kw <= 0:
        raise ValueError("conv2d: zero stride or kernel")
    if ih + 2 * ph < kh or iw + 2 * pw < kw:
        raise ValueError("conv2d: kernel larger than the padded input")
    oh, ow = (ih + 2 * ph - kh) // sh + 1, (iw + 2 * pw - kw) // sw + 1
    W = np.zeros((oc, oh, ow, ic, ih, iw), np.float32)
    for oy in range(oh):
        for ky in range(kh):
            iy = oy * sh - ph + ky
            if iy < 0 or iy >= ih:
                continue
            for ox in range(ow):
                for kx in range(kw):
                    ix = ox * sw - pw + kx
                    if ix < 0 or ix >= iw:
                        continue
                    W[:, oy, ox, :, iy, ix] = weight[:, :, ky, kx]
    b = None if bias is None else np.repeat(np.asarray(bias, np.float32), oh * ow)
    return W.reshape(oc * oh * ow, ic * ih * iw), b


def lower_residual(ws, bs, skips):
    """Sequential (dense) form of a network with identity skips {k: j} (relu(pre_j) added to layer k's output):
    the skipped activation is carried alongside as extra neurons through identity rows - relu is the identity on
    them, their interval being non-negative - and joins through an identity block of layer k:
        layers j+1 .. k-1:  [[W, 0], [0, I]],   layer k:  [W | I].
    The bounds of the original neurons are those of the leading dims of every layer.  Returns
    (weights, biases, widths) where widths[k] is the number of original neurons of layer k."""
    ws = [np.asarray(w, np.float32) for w in ws]
    out_w, out_b, widths = [], [], []
    carry = None  # (layer that consumes the carried activation, its width)
    for k, w in enumerate(ws):
        n_out, n_in = w.shape
        b = np.zeros(n_out, np.float32) if bs[k] is None else np.asarray(bs[k], np.float32)
        if carry is not None and carry[0] == k:      # the identity branch joins: [W | I]
            w = np.concatenate([w, np.eye(carry[1], dtype=np.float32)], axis=1)
            carry = None
        elif carry is not None:                      # pass the carried activation through: [[W, 0], [0, I]]
            c = carry[1]
            w = np.block([[w, np.zeros((n_out, c), np.float32)], [np.zeros((c, n_in), np.float32), np.eye(c, dtype=np.float32)]])
            b = np.concatenate([b, np.zeros(c, np.float32)])
        opens = [kk for kk, j in skips.items() if j == k - 1]
        if opens:                                     # this layer's input is skipped forward: duplicate it
            assert carry is None and len(opens) == 1 and w.shape[1] == n_in, "nested or overlapping skips"
            w = np.concatenate([w, np.eye(n_in, dtype=np.float32)], axis=0)
            b = np.concatenate([b, np.zeros(n_in, np.float32)])
            carry = (opens[0], n_in)
        out_w.append(np.ascontiguousarray(w, np.float32))
        out_b.append(b)
        widths.append(n_out)
    return out_w, out_b, widths


def lower_network(layers, biases):
    """Dense (weights, biases) lists for a sequential network whose entries are matrices or conv layer
    descriptions (objects with weight, bias, sh, sw, ph, pw, ih, iw attributes)."""
    ws, bs = [], []
    for w, b in zip(layers, biases):
        if hasattr(w, "kh"):
            dw, db = conv2d_dense(w.weight, w.bias, (w.sh, w.sw), (w.ph, w.pw), (w.ih, w.iw))
            ws.append(dw)
            bs.append(db)
        else:
            ws.append(w)
            bs.append(b)
    return ws, bs


def ibp_forward(net: Net, lo, hi):
    lo, hi = _f32(lo), _f32(hi)
    pl = np.empty(net.n_pre, np.float32)
    pu = np.empty(net.n_pre, np.float32)
    lib().nyo_ibp_forward(C.byref(net.c), _fp(lo), _fp(hi), _fp(pl), _fp(pu))
    return pl, pu


def crown(net: Net, lo, hi, want_intermediate=False, error_channel=True):
    """Plain CROWN with CROWN-IBP intermediates.  error_channel=False leaves the reference's certified
    per-coefficient error matrices out of the result (see nyo_set_error_channel)."""
    lo, hi = _f32(lo), _f32(hi)
    lib().nyo_set_error_channel(1 if error_channel else 0)
    try:
        return _crown(net, lo, hi, want_intermediate)
    finally:
        lib().nyo_set_error_channel(1)


def _crown(net: Net, lo, hi, want_intermediate):
    n = int(net.dims[-1])
    ol, ou = np.empty(n, np.float32), np.empty(n, np.float32)
    il = np.empty(net.n_pre, np.float32) if want_intermediate else None
    iu = np.empty(net.n_pre, np.float32) if want_intermediate else None
    lib().nyo_crown(C.byref(net.c), _fp(lo), _fp(hi), _fp(ol), _fp(ou), _fp(il), _fp(iu))
    return (ol, ou, il, iu) if want_intermediate else (ol, ou)


def crown_split(net: Net, lo, hi, splits: np.ndarray, error_channel=False):
    """Plain CROWN with CROWN-IBP intermediates for a ReLU-split domain: (lower, upper, inter_lo, inter_hi, infeasible)."""
    lo, hi = _f32(lo), _f32(hi)
    n = int(net.dims[-1])
    ol, ou = np.empty(n, np.float32), np.empty(n, np.float32)
    il, iu = np.empty(net.n_pre, np.float32), np.empty(net.n_pre, np.float32)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    lib().nyo_set_error_channel(1 if error_channel else 0)
    try:
        st = lib().nyo_crown_split(C.byref(net.c), _fp(lo), _fp(hi), splits.ctypes.data, len(splits), _fp(ol), _fp(ou), _fp(il), _fp(iu))
    finally:
        lib().nyo_set_error_channel(1)
    if st < 0:
        raise ValueError("nyo_crown_split: unsupported network")
    return ol, ou, il, iu, bool(st)


def make_splits(items) -> np.ndarray:
    """items: iterable of (relu, neuron, sign, beta)."""
    a = np.zeros(len(items), SPLIT_DTYPE)
    for i, (r, j, s, b) in enumerate(items):
        a[i] = (r, j, s, b)
    return a


def beta_crown_bound(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha=None):
    lo, hi, pre_lo, pre_hi = _f32(lo), _f32(hi), _f32(pre_lo), _f32(pre_hi)
    alpha = None if alpha is None else _f32(alpha)
    n = int(net.dims[-1])
    ol, ou = np.empty(n, np.float32), np.empty(n, np.float32)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    lib().nyo_beta_crown_bound(C.byref(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi),
                               splits.ctypes.data, len(splits), _fp(alpha), _fp(ol), _fp(ou))
    return ol, ou


def domain_bounds(net: Net, lo, hi, inh_lo, inh_hi, splits: np.ndarray, mode: int):
    lo, hi, inh_lo, inh_hi = _f32(lo), _f32(hi), _f32(inh_lo), _f32(inh_hi)
    pl, pu = np.empty(net.n_pre, np.float32), np.empty(net.n_pre, np.float32)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    inf = lib().nyo_domain_bounds(C.byref(net.c), _fp(lo), _fp(hi), _fp(inh_lo), _fp(inh_hi),
                                  splits.ctypes.data, len(splits), mode, _fp(pl), _fp(pu))
    return pl, pu, bool(inf)


def bab_bound_batch(net: Net, lo, hi, inh_lo, inh_hi, splits: np.ndarray, n_splits, mode: int, n_threads: int = 0):
    """splits: [D, max_splits] structured array; returns (lower [D,S], upper [D,S], infeasible [D], threads)."""
    lo, hi, inh_lo, inh_hi = _f32(lo), _f32(hi), _f32(inh_lo), _f32(inh_hi)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    D, M = splits.shape
    n_splits = np.ascontiguousarray(n_splits, np.int32)
    S = int(net.dims[-1])
    ol, ou = np.empty((D, S), np.float32), np.empty((D, S), np.float32)
    inf = np.zeros(D, np.int32)
    used = lib().nyo_bab_bound_batch(C.byref(net.c), _fp(lo), _fp(hi), _fp(inh_lo), _fp(inh_hi),
                                     splits.ctypes.data, _ip(n_splits), M, D, mode, _fp(ol), _fp(ou), _ip(inf),
                                     n_threads)
    return ol, ou, inf, used


def select_largest_width(net: Net, pre_lo, pre_hi, splits: np.ndarray):
    pre_lo, pre_hi = _f32(pre_lo), _f32(pre_hi)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    r, j, w = C.c_int32(-1), C.c_int32(-1), C.c_float(0)
    ok = lib().nyo_select_largest_width(C.byref(net.c), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data, len(splits),
                                        C.byref(r), C.byref(j), C.byref(w))
    return (r.value, j.value, w.value) if ok else None


def select_intercept(net: Net, pre_lo, pre_hi, splits: np.ndarray):
    """Intercept-score branching choice (relu, neuron, score) or None (picked.rs:153-233)."""
    pre_lo, pre_hi = _f32(pre_lo), _f32(pre_hi)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    r, j, w = C.c_int32(-1), C.c_int32(-1), C.c_float(0)
    ok = lib().nyo_select_intercept(C.byref(net.c), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data, len(splits),
                                    C.byref(r), C.byref(j), C.byref(w))
    return (r.value, j.value, w.value) if ok else None


def heuristic_alpha(net: Net, pre_lo, pre_hi):
    """alpha_0 = [u > -l] on unstable neurons (beta_crown/state/alpha/domain.rs:161), n_pre layout."""
    pre_lo, pre_hi = _f32(pre_lo), _f32(pre_hi)
    return np.where((pre_lo < 0) & (pre_hi > 0), (pre_hi > -pre_lo).astype(np.float32), 0.0).astype(np.float32)


def joint_gradient(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha=None, only_row: int = -1):
    """Returns (lower bounds [S] in binary64, grad_alpha [n_pre], grad_beta [n_splits]): the gradient of the sum of
    the rows' lower bounds, or of row `only_row` alone when it is >= 0."""
    lo, hi, pre_lo, pre_hi = _f32(lo), _f32(hi), _f32(pre_lo), _f32(pre_hi)
    alpha = None if alpha is None else _f32(alpha)
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    S = int(net.dims[-1])
    low = np.empty(S, np.float64)
    ga = np.zeros(net.n_pre, np.float32)
    gb = np.zeros(max(len(splits), 1), np.float32)
    lib().nyo_joint_gradient_rows(C.byref(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data,
                                  len(splits), _fp(alpha), low.ctypes.data_as(C.POINTER(C.c_double)), _fp(ga), _fp(gb),
                                  int(only_row))
    return low, ga, gb[: len(splits)]


def optimize(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha, iterations, lr_alpha, lr_beta,
             lr_decay=0.98, clip_beta=10.0, objective=0):
    """Returns (best_lo [S], best_hi [S], alpha, splits) after projected-Adam optimisation."""
    lo, hi, pre_lo, pre_hi = _f32(lo), _f32(hi), _f32(pre_lo), _f32(pre_hi)
    alpha = _f32(alpha).copy()
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE).copy()
    S = int(net.dims[-1])
    bl, bu = np.empty(S, np.float32), np.empty(S, np.float32)
    lib().nyo_optimize_objective(C.byref(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data,
                                 len(splits), _fp(alpha), iterations, lr_alpha, lr_beta, lr_decay, clip_beta, objective,
                                 _fp(bl), _fp(bu))
    return bl, bu, alpha, splits


class _OptCfg(C.Structure):
    _fields_ = [("iterations", C.c_int32), ("lr_alpha", C.c_float), ("lr_beta", C.c_float), ("lr_decay", C.c_float),
                ("clip_beta", C.c_float), ("objective", C.c_int32), ("rule", C.c_int32), ("tolerance", C.c_float),
                ("patience", C.c_int32), ("start_save_best", C.c_float)]


def optimize_ex(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha, iterations, lr_alpha, lr_beta, lr_decay=0.98,
                clip_beta=10.0, objective=0, rule=0, tolerance=0.0, patience=0, start_save_best=0.0):
    """nyo_optimize_ex: the optimisation loop with the update rule (0 Adam, 1 plain projected step, 2 AMSGrad) and the
    reference's stopping / best-saving rules.  Returns (best_lo, best_hi, alpha, splits, evaluations made)."""
    lo, hi, pre_lo, pre_hi = _f32(lo), _f32(hi), _f32(pre_lo), _f32(pre_hi)
    alpha = _f32(alpha).copy()
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE).copy()
    S = int(net.dims[-1])
    bl, bu = np.empty(S, np.float32), np.empty(S, np.float32)
    cfg = _OptCfg(iterations, lr_alpha, lr_beta, lr_decay, clip_beta, objective, rule, tolerance, patience, start_save_best)
    runs = C.c_int(0)
    fn = lib().nyo_optimize_ex
    fn.argtypes = [C.c_void_p] + [C.POINTER(C.c_float)] * 4 + [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.POINTER(_OptCfg),
                                                               C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float),
                                                               C.POINTER(C.c_int)]
    rc = fn(C.addressof(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data, len(splits), _fp(alpha),
            C.byref(cfg), _fp(bl), _fp(bu), None, C.byref(runs))
    if rc != 0:
        raise ValueError(f"nyo_optimize_ex returned {rc}")
    return bl, bu, alpha, splits, int(runs.value)


def beta_plain_step(values, grads, lr):
    """BetaState::gradient_step (beta_crown/state/beta.rs:272-305), the reference's default multiplier update:
    beta <- max(0, beta + lr * grad) (ascent on the lower bound, projected onto beta >= 0); a non-finite result resets
    the entry to zero.  Returns (values', max |grad|)."""
    v = np.asarray(values, np.float32)
    g = np.asarray(grads, np.float32)
    out = np.maximum(v + np.float32(lr) * g, np.float32(0))
    out = np.where(np.isfinite(v + np.float32(lr) * g), out, np.float32(0)).astype(np.float32)
    return out, float(np.max(np.abs(g))) if g.size else 0.0


def beta_adam_step(state, grads, t, beta_lr=0.05, beta1=0.9, beta2=0.999, epsilon=1e-8, grad_clip=10.0, lr_decay=0.98,
                   amsgrad=False, bias_correction=True):
    """BetaState::gradient_step_adam (beta_crown/state/beta.rs:314-441) with the default scheduler
    (ExponentialDecay: lr_t = beta_lr * lr_decay^(t-1)) and uniform per-layer factors: gradient clipped to
    [-grad_clip, grad_clip], moments m, v, bias corrections 1 - beta^t (floored at machine epsilon), AMSGrad's running
    maximum of v when enabled, beta <- max(0, beta + lr_t * m_hat / (sqrt(v_hat) + epsilon)); an entry whose moments
    became non-finite is reset.  state = dict(value, m, v, v_max) of fp32 arrays; returns (state', max |clipped grad|)."""
    f32 = np.float32
    g = np.asarray(grads, np.float32)
    if grad_clip > 0:
        g = np.clip(g, f32(-grad_clip), f32(grad_clip))
    tf = f32(max(t, 1))
    b1c = max(f32(1) - f32(beta1) ** tf, np.finfo(np.float32).eps) if bias_correction else f32(1)
    b2c = max(f32(1) - f32(beta2) ** tf, np.finfo(np.float32).eps) if bias_correction else f32(1)
    lr = f32(beta_lr) * f32(lr_decay) ** f32(max(t, 1) - 1)
    m = f32(beta1) * state["m"] + f32(1 - beta1) * g
    v = f32(beta2) * state["v"] + f32(1 - beta2) * g * g
    v_max = np.maximum(state["v_max"], v) if amsgrad else state["v_max"]
    v_use = v_max if amsgrad else v
    upd = lr * (m / f32(b1c)) / (np.sqrt(v_use / f32(b2c)) + f32(epsilon))
    val = np.maximum(state["value"] + upd, f32(0)).astype(np.float32)
    bad = ~np.isfinite(m) | ~np.isfinite(v)
    out = {"value": np.where(bad, f32(0), val).astype(np.float32), "m": np.where(bad, f32(0), m).astype(np.float32),
           "v": np.where(bad, f32(0), v).astype(np.float32), "v_max": np.where(bad, f32(0), v_max).astype(np.float32)}
    return out, float(np.max(np.abs(g))) if g.size else 0.0


def adam_clipping_step(m, v, t, gradient, x, lo, hi, lr0, lr_decay=0.99, beta1=0.9, beta2=0.999, eps=1e-8):
    """One AdamClippingState::step (ny-propagate/src/pgd_attack/adam_state.rs:46-88), fp32 state: moments updated
    with `gradient`, direction sign(m / (sqrt(v / bc2) + eps)) with sign(+0) = +1 and 0 where m or the denominator
    is not finite, uniform step lr0 * lr_decay^(t-1) / bc1 (step 1 uses lr0: the ExponentialLR ordering), result
    clamped to [lo, hi].  The caller passes the ascent direction: an attack that minimises flips the gradient first
    (optimizer.rs:296-305).  t is the 1-based step count.  Returns (x', m', v')."""
    f32 = np.float32
    g = np.asarray(gradient, np.float32)
    m = f32(beta1) * np.asarray(m, np.float32) + f32(1 - beta1) * g
    v = f32(beta2) * np.asarray(v, np.float32) + f32(1 - beta2) * g * g
    bc1, bc2 = f32(1 - beta1 ** t), f32(1 - beta2 ** t)
    with np.errstate(invalid="ignore", divide="ignore"):
        denom = np.sqrt(v / bc2) + f32(eps)
        q = m / denom
    d = np.where(np.isfinite(denom) & np.isfinite(m) & ~np.isnan(q), np.copysign(f32(1), q), f32(0)).astype(np.float32)
    step = f32(lr0 * lr_decay ** (t - 1)) / bc1
    xn = np.asarray(x, np.float32) + d * step
    xn = np.where(np.isnan(xn), np.asarray(lo, np.float32), xn)   # project_to_bounds: NaN -> lower end (optimizer.rs:121-127)
    return np.clip(xn, np.asarray(lo, np.float32), np.asarray(hi, np.float32)).astype(np.float32), m.astype(np.float32), v.astype(np.float32)


def pgd_attack(weights, biases, spec, lo, hi, x0, steps, step_size, lr_decay=0.99, beta1=0.9, beta2=0.999, eps=1e-8):
    """numpy restatement of the lock-step PGD attack on a dense sequential ReLU network (convolutions lowered
    with conv2d_dense): objective min_s spec[s] . f(x) per restart, exact gradient of the worst row
    (ny-cli commands/beta_crown/verify/graph_pgd.rs:655-685), AdamClipping step
    (ny-propagate/src/pgd_attack/adam_state.rs:46-88: direction sign(m / (sqrt(v / bc2) + eps)) with
    sign(+0) = +1 and 0 for non-finite values, step lr0 * decay^(t-1) / bc1, projection onto the box), best
    point per restart over all visited points (attacker/batched.rs:33-215), points kept in fp32.
    Returns (best objective [K], best points [K, n0])."""
    Ws = [np.asarray(w, np.float64) for w in weights]
    bs = [None if b is None else np.asarray(b, np.float64) for b in biases]
    spec = np.asarray(spec, np.float64)
    lo32, hi32 = np.asarray(lo, np.float32), np.asarray(hi, np.float32)
    x = np.asarray(x0, np.float32).copy()
    K = x.shape[0]
    m = np.zeros(x.shape, np.float32)
    v = np.zeros(x.shape, np.float32)
    best = np.full(K, np.inf, np.float32)
    best_x = x.copy()
    f32 = np.float32

    def forward(xx):
        acts, z = [], xx.astype(np.float64)
        for k, w in enumerate(Ws):
            z = z @ w.T
            if bs[k] is not None:
                z = z + bs[k]
            if k + 1 < len(Ws):
                z = np.maximum(z, 0.0)
            acts.append(z)
        return acts

    for t in range(1, steps + 2):
        acts = forward(x)
        marg = (acts[-1] @ spec.T).astype(np.float32)
        row = np.argmin(marg, axis=1)
        val = marg[np.arange(K), row]
        imp = val < best
        best[imp] = val[imp]
        best_x[imp] = x[imp]
        if t == steps + 1:
            break
        g = spec[row]
        for k in range(len(Ws) - 1, -1, -1):
            if k + 1 < len(Ws):
                g = g * (acts[k] > 0)
            g = g @ Ws[k]
        g = g.astype(np.float32)
        # the moments follow the objective's gradient; the point moves against their direction (the attack minimises)
        _, m, v = adam_clipping_step(m, v, t, g, x, lo32, hi32, step_size, lr_decay, beta1, beta2, eps)
        bc1, bc2 = f32(1 - beta1 ** t), f32(1 - beta2 ** t)
        denom = np.sqrt(v / bc2) + f32(eps)
        with np.errstate(invalid="ignore", divide="ignore"):
            q = m / denom
        d = np.where(np.isfinite(denom) & np.isfinite(m) & ~np.isnan(q), np.copysign(f32(1), q), f32(0)).astype(np.float32)
        step = f32(step_size * lr_decay ** (t - 1)) / bc1
        x = np.clip(x - d * step, lo32, hi32).astype(np.float32)
    vals = (forward(best_x)[-1] @ spec.T).min(axis=1).astype(np.float32)
    return vals, best_x


def crown_exact_f64(ws, bs, spec, lo, hi, sparse_rule=True):
    """The plain-CROWN pipeline of nyo_crown (CROWN-IBP collection, merge rules, sparse rule, final tighten) in
    plain binary64 numpy with NO outward rounding and no error accounting: the value an exact-arithmetic
    implementation of the same algorithm returns, up to binary64 noise.  A sound floating-point implementation
    can only be looser than this; tests use it to order the device result between the reference's certified
    bound and the exact value.  Returns ((lower [S], upper [S]), per-layer tightened bounds)."""
    ws = [np.asarray(w, np.float64) for w in ws] + [np.asarray(spec, np.float64)]
    bs = [None if b is None else np.asarray(b, np.float64) for b in bs] + [None]
    L = len(ws)
    relu_after = [1] * (L - 2) + [0, 0]
    lo = np.asarray(lo, np.float64); hi = np.asarray(hi, np.float64)
    def lin_ibp(k, l, u):
        wp, wn = np.maximum(ws[k], 0), np.minimum(ws[k], 0)
        b = 0 if bs[k] is None else bs[k]
        return wp @ l + wn @ u + b, wp @ u + wn @ l + b
    ibp = []
    l, u = lo, hi
    for k in range(L):
        a, b = lin_ibp(k, l, u); ibp.append((a, b))
        l, u = (np.maximum(a, 0), np.maximum(b, 0)) if relu_after[k] else (a, b)
    t = [None] * L
    def backward(top, seedn):
        la = np.eye(seedn); ua = np.eye(seedn); lb = np.zeros(seedn); ub = np.zeros(seedn)
        for k in range(top, -1, -1):
            if bs[k] is not None:
                lb = lb + la @ bs[k]; ub = ub + ua @ bs[k]
            la = la @ ws[k]; ua = ua @ ws[k]
            if k > 0 and relu_after[k - 1]:
                pl, pu = t[k - 1]
                ls = np.where(pl >= 0, 1.0, np.where(pu <= 0, 0.0, (pu > -pl) * 1.0))
                us = np.where(pl >= 0, 1.0, np.where(pu <= 0, 0.0, pu / np.where(pu - pl == 0, 1, pu - pl)))
                ui = np.where((pl < 0) & (pu > 0), -us * pl, 0.0)
                lb = lb + np.minimum(la, 0) @ ui; ub = ub + np.maximum(ua, 0) @ ui
                la = np.maximum(la, 0) * ls + np.minimum(la, 0) * us
                ua = np.maximum(ua, 0) * us + np.minimum(ua, 0) * ls
        return (np.maximum(la, 0) @ lo + np.minimum(la, 0) @ hi + lb, np.maximum(ua, 0) @ hi + np.minimum(ua, 0) @ lo + ub)
    def inter(a, b):
        l, u = np.maximum(a[0], b[0]), np.minimum(a[1], b[1])
        bad = l > u
        return np.where(bad, np.minimum(a[0], b[0]), l), np.where(bad, np.maximum(a[1], b[1]), u)
    for k in range(L):
        il, iu = ibp[k]
        if k < L - 1 and relu_after[k] and np.all((il >= 0) | (iu <= 0)):
            t[k] = (il, iu); continue
        if k == 0: zl, zu = lo, hi
        else:
            act = relu_after[k - 1]
            z = (np.maximum(t[k-1][0], 0), np.maximum(t[k-1][1], 0)) if act else t[k-1]
            f0 = (np.maximum(ibp[k-1][0], 0), np.maximum(ibp[k-1][1], 0)) if act else ibp[k-1]
            zl, zu = inter(f0, z)
        f = lin_ibp(k, zl, zu)
        if k < L - 1 and not relu_after[k]:
            t[k] = inter((il, iu), f); continue
        c = backward(k, ws[k].shape[0])
        unst = (f[0] < 0) & (f[1] > 0)
        n = len(il)
        if sparse_rule and unst.sum() > 0 and not (np.float32(1.0) - np.float32(unst.sum()) / np.float32(n) < np.float32(0.9)):
            c = (np.where(unst, c[0], f[0]), np.where(unst, c[1], f[1]))
        t[k] = inter((il, iu), c)
    c = backward(L - 1, ws[-1].shape[0])
    return inter(c, t[L - 1]), t


def beta_crown_bound_dual(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha, alpha_up):
    """beta-CROWN bound with a separate upper-path slope alpha_up (dual alpha)."""
    lo, hi, pre_lo, pre_hi, alpha, alpha_up = (_f32(x) for x in (lo, hi, pre_lo, pre_hi, alpha, alpha_up))
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    S = int(net.dims[-1])
    ol, ou = np.empty(S, np.float32), np.empty(S, np.float32)
    lib().nyo_beta_crown_bound_dual(C.byref(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data,
                                    len(splits), _fp(alpha), _fp(alpha_up), _fp(ol), _fp(ou))
    return ol, ou


def upper_gradient(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha, alpha_up):
    """(upper bounds [S] in binary64, gradient of their sum with respect to alpha_up [n_pre])."""
    lo, hi, pre_lo, pre_hi, alpha, alpha_up = (_f32(x) for x in (lo, hi, pre_lo, pre_hi, alpha, alpha_up))
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
    S = int(net.dims[-1])
    up = np.empty(S, np.float64)
    g = np.zeros(net.n_pre, np.float32)
    lib().nyo_upper_gradient(C.byref(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data, len(splits),
                             _fp(alpha), _fp(alpha_up), up.ctypes.data_as(C.POINTER(C.c_double)), _fp(g))
    return up, g


def optimize_dual(net: Net, lo, hi, pre_lo, pre_hi, splits: np.ndarray, alpha, iterations, lr_alpha, lr_beta,
                  lr_decay=0.98, clip_beta=10.0):
    """Dual-alpha optimisation: returns (best_lo, best_hi, alpha, alpha_up, splits)."""
    lo, hi, pre_lo, pre_hi = _f32(lo), _f32(hi), _f32(pre_lo), _f32(pre_hi)
    alpha = _f32(alpha).copy()
    splits = np.ascontiguousarray(splits, SPLIT_DTYPE).copy()
    S = int(net.dims[-1])
    bl, bu = np.empty(S, np.float32), np.empty(S, np.float32)
    aup = np.zeros(net.n_pre, np.float32)
    lib().nyo_optimize_dual(C.byref(net.c), _fp(lo), _fp(hi), _fp(pre_lo), _fp(pre_hi), splits.ctypes.data, len(splits),
                            _fp(alpha), iterations, lr_alpha, lr_beta, lr_decay, clip_beta, 2, _fp(bl), _fp(bu), _fp(aup))
    return bl, bu, alpha, aup, splits


def babsr_scores(weights, biases, spec, pre_lo, pre_hi, split_mask=None, with_backup=False):
    """numpy restatement of the reference's BaBSR scores for one domain of a dense sequential ReLU network
    (compute_babsr_scores, crates/ny-propagate/src/beta_crown/engine/branching/sequential.rs:784-882, with
    compute_babsr_score_parts, branching/score.rs:28-97, and relu_upper_slope, branching/mod.rs:93-111; reduce op Min
    as select_babsr_neuron uses it).  The specification rows play the role of the last Linear layer.
    pre_lo / pre_hi: [n_pre] pre-activation bounds of the domain (already clamped by its splits); split_mask: [n_pre]
    bool, True for split neurons.  Returns (scores [n_hidden] float32, -1 for neurons that are not candidates,
    (relu, neuron) of the first maximum or (-1, -1))."""
    f32 = np.float32
    dims = [w.shape[0] for w in weights]
    offs = np.concatenate([[0], np.cumsum(dims)]).astype(int)
    n_hidden = int(offs[len(weights) - 1])
    scores = np.full(n_hidden, -1.0, f32)
    backup = np.full(n_hidden, 1.0, f32)   # BabsrScoreParts::backup_score: mean intercept term (+1: not a candidate)
    C = np.asarray(spec, f32)
    for k in range(len(weights) - 1, 0, -1):
        C = (C.astype(np.float64) @ np.asarray(weights[k], np.float64)).astype(f32)
        off, n = int(offs[k - 1]), dims[k - 1]
        b = np.zeros(n, f32) if biases[k - 1] is None else np.asarray(biases[k - 1], f32)
        for j in range(n):
            l, u = f32(pre_lo[off + j]), f32(pre_hi[off + j])
            have = np.isfinite(l) and np.isfinite(u)
            r0 = r1 = f32(0)
            if have:
                lt, ut = min(l, f32(0)), max(u, f32(0))
                w = f32(ut - lt)
                if abs(w) <= f32(1e-6):
                    have = False
                else:
                    r0 = f32(ut / w)
                    r1 = f32(-lt * r0)
                    have = bool(np.isfinite(r0) and np.isfinite(r1))
            col = C[:, j]
            ok, total, btotal = have, 0.0, 0.0
            if ok:
                for c in col:
                    if not np.isfinite(c):
                        ok = False
                        break
                    ic = f32(min(c, f32(0)) * r1)
                    bs = f32(b[j] * c)
                    bc = min(f32(bs * f32(r0 - f32(1))), f32(bs * r0))
                    mc = f32(abs(f32(bc + ic)))
                    if not (np.isfinite(ic) and np.isfinite(mc)):
                        ok = False
                        break
                    total += float(mc)
                    btotal += float(ic)
            cand = l < 0 and u > 0 and not (split_mask is not None and split_mask[off + j])
            if cand:
                scores[off + j] = f32(total / len(col)) if ok else f32(0)
                backup[off + j] = f32(btotal / len(col)) if ok else f32(0)
            if not (np.isfinite(l) and np.isfinite(u)) or l >= 0:
                slope = f32(1)
            elif u <= 0:
                slope = f32(0)
            else:
                slope = f32(u / max(f32(u - l), f32(1e-8)))
            C[:, j] = (col * slope).astype(f32)
    best, pick = f32(-1), -1
    for i, s in enumerate(scores):
        if s > best:
            best, pick = s, i
    if pick < 0:
        sel = (-1, -1)
    else:
        r = int(np.searchsorted(offs[1:], pick, side="right"))
        sel = (r, pick - int(offs[r]))
    return (scores, sel, backup) if with_backup else (scores, sel)
