"""Python host mirror of ny's engine plugin interface over the nyb200 C ABI.

Method names and argument meaning follow the reference traits so that parity tests read like
the reference's own (paths inside the ny project):
  GemmEngine::gemm_f32                      crates/ny-core/src/gemm.rs:325
  GpuIbpForward::ibp_forward_gpu_sound      crates/ny-core/src/gemm_gpu_ibp.rs:78-135
  GpuCrownBackward::*_beta_batched          crates/ny-core/src/gemm.rs:3944
  BetaCrownVerifier (batched BaB round)     crates/ny-propagate/src/beta_crown/engine/graph/gpu_bab/batched_gpu.rs:89
Errors map NyError variants (crates/ny-core/src/error.rs:18) onto EngineError.code.

There is no CPU fallback: constructing an engine without the compiled library or without a
CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libnyb200.so")

SPLIT_DTYPE = np.dtype([("relu", "<i4"), ("neuron", "<i4"), ("sign", "<i4"), ("beta", "<f4")])

OK, UNSUPPORTED, SHAPE, INVALID, NUMERICAL, DEADLINE, OOM, INTERNAL = range(8)
_NAMES = {
    UNSUPPORTED: "UnsupportedOp", SHAPE: "ShapeMismatch", INVALID: "InvalidSpec", NUMERICAL: "NumericalInstability",
    DEADLINE: "DeadlineExceeded", OOM: "MemoryExceeded", INTERNAL: "InternalError",
}
PATH_F64, PATH_TF32X3 = 0, 1
ERRCH_IMMEDIATE, ERRCH_REFERENCE = 0, 1

EXPORTS = [
    "nyb200_create", "nyb200_destroy", "nyb200_backend_provenance", "nyb200_last_error", "nyb200_set_stream",
    "nyb200_set_path", "nyb200_set_refine_tolerance", "nyb200_batch_refined", "nyb200_batch_poll", "nyb200_crown_bounds_split", "nyb200_batch_set_inherited", "nyb200_batch_set_thresholds", "nyb200_frontier_create", "nyb200_frontier_round", "nyb200_frontier_round_optimized", "nyb200_frontier_set_refinement", "nyb200_frontier_destroy", "nyb200_frontier_count", "nyb200_frontier_take", "nyb200_frontier_give", "nyb200_frontier_download", "nyb200_frontier_upload", "nyb200_launch_count", "nyb200_clear_working_set", "nyb200_gemm_f32", "nyb200_gemm_f32_fast", "nyb200_net_create",
    "nyb200_net_destroy", "nyb200_ibp_forward", "nyb200_ibp_forward_noalloc", "nyb200_bab_bound_batch", "nyb200_batch_upload", "nyb200_batch_run",
    "nyb200_batch_download", "nyb200_batch_min_lower", "nyb200_batch_min_lower_device",
    "nyb200_batch_download_pre_bounds", "nyb200_batch_select_branch", "nyb200_timing_enable", "nyb200_timing_reset",
    "nyb200_timing_read", "nyb200_batch_optimize", "nyb200_batch_download_params",
    "nyb200_net_create_layers", "nyb200_pgd_attack", "nyb200_batch_select_branch_scored",
    "nyb200_crown_bounds", "nyb200_batch_download_alpha_upper",
    "nyb200_batch_verdicts", "nyb200_gemm_f64", "nyb200_conv_transpose_2d", "nyb200_set_deadline_ns",
    "nyb200_batch_gradient", "nyb200_point_vjp_batched", "nyb200_crown_input_coeffs", "nyb200_batch_download_branch_scores",
    "nyb200_set_error_channel", "nyb200_set_fusion", "nyb200_use_own_stream", "nyb200_set_reserved_sms", "nyb200_set_launch_overlap", "nyb200_batch_download_opt_evaluations",
    "nyb200_crown_backward", "nyb200_crown_resnet_beta_batched", "nyb200_crown_resnet_beta_batched_adam", "nyb200_gemm_f64_triplet",
]


class OptConfig(C.Structure):
    """nyb200_opt_config: projected-Adam settings of nyb200_batch_optimize (zeros select Adam's defaults)."""
    _fields_ = [("iterations", C.c_int32), ("lr_alpha", C.c_float), ("lr_beta", C.c_float), ("lr_decay", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float), ("clip_beta", C.c_float),
                ("objective", C.c_int32), ("rule", C.c_int32), ("tolerance", C.c_float), ("patience", C.c_int32),
                ("start_save_best", C.c_float)]


class ConvTransposeParams(C.Structure):
    """nyb200_conv_transpose_params (ConvTranspose2dParams, crates/ny-core/src/gemm.rs:150-177)."""
    _fields_ = [(n, C.c_int32) for n in ("num_specs", "out_channels", "in_channels", "out_h", "out_w", "in_h", "in_w",
                                         "kernel_h", "kernel_w", "stride_h", "stride_w", "pad_h", "pad_w")]


class CrownLayer(C.Structure):
    """nyb200_crown_layer (GpuCrownLayer::{Linear, Activation, ActivationReluDualAlpha}, crates/ny-core/src/gemm.rs:1524-1645)."""
    _fields_ = [("kind", C.c_int32), ("weight", C.POINTER(C.c_float)), ("bias", C.POINTER(C.c_float)),
                ("out_features", C.c_int32), ("in_features", C.c_int32),
                ("lower_slope", C.POINTER(C.c_float)), ("upper_slope", C.POINTER(C.c_float)),
                ("lower_intercept", C.POINTER(C.c_float)), ("upper_intercept", C.POINTER(C.c_float)),
                ("upper_neg_slope", C.POINTER(C.c_float)), ("num_neurons", C.c_int32)]


class CrownSeed(C.Structure):
    """nyb200_crown_seed (GpuCrownSeed, gemm.rs:1684-1691)."""
    _fields_ = [("lower_a", C.POINTER(C.c_float)), ("upper_a", C.POINTER(C.c_float)), ("lower_b", C.POINTER(C.c_float)),
                ("upper_b", C.POINTER(C.c_float)), ("num_specs", C.c_int32), ("current_dim", C.c_int32)]


class DomainRef(C.Structure):
    """nyb200_domain_ref (GpuResnetBatchedDomainRef, gemm.rs:2939-2952)."""
    _fields_ = [("layers", C.POINTER(CrownLayer)), ("n_layers", C.c_int32), ("input_lower", C.POINTER(C.c_float)),
                ("input_upper", C.POINTER(C.c_float)), ("beta_signed", C.POINTER(C.POINTER(C.c_float))),
                ("frontier_abs", C.POINTER(C.POINTER(C.c_float))), ("node_abs", C.POINTER(C.POINTER(C.c_float))),
                ("splits", C.c_void_p), ("n_splits", C.c_int32)]


class BetaAdamConfig(C.Structure):
    """nyb200_beta_adam_config (GpuBetaAdamConfig, gemm.rs:2960-2993)."""
    _fields_ = [("iterations", C.c_int32), ("beta_lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("epsilon", C.c_float), ("tolerance", C.c_float)]


class EngineError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{_NAMES.get(code, code)}: {message}")
        self.code = code


_lib = None


def load_library():
    """Load libnyb200.so; raises if it has not been built (python -m ny_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise EngineError(UNSUPPORTED, f"{_LIB_PATH} is missing: build it with `python -m ny_b200.build`")
    L = C.CDLL(_LIB_PATH)
    fp, ip, vp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_void_p
    L.nyb200_create.argtypes = [C.c_int32, C.POINTER(vp)]
    L.nyb200_destroy.argtypes = [vp]
    L.nyb200_destroy.restype = None
    L.nyb200_backend_provenance.restype = C.c_char_p
    L.nyb200_last_error.argtypes = [vp]
    L.nyb200_last_error.restype = C.c_char_p
    L.nyb200_set_stream.argtypes = [vp, vp]
    L.nyb200_set_path.argtypes = [vp, C.c_int32]
    L.nyb200_set_error_channel.argtypes = [vp, C.c_int32]
    L.nyb200_set_fusion.argtypes = [vp, C.c_int32]
    L.nyb200_batch_download_opt_evaluations.argtypes = [vp, ip]
    L.nyb200_set_refine_tolerance.argtypes = [vp, C.c_float]
    L.nyb200_batch_refined.argtypes = [vp, ip]
    L.nyb200_batch_poll.argtypes = [vp, ip, ip]
    L.nyb200_launch_count.argtypes = [vp]
    L.nyb200_launch_count.restype = C.c_int64
    L.nyb200_clear_working_set.argtypes = [vp]
    L.nyb200_gemm_f32.argtypes = [vp, C.c_int32, C.c_int32, C.c_int32, fp, fp, fp]
    L.nyb200_gemm_f32_fast.argtypes = [vp, C.c_int32, C.c_int32, C.c_int32, fp, fp, fp]
    L.nyb200_net_create.argtypes = [vp, C.c_int32, ip, fp, fp, ip, ip]
    L.nyb200_net_create_layers.argtypes = [vp, C.c_int32, C.POINTER(LayerDesc), fp, fp, ip]
    L.nyb200_net_destroy.argtypes = [vp, C.c_int32]
    L.nyb200_ibp_forward.argtypes = [vp, C.c_int32, C.c_int32, fp, fp, C.c_int32, fp, fp]
    L.nyb200_ibp_forward_noalloc.argtypes = [vp, C.c_int32, vp, vp, vp, vp]
    batch_args = [vp, C.c_int32, fp, C.c_int32, fp, fp, C.c_int32, fp, fp, vp, ip, C.c_int32, C.c_int32, C.c_int32, fp]
    L.nyb200_bab_bound_batch.argtypes = batch_args + [fp, fp, ip]
    L.nyb200_batch_upload.argtypes = batch_args
    L.nyb200_batch_run.argtypes = [vp]
    L.nyb200_batch_download.argtypes = [vp, fp, fp, ip]
    L.nyb200_batch_min_lower.argtypes = [vp, fp]
    L.nyb200_batch_min_lower_device.argtypes = [vp, C.POINTER(vp)]
    L.nyb200_batch_download_pre_bounds.argtypes = [vp, fp, fp]
    L.nyb200_batch_verdicts.argtypes = [vp, C.c_float, ip]
    L.nyb200_batch_select_branch.argtypes = [vp, ip, ip, fp]
    L.nyb200_batch_select_branch_scored.argtypes = [vp, C.c_int32, ip, ip, fp]
    L.nyb200_timing_enable.argtypes = [vp, C.c_int32]
    L.nyb200_timing_reset.argtypes = [vp]
    L.nyb200_timing_read.argtypes = [vp, C.c_char_p, C.POINTER(C.c_double), ip]
    L.nyb200_crown_bounds.argtypes = [vp, C.c_int32, fp, C.c_int32, fp, fp, C.c_int32, C.c_int32, fp, fp, fp, fp]
    L.nyb200_pgd_attack.argtypes = [vp, C.c_int32, fp, C.c_int32, fp, fp, fp, C.c_int32, C.POINTER(PgdConfig), fp, fp, ip]
    L.nyb200_batch_optimize.argtypes = [vp, C.POINTER(OptConfig)]
    L.nyb200_batch_download_params.argtypes = [vp, fp, fp]
    L.nyb200_batch_download_alpha_upper.argtypes = [vp, fp]
    dp = C.POINTER(C.c_double)
    L.nyb200_gemm_f64.argtypes = [vp, C.c_int32, C.c_int32, C.c_int32, dp, dp, dp]
    L.nyb200_conv_transpose_2d.argtypes = [vp, fp, fp, C.POINTER(ConvTransposeParams), fp]
    L.nyb200_set_deadline_ns.argtypes = [vp, C.c_int64]
    L.nyb200_batch_gradient.argtypes = [vp, C.c_int32, fp]
    L.nyb200_crown_input_coeffs.argtypes = [vp, fp, fp]
    L.nyb200_batch_download_branch_scores.argtypes = [vp, fp, fp]
    L.nyb200_point_vjp_batched.argtypes = [vp, C.c_int32, C.c_int32, fp, fp, fp, fp, fp]
    _lib = L
    return L


def _fp(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def _ip(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class PgdConfig(C.Structure):
    """nyb200_pgd_config (zeros select the reference's defaults for decay and the Adam moments)."""
    _fields_ = [("steps", C.c_int32), ("step_size", C.c_float), ("lr_decay", C.c_float), ("beta1", C.c_float),
                ("beta2", C.c_float), ("epsilon", C.c_float)]


class LayerDesc(C.Structure):
    """nyb200_layer_desc."""
    _fields_ = [(n, C.c_int32) for n in (
        "kind", "in_features", "out_features", "has_bias", "in_channels", "in_h", "in_w", "out_channels", "out_h",
        "out_w", "kernel_h", "kernel_w", "stride_h", "stride_w", "pad_h", "pad_w", "skip_from")]


class Conv2d:
    """Conv2d layer description (host side): weight [oc, ic, kh, kw], optional per-channel bias [oc]; tensors
    are NCHW flattened, dilation 1, one group (the Conv2d member of GpuCrownLayer)."""

    def __init__(self, weight, bias=None, stride=(1, 1), pad=(0, 0), in_hw=None):
        self.weight = _f32(weight)
        if self.weight.ndim != 4:
            raise EngineError(SHAPE, "conv2d kernel must be 4-D [oc, ic, kh, kw]")
        if in_hw is None:
            raise EngineError(SHAPE, "conv2d needs its input height and width")
        self.oc, self.ic, self.kh, self.kw = (int(x) for x in self.weight.shape)
        self.sh, self.sw = int(stride[0]), int(stride[1])
        self.ph, self.pw = int(pad[0]), int(pad[1])
        self.ih, self.iw = int(in_hw[0]), int(in_hw[1])
        if min(self.sh, self.sw) <= 0 or min(self.kh, self.kw) <= 0:
            raise EngineError(SHAPE, "conv2d: zero stride or kernel")
        if self.ih + 2 * self.ph < self.kh or self.iw + 2 * self.pw < self.kw:
            raise EngineError(SHAPE, "conv2d: kernel larger than the padded input")
        self.oh = (self.ih + 2 * self.ph - self.kh) // self.sh + 1
        self.ow = (self.iw + 2 * self.pw - self.kw) // self.sw + 1
        self.bias = None if bias is None else _f32(bias)
        if self.bias is not None and self.bias.shape != (self.oc,):
            raise EngineError(SHAPE, "conv2d bias must be [oc]")
        self.in_features = self.ic * self.ih * self.iw
        self.out_features = self.oc * self.oh * self.ow

    def apply(self, x: np.ndarray) -> np.ndarray:
        """Concrete forward convolution of rows x [N, in_features] in binary64 (used by sampling checks)."""
        x = np.asarray(x, np.float64).reshape(-1, self.ic, self.ih, self.iw)
        xp = np.pad(x, ((0, 0), (0, 0), (self.ph, self.ph), (self.pw, self.pw)))
        win = np.lib.stride_tricks.sliding_window_view(xp, (self.kh, self.kw), axis=(2, 3))
        win = win[:, :, :: self.sh, :: self.sw][:, :, : self.oh, : self.ow]
        y = np.einsum("nchwyx,ocyx->nohw", win, self.weight.astype(np.float64), optimize=True)
        if self.bias is not None:
            y = y + self.bias.astype(np.float64)[None, :, None, None]
        return y.reshape(x.shape[0], self.out_features)

    def desc(self) -> LayerDesc:
        return LayerDesc(1, self.in_features, self.out_features, 0 if self.bias is None else 1, self.ic, self.ih, self.iw,
                         self.oc, self.oh, self.ow, self.kh, self.kw, self.sh, self.sw, self.ph, self.pw)


def lower_projection_block(function, projection):
    """A projection residual block `out = F(z) + P(z)` (GpuResnetSegment::ResidualProj, crates/ny-core/src/gemm.rs:
    1658-1669) as plain sequential layers, for a block input z that is a post-ReLU tensor (z >= 0).

    function: [(weight, bias), ...] the layers of F in forward order, a ReLU between consecutive ones (two or more
    layers); projection: (weight, bias), one layer without activation.  All Linear ([out, in] matrices) or all Conv2d.
    Every layer of F but the last is widened by channels (neurons) that carry z through unchanged - an identity row,
    or for a convolution the tap that reads the output pixel's own input pixel, so a strided first layer carries z
    subsampled exactly as a strided 1x1 projection reads it; the ReLUs leave the carried values alone because
    z >= 0 - and the last layer reads P's weights from the carried channels.  The result computes F(z) + P(z) exactly;
    in bound propagation the carried neurons are stably active, their relaxation is the identity, so the bounds are
    those of relaxing F and P separately and adding them (the reference's merge).  Returns [(weight, bias), ...]."""
    (pw, pb) = projection
    n = len(function)
    if n < 2:
        raise EngineError(UNSUPPORTED, "projection block: F needs at least two layers (a one-layer F folds into P)")
    conv = isinstance(function[0][0], Conv2d)
    if any(isinstance(w, Conv2d) != conv for w, _ in function) or isinstance(pw, Conv2d) != conv:
        raise EngineError(UNSUPPORTED, "projection block: mixed Linear and Conv2d layers")
    out = []
    if not conv:
        ws = [_f32(w) for w, _ in function]
        bs = [None if b is None else _f32(b) for _, b in function]
        pw = _f32(pw)
        nz = ws[0].shape[1]
        if pw.shape != (ws[-1].shape[0], nz):
            raise EngineError(SHAPE, "projection block: P must map the block input to the block output")
        # when both F's last layer and P have a bias, their fp32 sum need not be exact: P's bias then rides on one more
        # carried neuron that holds the constant 1
        one = 1 if (pb is not None and bs[-1] is not None) else 0
        nc = nz + one
        for k in range(n - 1):
            w, b = ws[k], bs[k]
            if k == 0:
                w2 = np.zeros((w.shape[0] + nc, nz), np.float32)
                w2[: w.shape[0]] = w
                w2[w.shape[0] + np.arange(nz), np.arange(nz)] = 1.0
            else:
                w2 = np.zeros((w.shape[0] + nc, w.shape[1] + nc), np.float32)
                w2[: w.shape[0], : w.shape[1]] = w
                w2[w.shape[0] + np.arange(nc), w.shape[1] + np.arange(nc)] = 1.0
            b2 = np.concatenate([np.zeros(w.shape[0], np.float32) if b is None else b, np.zeros(nc, np.float32)])
            if one and k == 0:
                b2[-1] = 1.0
            out.append((w2, b2))
        w, b = ws[-1], bs[-1]
        cols = [w, pw] + ([_f32(pb).reshape(-1, 1)] if one else [])
        wl = np.concatenate(cols, axis=1)
        bl = b if b is not None else (None if pb is None else _f32(pb))
        out.append((wl, bl))
        return out
    # convolutions
    if (pw.kh, pw.kw, pw.ph, pw.pw) != (1, 1, 0, 0):
        raise EngineError(UNSUPPORTED, "projection block: P must be a 1x1 convolution without padding")
    first = function[0][0]
    if (first.sh, first.sw) != (pw.sh, pw.sw) or first.ic != pw.ic or (first.ih, first.iw) != (pw.ih, pw.iw):
        raise EngineError(UNSUPPORTED, "projection block: P's stride and input must be those of F's first layer")
    cz = first.ic
    for k, (w, _) in enumerate(function):
        if w.ph >= w.kh or w.pw >= w.kw:
            raise EngineError(UNSUPPORTED, "projection block: a layer of F has no tap on its own input pixel")
        if k > 0 and (w.sh, w.sw) != (1, 1):
            raise EngineError(UNSUPPORTED, "projection block: only F's first layer may be strided")
        if k > 0 and ((w.oh, w.ow) != (w.ih, w.iw)):
            raise EngineError(UNSUPPORTED, "projection block: F's later layers must keep the image size")
    if (pw.oh, pw.ow) != (first.oh, first.ow) or pw.oc != function[-1][0].oc:
        raise EngineError(SHAPE, "projection block: P must map the block input to the block output")
    one = 1 if (pw.bias is not None and function[-1][0].bias is not None) else 0   # as for Linear: a channel of ones
    nc = cz + one
    for k, (w, _) in enumerate(function):
        last = k == n - 1
        ic2 = w.ic + (0 if k == 0 else nc)
        oc2 = w.oc + (0 if last else nc)
        ker = np.zeros((oc2, ic2, w.kh, w.kw), np.float32)
        ker[: w.oc, : w.ic] = w.weight
        if last:
            ker[: w.oc, w.ic: w.ic + cz, w.ph, w.pw] = pw.weight[:, :, 0, 0]
            if one:
                ker[: w.oc, w.ic + cz, w.ph, w.pw] = pw.bias
        elif k == 0:
            ker[w.oc + np.arange(cz), np.arange(cz), w.ph, w.pw] = 1.0
        else:
            ker[w.oc + np.arange(nc), w.ic + np.arange(nc), w.ph, w.pw] = 1.0
        b = np.zeros(w.oc, np.float32) if w.bias is None else w.bias
        if last:
            b2 = w.bias if w.bias is not None else pw.bias
        else:
            b2 = np.concatenate([b, np.zeros(nc, np.float32)])
            if one and k == 0:
                b2[-1] = 1.0
        out.append((Conv2d(ker, None if b2 is None else np.asarray(b2, np.float32), (w.sh, w.sw), (w.ph, w.pw), (w.ih, w.iw)), None))
    return out


class Network:
    """Sequential ReLU network description (host side): weights[k] is a [out, in] row-major matrix (Linear) or a
    Conv2d; every layer but the last is followed by a ReLU."""

    def __init__(self, weights, biases=None, skips=None):
        """skips: optional {k: j}: the post-activation output of layer j is added to layer k's output before its
        ReLU (a residual block's identity branch); j <= k - 2, equal widths."""
        self.weights = [w if isinstance(w, Conv2d) else _f32(w) for w in weights]
        L = len(self.weights)
        self.skips = dict(skips or {})
        biases = biases if biases is not None else [None] * L
        self.biases = [w.bias if isinstance(w, Conv2d) else (None if b is None else _f32(b))
                       for w, b in zip(self.weights, biases)]
        first = self.weights[0]
        n0 = first.in_features if isinstance(first, Conv2d) else first.shape[1]
        self.dims = np.array([n0] + [w.out_features if isinstance(w, Conv2d) else w.shape[0] for w in self.weights],
                             dtype=np.int32)
        for k, w in enumerate(self.weights):
            if isinstance(w, Conv2d):
                if w.in_features != self.dims[k]:
                    raise EngineError(SHAPE, f"layer {k}: conv input size {w.in_features} != {self.dims[k]}")
            elif w.shape != (self.dims[k + 1], self.dims[k]):
                raise EngineError(SHAPE, f"layer {k}: weight shape {w.shape}")

        for k, j in self.skips.items():
            if not (0 <= j <= k - 2) or k >= L - 1 or self.dims[j + 1] != self.dims[k + 1]:
                raise EngineError(SHAPE, f"residual connection {j} -> {k}")

    @property
    def has_conv(self) -> bool:
        return any(isinstance(w, Conv2d) for w in self.weights)

    def layer_forward(self, k: int, z: np.ndarray) -> np.ndarray:
        """Concrete image of rows z under layer k (binary64, bias included, no activation)."""
        w = self.weights[k]
        if isinstance(w, Conv2d):
            return w.apply(z)
        z = z @ w.astype(np.float64).T
        return z if self.biases[k] is None else z + self.biases[k].astype(np.float64)

    @property
    def n_pre(self) -> int:
        return int(self.dims[1:].sum())


class B200Engine:
    """One engine per GPU (and per thread of control); mirrors `Arc<dyn GemmEngine>`."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._L = load_library()
        h = C.c_void_p()
        st = self._L.nyb200_create(device, C.byref(h))
        if st != OK:
            raise EngineError(st, "no usable sm_100 CUDA device for nyb200_create (there is no CPU fallback)")
        self._h = h
        self._nets = {}
        if stream is not None:
            self.set_stream(stream)

    def close(self):
        if getattr(self, "_h", None):
            self._L.nyb200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int):
        if st != OK:
            raise EngineError(st, self._L.nyb200_last_error(self._h).decode())

    # -- configuration ---------------------------------------------------------------------
    def backend_provenance(self) -> str:
        return self._L.nyb200_backend_provenance().decode()

    def set_stream(self, cuda_stream: int):
        self._check(self._L.nyb200_set_stream(self._h, C.c_void_p(cuda_stream)))

    def use_own_stream(self):
        """A non-blocking stream of the engine's own (several engines on one GPU then overlap: ny_b200.pool)."""
        self._L.nyb200_use_own_stream.argtypes = [C.c_void_p]
        self._check(self._L.nyb200_use_own_stream(self._h))

    def set_reserved_sms(self, n: int):
        """SMs the persistent kernels leave to a collective that runs beside them on another stream (default 0)."""
        self._L.nyb200_set_reserved_sms.argtypes = [C.c_void_p, C.c_int32]
        self._check(self._L.nyb200_set_reserved_sms(self._h, int(n)))

    def set_launch_overlap(self, on: bool):
        """Programmatic dependent launch of this engine's kernels (default on; off pays with several engines per GPU)."""
        self._L.nyb200_set_launch_overlap.argtypes = [C.c_void_p, C.c_int32]
        self._check(self._L.nyb200_set_launch_overlap(self._h, 1 if on else 0))

    def set_path(self, path: int):
        self._check(self._L.nyb200_set_path(self._h, path))

    def set_error_channel(self, mode: int):
        """ERRCH_IMMEDIATE (default: roundings discharged layer by layer, tighter than the reference on deep nets) or
        ERRCH_REFERENCE (the reference's carried per-coefficient error matrices, binary64: plain-CROWN bounds equal to
        the reference's CPU bounds within 1e-4)."""
        self._check(self._L.nyb200_set_error_channel(self._h, mode))

    def set_fusion(self, on: bool):
        """Fused backward chain (default on) or one launch per layer."""
        self._check(self._L.nyb200_set_fusion(self._h, 1 if on else 0))

    # -- reference-shaped calls (caller-baked relaxation tables, layer lists in backward order) -------------
    @staticmethod
    def _crown_layers(layers, keep):
        """layers: backward-order list of ("linear", W [out, in], b or None) and ("act", lower_slope, upper_slope,
        lower_intercept or None, upper_intercept) entries -> ctypes array (buffers appended to `keep`)."""
        arr = (CrownLayer * len(layers))()
        for i, l in enumerate(layers):
            if l[0] == "linear":
                w = _f32(l[1]); b = None if l[2] is None else _f32(l[2])
                keep += [w, b]
                arr[i].kind = 0
                arr[i].weight = _fp(w); arr[i].bias = _fp(b)
                arr[i].out_features, arr[i].in_features = int(w.shape[0]), int(w.shape[1])
            elif l[0] == "act":
                ls, us, ui = _f32(l[1]), _f32(l[2]), _f32(l[4])
                li = None if l[3] is None else _f32(l[3])
                keep += [ls, us, li, ui]
                arr[i].kind = 1
                arr[i].lower_slope, arr[i].upper_slope, arr[i].lower_intercept, arr[i].upper_intercept = _fp(ls), _fp(us), _fp(li), _fp(ui)
                arr[i].num_neurons = int(ls.shape[0])
            else:
                raise EngineError(UNSUPPORTED, f"layer kind {l[0]}")
        return arr

    def crown_backward(self, layers, spec, in_lo, in_hi, seed=None):
        """crown_backward_gpu_sound / _seeded_sound: backward-order layers with caller-baked slopes, one box.
        seed = (lower_a, upper_a, lower_b, upper_b) starts the pass from an asymmetric frontier.  Returns (lower, upper)."""
        keep = []
        arr = self._crown_layers(layers, keep)
        lo, hi = _f32(in_lo), _f32(in_hi)
        if seed is None:
            sp = _f32(spec)
            S = int(sp.shape[0])
            sd = None
        else:
            la, ua = _f32(seed[0]), _f32(seed[1])
            lb = None if seed[2] is None else _f32(seed[2])
            ub = None if seed[3] is None else _f32(seed[3])
            keep += [la, ua, lb, ub]
            S = int(la.shape[0])
            sd = CrownSeed(_fp(la), _fp(ua), _fp(lb), _fp(ub), S, int(la.shape[1]))
            sp = None
        ol, ou = np.empty(S, np.float32), np.empty(S, np.float32)
        fn = self._L.nyb200_crown_backward
        fn.argtypes = [C.c_void_p, C.POINTER(CrownLayer), C.c_int32, C.POINTER(C.c_float), C.c_int32, C.POINTER(CrownSeed),
                       C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]
        self._check(fn(self._h, arr, len(layers), _fp(sp), S, C.byref(sd) if sd is not None else None, _fp(lo), _fp(hi), _fp(ol), _fp(ou)))
        return ol, ou

    def _domain_refs(self, domains, keep):
        refs = (DomainRef * len(domains))()
        fpp = C.POINTER(C.c_float)
        for d, dom in enumerate(domains):
            arr = self._crown_layers(dom["layers"], keep)
            lo, hi = _f32(dom["lo"]), _f32(dom["hi"])
            n_act = len(dom["node_abs"])
            na = [_f32(a) for a in dom["node_abs"]]
            bs = [None if b is None else _f32(b) for b in dom.get("beta_signed", [None] * n_act)]
            na_p = (fpp * n_act)(*[_fp(a) for a in na])
            bs_p = (fpp * n_act)(*[_fp(b) for b in bs])
            sp = dom.get("splits")
            sp = None if sp is None else np.ascontiguousarray(sp, SPLIT_DTYPE)
            keep += [arr, lo, hi, na, bs, na_p, bs_p, sp]
            refs[d].layers = arr; refs[d].n_layers = len(dom["layers"])
            refs[d].input_lower, refs[d].input_upper = _fp(lo), _fp(hi)
            refs[d].beta_signed = bs_p; refs[d].frontier_abs = None; refs[d].node_abs = na_p
            refs[d].splits = None if sp is None else sp.ctypes.data
            refs[d].n_splits = 0 if sp is None else len(sp)
        return refs

    def crown_resnet_beta_batched(self, domains, spec):
        """crown_backward_gpu_resnet_sound_beta_batched for Chain networks: domains = list of dicts with layers (backward
        order, shared weight arrays), lo, hi, node_abs (fold order), beta_signed (fold order).  Returns (lower, upper) [D, S]."""
        keep = []
        refs = self._domain_refs(domains, keep)
        sp = _f32(spec)
        D, S = len(domains), int(sp.shape[0])
        ol, ou = np.empty((D, S), np.float32), np.empty((D, S), np.float32)
        fn = self._L.nyb200_crown_resnet_beta_batched
        fn.argtypes = [C.c_void_p, C.POINTER(DomainRef), C.c_int32, C.POINTER(C.c_float), C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        self._check(fn(self._h, refs, D, _fp(sp), S, _fp(ol), _fp(ou)))
        return ol, ou

    def crown_resnet_beta_batched_adam(self, domains, spec, iterations=3, beta_lr=0.05, beta1=0.9, beta2=0.999, epsilon=1e-8,
                                       tolerance=1e-5):
        """..._beta_batched_adam: as above plus `splits` per domain naming the multipliers to optimise.
        Returns (best lower, best upper, final beta [D, max_splits])."""
        keep = []
        refs = self._domain_refs(domains, keep)
        sp = _f32(spec)
        D, S = len(domains), int(sp.shape[0])
        ms = max([1] + [0 if d.get("splits") is None else len(d["splits"]) for d in domains])
        ol, ou, ob = np.empty((D, S), np.float32), np.empty((D, S), np.float32), np.zeros((D, ms), np.float32)
        cfg = BetaAdamConfig(iterations, beta_lr, beta1, beta2, epsilon, tolerance)
        fn = self._L.nyb200_crown_resnet_beta_batched_adam
        fn.argtypes = [C.c_void_p, C.POINTER(DomainRef), C.c_int32, C.POINTER(C.c_float), C.c_int32, C.POINTER(BetaAdamConfig),
                       C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int32]
        self._check(fn(self._h, refs, D, _fp(sp), S, C.byref(cfg), _fp(ol), _fp(ou), _fp(ob), ms))
        return ol, ou, ob

    def gemm_f64_triplet(self, m, k, n, a3, b3):
        """GemmEngine::gemm_f64_triplet: three same-shape binary64 products."""
        a3 = [np.ascontiguousarray(a, np.float64) for a in a3]
        b3 = [np.ascontiguousarray(b, np.float64) for b in b3]
        c3 = [np.empty((m, n), np.float64) for _ in range(3)]
        dp = C.POINTER(C.c_double)
        pa = (dp * 3)(*[a.ctypes.data_as(dp) for a in a3])
        pb = (dp * 3)(*[b.ctypes.data_as(dp) for b in b3])
        pc = (dp * 3)(*[c.ctypes.data_as(dp) for c in c3])
        fn = self._L.nyb200_gemm_f64_triplet
        fn.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, dp * 3, dp * 3, dp * 3]
        self._check(fn(self._h, m, k, n, pa, pb, pc))
        return c3

    def set_refine_tolerance(self, tol: float):
        self._check(self._L.nyb200_set_refine_tolerance(self._h, tol))

    def batch_poll(self):
        """Non-blocking: (newest run finished on the device, some run since the last finishing call flagged a domain
        for the binary64 re-evaluation - call batch_refined() then).  Raises on a latched pipeline error."""
        done, att = C.c_int32(0), C.c_int32(0)
        self._check(self._L.nyb200_batch_poll(self._h, C.byref(done), C.byref(att)))
        return bool(done.value), bool(att.value)

    def batch_refined(self) -> int:
        n = C.c_int32(0)
        self._check(self._L.nyb200_batch_refined(self._h, C.byref(n)))
        return int(n.value)

    def launch_count(self) -> int:
        return int(self._L.nyb200_launch_count(self._h))

    def clear_crown_working_set(self):
        self._check(self._L.nyb200_clear_working_set(self._h))

    # -- GemmEngine ------------------------------------------------------------------------
    def gemm_f32(self, m: int, k: int, n: int, a, b) -> np.ndarray:
        a, b = _f32(a).reshape(-1), _f32(b).reshape(-1)
        if a.size != m * k or b.size != k * n:
            raise EngineError(SHAPE, f"gemm_f32: expected {m * k} and {k * n} elements, got {a.size} and {b.size}")
        c = np.empty(m * n, np.float32)
        self._check(self._L.nyb200_gemm_f32(self._h, m, k, n, _fp(a), _fp(b), _fp(c)))
        return c.reshape(m, n)

    def gemm_f32_fast(self, m: int, k: int, n: int, a, b) -> np.ndarray:
        """GemmEngine::gemm_f32_fast: no precision contract (attack and scoring only); always the tensor-core product."""
        a, b = _f32(a).reshape(-1), _f32(b).reshape(-1)
        if a.size != m * k or b.size != k * n:
            raise EngineError(SHAPE, f"gemm_f32_fast: expected {m * k} and {k * n} elements, got {a.size} and {b.size}")
        c = np.empty(m * n, np.float32)
        self._check(self._L.nyb200_gemm_f32_fast(self._h, m, k, n, _fp(a), _fp(b), _fp(c)))
        return c.reshape(m, n)

    def gemm_f64(self, m: int, k: int, n: int, a, b) -> np.ndarray:
        """GemmEngine::gemm_f64: row-major binary64 product."""
        a = np.ascontiguousarray(a, np.float64).reshape(-1)
        b = np.ascontiguousarray(b, np.float64).reshape(-1)
        if a.size != m * k or b.size != k * n:
            raise EngineError(SHAPE, f"gemm_f64: got {a.size} and {b.size} values for {m}x{k} and {k}x{n}")
        c = np.empty(m * n, np.float64)
        dp = C.POINTER(C.c_double)
        self._check(self._L.nyb200_gemm_f64(self._h, m, k, n, a.ctypes.data_as(dp), b.ctypes.data_as(dp), c.ctypes.data_as(dp)))
        return c.reshape(m, n)

    def conv_transpose_2d(self, a_reshaped, weight_col, params: ConvTransposeParams) -> np.ndarray:
        """GemmEngine::conv_transpose_2d: a_reshaped [(S*OH*OW) x OC], weight_col [OC x IC*KH*KW] ->
        [S x IC*IH*IW]."""
        p = params
        a, w = _f32(a_reshaped).reshape(-1), _f32(weight_col).reshape(-1)
        if a.size != p.num_specs * p.out_h * p.out_w * p.out_channels:
            raise EngineError(SHAPE, "conv_transpose_2d: a_reshaped size")
        if w.size != p.out_channels * p.in_channels * p.kernel_h * p.kernel_w:
            raise EngineError(SHAPE, "conv_transpose_2d: weight_col size")
        out = np.empty((max(p.num_specs, 0), max(p.in_channels * p.in_h * p.in_w, 0)), np.float32)
        self._check(self._L.nyb200_conv_transpose_2d(self._h, _fp(a), _fp(w), C.byref(p), _fp(out)))
        return out

    def set_deadline(self, seconds_from_now: float | None):
        """GpuCrownBackward::set_crown_backward_deadline: None clears it."""
        ns = -1 if seconds_from_now is None else max(0, int(seconds_from_now * 1e9))
        self._check(self._L.nyb200_set_deadline_ns(self._h, ns))

    # -- network residency -----------------------------------------------------------------
    def register_network(self, net: Network) -> int:
        if net.has_conv or net.skips:
            return self._register_layers(net)
        w = np.concatenate([x.ravel() for x in net.weights]).astype(np.float32)
        bl = [b for b in net.biases if b is not None]
        b = np.concatenate(bl).astype(np.float32) if bl else np.zeros(1, np.float32)
        hb = np.array([0 if x is None else 1 for x in net.biases], np.int32)
        nid = C.c_int32(0)
        self._check(self._L.nyb200_net_create(self._h, len(net.weights), _ip(net.dims), _fp(w), _fp(b), _ip(hb),
                                              C.byref(nid)))
        self._nets[nid.value] = net
        return nid.value

    def _register_layers(self, net: Network) -> int:
        descs = (LayerDesc * len(net.weights))()
        ws, bs = [], []
        for k, w in enumerate(net.weights):
            if isinstance(w, Conv2d):
                descs[k] = w.desc()
                ws.append(w.weight.ravel())
            else:
                descs[k] = LayerDesc(0, w.shape[1], w.shape[0], 0 if net.biases[k] is None else 1)
                ws.append(w.ravel())
            descs[k].skip_from = net.skips.get(k, -1) + 1
            if net.biases[k] is not None:
                bs.append(net.biases[k])
        wf = np.concatenate(ws).astype(np.float32)
        bf = np.concatenate(bs).astype(np.float32) if bs else np.zeros(1, np.float32)
        nid = C.c_int32(0)
        self._check(self._L.nyb200_net_create_layers(self._h, len(net.weights), descs, _fp(wf), _fp(bf), C.byref(nid)))
        self._nets[nid.value] = net
        return nid.value

    def release_network(self, net_id: int):
        self._check(self._L.nyb200_net_destroy(self._h, net_id))
        self._nets.pop(net_id, None)

    # -- GpuIbpForward ---------------------------------------------------------------------
    def ibp_forward_gpu(self, net_id: int, in_lo, in_hi):
        """in_lo/in_hi: [n0] (one box) or [D, n0].  Returns pre-activation bounds [D, n_pre] x2."""
        net = self._nets[net_id]
        lo, hi = _f32(in_lo), _f32(in_hi)
        if lo.ndim == 1:
            lo, hi = lo[None, :], hi[None, :]
        D = lo.shape[0]
        if lo.shape != hi.shape or lo.shape[1] != net.dims[0]:
            raise EngineError(SHAPE, f"ibp_forward_gpu: box shape {lo.shape}")
        pl = np.empty((D, net.n_pre), np.float32)
        pu = np.empty((D, net.n_pre), np.float32)
        self._check(self._L.nyb200_ibp_forward(self._h, net_id, D, _fp(lo), _fp(hi), int(net.dims[0]), _fp(pl), _fp(pu)))
        return pl, pu

    def ibp_forward_noalloc(self, net_id: int, dev_in_lo: int, dev_in_hi: int, dev_pre_lo: int, dev_pre_hi: int):
        """Single-box interval forward pass on caller-owned DEVICE buffers (raw addresses); the library
        allocates nothing.  Linear layers without skips only; widths above 8192 are refused; concurrent calls on
        one GPU race."""
        self._check(self._L.nyb200_ibp_forward_noalloc(self._h, net_id, C.c_void_p(dev_in_lo), C.c_void_p(dev_in_hi),
                                                       C.c_void_p(dev_pre_lo), C.c_void_p(dev_pre_hi)))

    # -- batched beta-CROWN ----------------------------------------------------------------
    def _batch_args(self, net_id, spec, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits, mode, alpha):
        net = self._nets[net_id]
        spec = _f32(spec)
        if spec.ndim != 2 or spec.shape[1] != net.dims[-1]:
            raise EngineError(SHAPE, f"spec shape {spec.shape}, expected [S, {net.dims[-1]}]")
        lo, hi = _f32(in_lo), _f32(in_hi)
        splits = np.ascontiguousarray(splits, SPLIT_DTYPE)
        if splits.ndim != 2:
            raise EngineError(SHAPE, "splits must be [D, max_splits]")
        D, M = splits.shape
        n_splits = np.ascontiguousarray(n_splits, np.int32)
        if n_splits.shape != (D,):
            raise EngineError(SHAPE, "n_splits must be [D]")
        if lo.ndim == 1:
            stride = 0
            if lo.shape[0] != net.dims[0]:
                raise EngineError(SHAPE, "input box width")
        else:
            stride = int(net.dims[0])
            if lo.shape != (D, net.dims[0]):
                raise EngineError(SHAPE, "per-domain input box shape")
        inh_lo, inh_hi = _f32(inh_lo), _f32(inh_hi)
        if inh_lo.shape != (net.n_pre,) or inh_hi.shape != (net.n_pre,):
            raise EngineError(SHAPE, "inherited bounds must be [n_pre]")
        if alpha is not None:
            alpha = _f32(alpha)
            if alpha.shape != (D, net.n_pre):
                raise EngineError(SHAPE, "alpha must be [D, n_pre]")
        keep = (spec, lo, hi, inh_lo, inh_hi, splits, n_splits, alpha)
        args = [self._h, net_id, _fp(spec), spec.shape[0], _fp(lo), _fp(hi), stride, _fp(inh_lo), _fp(inh_hi),
                C.c_void_p(splits.ctypes.data), _ip(n_splits), M, D, mode, _fp(alpha)]
        return args, keep, D, spec.shape[0]

    def bab_bound_batch(self, net_id, spec, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits, mode=1, alpha=None):
        """Host buffers in, host buffers out: (lower [D,S], upper [D,S], infeasible [D])."""
        args, keep, D, S = self._batch_args(net_id, spec, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits, mode, alpha)
        ol, ou = np.empty((D, S), np.float32), np.empty((D, S), np.float32)
        inf = np.zeros(D, np.int32)
        self._check(self._L.nyb200_bab_bound_batch(*args, _fp(ol), _fp(ou), _ip(inf)))
        self._batch_shape = (D, S, self._nets[net_id].n_pre)
        self._batch_max_splits = int(np.asarray(splits).shape[1])
        return ol, ou, inf

    def batch_upload(self, net_id, spec, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits, mode=1, alpha=None):
        args, keep, D, S = self._batch_args(net_id, spec, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits, mode, alpha)
        self._check(self._L.nyb200_batch_upload(*args))
        self._batch_shape = (D, S, self._nets[net_id].n_pre)
        self._batch_max_splits = int(np.asarray(splits).shape[1])

    def batch_run(self):
        self._check(self._L.nyb200_batch_run(self._h))

    def crown_bounds(self, net_id, spec, in_lo, in_hi):
        """Plain CROWN with CROWN-IBP intermediate bounds.  in_lo/in_hi: [n0] (one box) or [D, n0].
        Returns (lower [D, S], upper [D, S], inter_lo [D, n_pre], inter_hi [D, n_pre])."""
        net = self._nets[net_id]
        spec, lo, hi = _f32(spec), _f32(in_lo), _f32(in_hi)
        if spec.ndim != 2 or spec.shape[1] != net.dims[-1]:
            raise EngineError(SHAPE, f"spec shape {spec.shape}")
        one = lo.ndim == 1
        D = 1 if one else lo.shape[0]
        if lo.shape != hi.shape or lo.shape[-1] != net.dims[0]:
            raise EngineError(SHAPE, "crown_bounds: box shape")
        S = spec.shape[0]
        ol, ou = np.empty((D, S), np.float32), np.empty((D, S), np.float32)
        il, iu = np.empty((D, net.n_pre), np.float32), np.empty((D, net.n_pre), np.float32)
        self._check(self._L.nyb200_crown_bounds(self._h, net_id, _fp(spec), S, _fp(lo), _fp(hi), 0 if one else int(net.dims[0]),
                                                D, _fp(ol), _fp(ou), _fp(il), _fp(iu)))
        return ol, ou, il, iu

    def crown_bounds_split(self, net_id, spec, in_lo, in_hi, splits, n_splits):
        """Plain CROWN with CROWN-IBP intermediate bounds for ReLU-split domains: in_lo/in_hi [n0] (one box shared by
        all domains) or [D, n0]; splits [D, max_splits] of SPLIT_DTYPE, n_splits [D].  Returns (lower [D, S],
        upper [D, S], inter_lo [D, n_pre], inter_hi [D, n_pre], infeasible [D])."""
        net = self._nets[net_id]
        spec, lo, hi = _f32(spec), _f32(in_lo), _f32(in_hi)
        ns = np.ascontiguousarray(n_splits, np.int32)
        D = len(ns)
        sp = np.ascontiguousarray(splits, SPLIT_DTYPE).reshape(D, -1)
        if spec.ndim != 2 or spec.shape[1] != net.dims[-1]:
            raise EngineError(SHAPE, f"spec shape {spec.shape}")
        shared = lo.ndim == 1
        if lo.shape != hi.shape or lo.shape[-1] != net.dims[0] or (not shared and lo.shape[0] != D):
            raise EngineError(SHAPE, "crown_bounds_split: box shape")
        S = spec.shape[0]
        ol, ou = np.empty((D, S), np.float32), np.empty((D, S), np.float32)
        il, iu = np.empty((D, net.n_pre), np.float32), np.empty((D, net.n_pre), np.float32)
        inf = np.zeros(D, np.int32)
        fn = self._L.nyb200_crown_bounds_split
        fn.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_float), C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_float),
                       C.c_int32, C.c_void_p, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.POINTER(C.c_float),
                       C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_int32)]
        self._check(fn(self._h, net_id, _fp(spec), S, _fp(lo), _fp(hi), 0 if shared else int(net.dims[0]), sp.ctypes.data,
                       ns.ctypes.data_as(C.POINTER(C.c_int32)), int(sp.shape[1]), D, _fp(ol), _fp(ou), _fp(il), _fp(iu),
                       inf.ctypes.data_as(C.POINTER(C.c_int32))))
        return ol, ou, il, iu, inf

    def batch_set_inherited(self, inh_lo, inh_hi):
        """Per-domain inherited bounds [D, n_pre] for the resident batch (see nyb200_batch_set_inherited)."""
        lo, hi = _f32(inh_lo), _f32(inh_hi)
        fn = self._L.nyb200_batch_set_inherited
        fn.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        self._check(fn(self._h, _fp(lo), _fp(hi)))

    def batch_set_thresholds(self, thresholds):
        """Verdict-only refinement for the uploaded batch: one threshold per specification row (None clears)."""
        fn = self._L.nyb200_batch_set_thresholds
        fn.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.c_int32]
        if thresholds is None:
            self._check(fn(self._h, None, 0))
            return
        t = _f32(thresholds).reshape(-1)
        self._check(fn(self._h, _fp(t), int(t.size)))

    def frontier_create(self, net_id, spec, thresholds, owner, n_clauses, in_lo, in_hi, inh_lo, inh_hi, max_depth, capacity):
        """Device-resident BaB frontier holding the root domain (see nyb200_frontier_create)."""
        spec, thr = _f32(spec), _f32(thresholds)
        own = np.ascontiguousarray(owner, np.int32)
        lo, hi, il, iu = _f32(in_lo), _f32(in_hi), _f32(inh_lo), _f32(inh_hi)
        fn = self._L.nyb200_frontier_create
        fp = C.POINTER(C.c_float)
        fn.argtypes = [C.c_void_p, C.c_int32, fp, fp, C.POINTER(C.c_int32), C.c_int32, C.c_int32, fp, fp, fp, fp, C.c_int32, C.c_int64]
        self._check(fn(self._h, net_id, _fp(spec), _fp(thr), own.ctypes.data_as(C.POINTER(C.c_int32)), int(spec.shape[0]),
                       int(n_clauses), _fp(lo), _fp(hi), _fp(il), _fp(iu), int(max_depth), int(capacity)))

    def frontier_round(self, batch: int, branching: int = 1):
        """One search round on the device.  Returns (bounded, verified, infeasible, stuck, open_after, deepest, min_lower)."""
        st = (C.c_int64 * 6)()
        ml = C.c_float(0)
        fn = self._L.nyb200_frontier_round
        fn.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_float)]
        self._check(fn(self._h, int(batch), int(branching), st, C.byref(ml)))
        return int(st[0]), int(st[1]), int(st[2]), int(st[3]), int(st[4]), int(st[5]), float(ml.value)

    def frontier_round_optimized(self, batch: int, branching: int, iterations: int, lr_alpha: float = 0.1, lr_beta: float = 0.05,
                                 lr_decay: float = 0.98, clip_beta: float = 10.0, objective: int = 0, rule: int = 0,
                                 tolerance: float = 0.0, patience: int = 0, start_save_best: float = 0.0):
        """frontier_round with `iterations` optimisation steps per domain (arguments as batch_optimize) and warm
        starts: children inherit their parent's optimised slopes and multipliers."""
        cfg = OptConfig(iterations, lr_alpha, lr_beta, lr_decay, 0.0, 0.0, 0.0, clip_beta, objective, rule, tolerance,
                        patience, start_save_best)
        st = (C.c_int64 * 6)()
        ml = C.c_float(0)
        fn = self._L.nyb200_frontier_round_optimized
        fn.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(OptConfig), C.POINTER(C.c_int64), C.POINTER(C.c_float)]
        self._check(fn(self._h, int(batch), int(branching), C.byref(cfg), st, C.byref(ml)))
        return int(st[0]), int(st[1]), int(st[2]), int(st[3]), int(st[4]), int(st[5]), float(ml.value)

    def frontier_set_refinement(self, verdict_only: bool):
        """Re-evaluate in binary64 only the domains whose verdict the rounding charge could change (True), or every
        domain whose charge is visible at the refinement tolerance (False, the default)."""
        fn = self._L.nyb200_frontier_set_refinement
        fn.argtypes = [C.c_void_p, C.c_int32]
        self._check(fn(self._h, 1 if verdict_only else 0))

    def frontier_count(self) -> int:
        n = C.c_int64(0)
        fn = self._L.nyb200_frontier_count
        fn.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        self._check(fn(self._h, C.byref(n)))
        return int(n.value)

    def frontier_take(self, n: int, dev_splits: int, dev_nsplits: int) -> int:
        """Moves up to n records from the back of the device frontier into device arrays given by address
        ([n, max_depth] split records of 16 bytes, [n] int32); returns how many left."""
        got = C.c_int64(0)
        fn = self._L.nyb200_frontier_take
        fn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
        self._check(fn(self._h, int(n), C.c_void_p(dev_splits), C.c_void_p(dev_nsplits), C.byref(got)))
        return int(got.value)

    def frontier_give(self, n: int, dev_splits: int, dev_nsplits: int):
        """Appends n records (device arrays by address, contents complete) at the back of the device frontier."""
        fn = self._L.nyb200_frontier_give
        fn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        self._check(fn(self._h, int(n), C.c_void_p(dev_splits), C.c_void_p(dev_nsplits)))

    def frontier_download(self, max_depth: int):
        """The open records in frontier order as host arrays (splits [n, max_depth], n_splits [n]); the frontier keeps
        them.  max_depth: the value the frontier was created with."""
        n = self.frontier_count()
        splits = np.zeros((n, max_depth), SPLIT_DTYPE)
        ns = np.zeros(n, np.int32)
        got = C.c_int64(0)
        fn = self._L.nyb200_frontier_download
        fn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
        self._check(fn(self._h, n, C.c_void_p(splits.ctypes.data), C.c_void_p(ns.ctypes.data), C.byref(got)))
        return splits, ns

    def frontier_upload(self, splits, n_splits):
        """Replaces the device frontier's contents by host records (splits [n, depth], n_splits [n])."""
        ns = np.ascontiguousarray(n_splits, np.int32)
        splits = np.asarray(splits, SPLIT_DTYPE)
        splits = np.ascontiguousarray(splits.reshape(len(ns), -1)) if len(ns) else np.zeros((0, 1), SPLIT_DTYPE)
        fn = self._L.nyb200_frontier_upload
        fn.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]
        self._check(fn(self._h, len(ns), int(splits.shape[1]) if len(ns) else 1, C.c_void_p(splits.ctypes.data), C.c_void_p(ns.ctypes.data)))

    def frontier_destroy(self):
        self._L.nyb200_frontier_destroy.argtypes = [C.c_void_p]
        self._L.nyb200_frontier_destroy.restype = None
        self._L.nyb200_frontier_destroy(self._h)

    def crown_input_coeffs(self, D: int, S: int, n0: int):
        """(lower_a, upper_a), each [D, S, n0]: input-level coefficients of the last crown_bounds call."""
        la, ua = np.empty((D, S, n0), np.float32), np.empty((D, S, n0), np.float32)
        self._check(self._L.nyb200_crown_input_coeffs(self._h, _fp(la), _fp(ua)))
        return la, ua

    def pgd_attack(self, net_id, spec, in_lo, in_hi, x0, steps: int, step_size: float, lr_decay: float = 0.99):
        """PGD batched over the K rows of x0 [K, n0]; returns (best objective per restart [K], best points [K, n0],
        index of the counterexample restart or -1).  The objective of a point is min_s spec[s] . f(x)."""
        net = self._nets[net_id]
        spec, lo, hi, x0 = _f32(spec), _f32(in_lo), _f32(in_hi), _f32(x0)
        if spec.ndim != 2 or spec.shape[1] != net.dims[-1]:
            raise EngineError(SHAPE, f"spec shape {spec.shape}")
        if x0.ndim != 2 or x0.shape[1] != net.dims[0] or lo.shape != (net.dims[0],) or hi.shape != lo.shape:
            raise EngineError(SHAPE, "pgd_attack: x0 must be [K, n0] and the box [n0]")
        K = x0.shape[0]
        best = np.empty(K, np.float32)
        bx = np.empty((K, int(net.dims[0])), np.float32)
        ce = C.c_int32(-1)
        cfg = PgdConfig(steps, step_size, lr_decay, 0.0, 0.0, 0.0)
        self._check(self._L.nyb200_pgd_attack(self._h, net_id, _fp(spec), spec.shape[0], _fp(lo), _fp(hi), _fp(x0), K,
                                              C.byref(cfg), _fp(best), _fp(bx), C.byref(ce)))
        return best, bx, int(ce.value)

    def batch_optimize(self, iterations: int, lr_alpha: float = 0.1, lr_beta: float = 0.05, lr_decay: float = 0.98,
                       clip_beta: float = 10.0, objective: int = 0, rule: int = 0, tolerance: float = 0.0, patience: int = 0,
                       start_save_best: float = 0.0):
        """alpha/beta optimisation of the resident batch (asynchronous); results through batch_download (element-wise
        best bounds) and batch_download_params.  rule: 0 projected Adam, 1 the reference's default plain projected
        step, 2 Adam with AMSGrad; tolerance / patience: the reference's per-domain stopping rules
        (beta_tolerance, early_stop_patience); start_save_best: the alpha loop's best-saving window."""
        cfg = OptConfig(iterations, lr_alpha, lr_beta, lr_decay, 0.0, 0.0, 0.0, clip_beta, objective, rule, tolerance,
                        patience, start_save_best)
        self._check(self._L.nyb200_batch_optimize(self._h, C.byref(cfg)))

    def batch_opt_evaluations(self) -> np.ndarray:
        """Bound evaluations every domain took part in before it stopped (== iterations when it never did)."""
        D = self._batch_shape[0]
        out = np.zeros(D, np.int32)
        self._check(self._L.nyb200_batch_download_opt_evaluations(self._h, _ip(out)))
        return out

    def batch_gradient(self, objective: int = 0) -> np.ndarray:
        """Joint gradient at the batch's current parameters, [D, n_pre]: d/d alpha on unstable unsplit neurons,
        d/d beta on split neurons, zero elsewhere.  The evaluation's bounds are then available through
        batch_download()."""
        D, S, n_pre = self._batch_shape
        g = np.empty((D, n_pre), np.float32)
        self._check(self._L.nyb200_batch_gradient(self._h, objective, _fp(g)))
        return g

    def point_vjp_batched(self, net_id: int, spec_rows, x=None, masks=None):
        """crown_point_vjp_batched: per-restart exact gradients spec_rows[k] . df/dx.  Give the points x [K, n0]
        (returns (grads, values)) or the 0/1 masks [K, n_pre] (returns grads)."""
        net = self._nets[net_id]
        spec_rows = _f32(spec_rows)
        K = spec_rows.shape[0]
        if spec_rows.ndim != 2 or spec_rows.shape[1] != net.dims[-1]:
            raise EngineError(SHAPE, f"spec_rows shape {spec_rows.shape}")
        grads = np.empty((K, int(net.dims[0])), np.float32)
        if x is not None and masks is None:
            x = _f32(x)
            if x.shape != (K, net.dims[0]):
                raise EngineError(SHAPE, "x must be [K, n0]")
            vals = np.empty(K, np.float32)
            self._check(self._L.nyb200_point_vjp_batched(self._h, net_id, K, _fp(x), None, _fp(spec_rows), _fp(grads), _fp(vals)))
            return grads, vals
        if masks is not None and x is None:
            masks = _f32(masks)
            if masks.shape != (K, net.n_pre):
                raise EngineError(SHAPE, "masks must be [K, n_pre]")
            self._check(self._L.nyb200_point_vjp_batched(self._h, net_id, K, None, _fp(masks), _fp(spec_rows), _fp(grads), None))
            return grads
        raise EngineError(INVALID, "exactly one of x and masks must be given")

    def batch_download_params(self):
        """(alpha [D, n_pre], beta [D, max_splits]) after the last run."""
        D, _, n_pre = self._batch_shape
        ms = self._batch_max_splits
        alpha = np.empty((D, n_pre), np.float32)
        beta = np.zeros((D, max(ms, 1)), np.float32)
        self._check(self._L.nyb200_batch_download_params(self._h, _fp(alpha), _fp(beta) if ms > 0 else None))
        return alpha, beta[:, :ms]

    def batch_download_alpha_upper(self):
        """The upper path's slopes [D, n_pre] after the last run (dual alpha)."""
        D, _, n_pre = self._batch_shape
        a = np.empty((D, n_pre), np.float32)
        self._check(self._L.nyb200_batch_download_alpha_upper(self._h, _fp(a)))
        return a

    def batch_download(self):
        D, S, _ = self._batch_shape
        ol, ou = np.empty((D, S), np.float32), np.empty((D, S), np.float32)
        inf = np.zeros(D, np.int32)
        self._check(self._L.nyb200_batch_download(self._h, _fp(ol), _fp(ou), _ip(inf)))
        return ol, ou, inf

    def batch_min_lower(self) -> float:
        v = C.c_float(0)
        self._check(self._L.nyb200_batch_min_lower(self._h, C.byref(v)))
        return float(v.value)

    def batch_min_lower_device(self) -> int:
        p = C.c_void_p()
        self._check(self._L.nyb200_batch_min_lower_device(self._h, C.byref(p)))
        return int(p.value)

    def batch_download_pre_bounds(self):
        D, _, n_pre = self._batch_shape
        pl, pu = np.empty((D, n_pre), np.float32), np.empty((D, n_pre), np.float32)
        self._check(self._L.nyb200_batch_download_pre_bounds(self._h, _fp(pl), _fp(pu)))
        return pl, pu

    def batch_verdicts(self, threshold: float = 0.0) -> np.ndarray:
        """Per-domain verdict of the last run: 0 unknown, 1 verified, 2 violated, 3 infeasible."""
        D = self._batch_shape[0]
        st = np.empty(D, np.int32)
        self._check(self._L.nyb200_batch_verdicts(self._h, threshold, _ip(st)))
        return st

    def batch_select_branch(self, kind: int = 0):
        """kind 0: largest width (sequential engine); 1: intercept score (batched graph engine)."""
        D = self._batch_shape[0]
        r, j, w = np.empty(D, np.int32), np.empty(D, np.int32), np.empty(D, np.float32)
        self._check(self._L.nyb200_batch_select_branch_scored(self._h, kind, _ip(r), _ip(j), _fp(w)))
        return r, j, w

    def batch_branch_scores(self, with_backup: bool = False):
        """Scores of the last BaBSR selection (batch_select_branch(2)), [D, n_pre]; -1 marks non-candidates.
        with_backup: also the intercept ("backup") scores, <= 0 for candidates and +1 otherwise."""
        D, S, n_pre = self._batch_shape
        sc = np.empty((D, n_pre), np.float32)
        bk = np.empty((D, n_pre), np.float32) if with_backup else None
        self._check(self._L.nyb200_batch_download_branch_scores(self._h, _fp(sc), _fp(bk)))
        return (sc, bk) if with_backup else sc

    def timing_enable(self, per_kernel: bool):
        self._check(self._L.nyb200_timing_enable(self._h, 1 if per_kernel else 0))

    def timing_reset(self):
        self._check(self._L.nyb200_timing_reset(self._h))

    def timing_read(self, phase: str):
        ms, n = C.c_double(0), C.c_int32(0)
        self._check(self._L.nyb200_timing_read(self._h, phase.encode(), C.byref(ms), C.byref(n)))
        return float(ms.value), int(n.value)
