//! B200 backend for ny's engine traits over the nyb200 C ABI (`include/nyb200.h`).
//!
//! NOT BUILT HERE: there is no Rust toolchain in this repository's build environment; the file is the binding a
//! maintainer adds as `crates/ny-b200`.  It implements the three traits the bound-propagation path dispatches
//! through (`crates/ny-core/src/gemm.rs`, `gemm_gpu_ibp.rs`):
//!   * `GemmEngine`        gemm_f32 / gemm_f32_fast / gemm_f64 / gemm_f64_triplet / conv_transpose_2d
//!   * `GpuIbpForward`     ibp_forward_gpu(_sound) for Linear / ReLU chains
//!   * `GpuCrownBackward`  crown_backward_gpu(_sound), _seeded(_sound), the resnet beta-batched calls for Chain
//!                         segments, the deadline and working-set hooks
//! Every method either returns the library's result or maps its status to the `NyError` variant the trait documents
//! (`UnsupportedOp` = decline, the caller falls back to CPU).  Registration is the CLI's factory seam
//! (`crates/ny-cli/src/main.rs:577-700`):
//!     sound_gpu_gate::set_wide_sound_gpu_crown_factory(Box::new(|| B200Engine::new(0).ok().map(|e| Arc::new(e) as _)));
#![allow(clippy::too_many_arguments)]

use std::ffi::{c_char, c_void, CStr};
use std::ptr;
use std::sync::Arc;

use ny_core::gemm::{
    ConvTranspose2dParams, GemmEngine, GpuBetaAdamConfig, GpuCrownBackward, GpuCrownLayer, GpuCrownResult, GpuCrownSeed,
    GpuResnetBatchedDomainRef, GpuResnetSegment,
};
use ny_core::gemm_gpu_ibp::{GpuIbpForward, GpuIbpLayer, GpuIbpResult};
use ny_core::{NyError, Result};

// ---------------------------------------------------------------------------------------------- FFI
#[repr(C)]
pub struct NyB200Engine {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy)]
struct CrownLayer {
    kind: i32,
    weight: *const f32,
    bias: *const f32,
    out_features: i32,
    in_features: i32,
    lower_slope: *const f32,
    upper_slope: *const f32,
    lower_intercept: *const f32,
    upper_intercept: *const f32,
    upper_neg_slope: *const f32,
    num_neurons: i32,
}

#[repr(C)]
struct CrownSeed {
    lower_a: *const f32,
    upper_a: *const f32,
    lower_b: *const f32,
    upper_b: *const f32,
    num_specs: i32,
    current_dim: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
struct Split {
    relu: i32,
    neuron: i32,
    sign: i32,
    beta: f32,
}

#[repr(C)]
struct DomainRef {
    layers: *const CrownLayer,
    n_layers: i32,
    input_lower: *const f32,
    input_upper: *const f32,
    beta_signed: *const *const f32,
    frontier_abs: *const *const f32,
    node_abs: *const *const f32,
    splits: *const Split,
    n_splits: i32,
}

#[repr(C)]
struct BetaAdamConfig {
    iterations: i32,
    beta_lr: f32,
    beta1: f32,
    beta2: f32,
    epsilon: f32,
    tolerance: f32,
}

#[repr(C)]
struct ConvTransposeParams {
    num_specs: i32,
    out_channels: i32,
    in_channels: i32,
    out_h: i32,
    out_w: i32,
    in_h: i32,
    in_w: i32,
    kernel_h: i32,
    kernel_w: i32,
    stride_h: i32,
    stride_w: i32,
    pad_h: i32,
    pad_w: i32,
}

extern "C" {
    fn nyb200_create(device_ordinal: i32, out: *mut *mut NyB200Engine) -> i32;
    fn nyb200_destroy(e: *mut NyB200Engine);
    fn nyb200_backend_provenance() -> *const c_char;
    fn nyb200_last_error(e: *const NyB200Engine) -> *const c_char;
    fn nyb200_clear_working_set(e: *mut NyB200Engine) -> i32;
    fn nyb200_use_own_stream(e: *mut NyB200Engine) -> i32;
    fn nyb200_set_deadline_ns(e: *mut NyB200Engine, ns_from_now: i64) -> i32;
    fn nyb200_gemm_f32(e: *mut NyB200Engine, m: i32, k: i32, n: i32, a: *const f32, b: *const f32, c: *mut f32) -> i32;
    fn nyb200_gemm_f32_fast(e: *mut NyB200Engine, m: i32, k: i32, n: i32, a: *const f32, b: *const f32, c: *mut f32) -> i32;
    fn nyb200_gemm_f64(e: *mut NyB200Engine, m: i32, k: i32, n: i32, a: *const f64, b: *const f64, c: *mut f64) -> i32;
    fn nyb200_gemm_f64_triplet(e: *mut NyB200Engine, m: i32, k: i32, n: i32, a: *const *const f64, b: *const *const f64,
                               c: *const *mut f64) -> i32;
    fn nyb200_conv_transpose_2d(e: *mut NyB200Engine, a: *const f32, w: *const f32, p: *const ConvTransposeParams, out: *mut f32) -> i32;
    fn nyb200_net_create(e: *mut NyB200Engine, n_linear: i32, dims: *const i32, wflat: *const f32, bflat: *const f32,
                         has_bias: *const i32, net_id: *mut i32) -> i32;
    fn nyb200_net_destroy(e: *mut NyB200Engine, net_id: i32) -> i32;
    fn nyb200_ibp_forward(e: *mut NyB200Engine, net_id: i32, d: i32, in_lo: *const f32, in_hi: *const f32, box_stride: i32,
                          pre_lo: *mut f32, pre_hi: *mut f32) -> i32;
    fn nyb200_crown_backward(e: *mut NyB200Engine, layers: *const CrownLayer, n_layers: i32, spec: *const f32, num_specs: i32,
                             seed: *const CrownSeed, in_lo: *const f32, in_hi: *const f32, out_lo: *mut f32, out_hi: *mut f32) -> i32;
    fn nyb200_crown_resnet_beta_batched(e: *mut NyB200Engine, domains: *const DomainRef, d: i32, spec: *const f32, num_specs: i32,
                                        out_lo: *mut f32, out_hi: *mut f32) -> i32;
    fn nyb200_crown_resnet_beta_batched_adam(e: *mut NyB200Engine, domains: *const DomainRef, d: i32, spec: *const f32, num_specs: i32,
                                             cfg: *const BetaAdamConfig, out_lo: *mut f32, out_hi: *mut f32, out_beta: *mut f32,
                                             max_splits: i32) -> i32;
}

// ---------------------------------------------------------------------------------------------- engine
/// One engine per GPU.  The library serialises the calls of a handle behind its own mutex (as ny-cuda does,
/// `crates/ny-cuda/src/lib.rs:1402-1420`), so `&self` methods from rayon workers are safe.
pub struct B200Engine {
    h: *mut NyB200Engine,
}
unsafe impl Send for B200Engine {}
unsafe impl Sync for B200Engine {}

impl B200Engine {
    pub fn new(device_ordinal: i32) -> Result<Self> {
        let mut h: *mut NyB200Engine = ptr::null_mut();
        let st = unsafe { nyb200_create(device_ordinal, &mut h) };
        if st != 0 || h.is_null() {
            return Err(NyError::UnsupportedOp("no usable sm_100 CUDA device for nyb200_create".into()));
        }
        Ok(Self { h })
    }

    /// An engine on a non-blocking stream of its own.  Several such engines on one GPU (one per worker thread, each with
    /// its own batches) overlap on the device: one batch's interval pass runs beside another's backward chain, one's
    /// transfers beside another's kernels (measured: 3 engines bound 4.1 M domains/s end to end where one bounds 3.3 M).
    pub fn with_own_stream(device_ordinal: i32) -> Result<Self> {
        let e = Self::new(device_ordinal)?;
        e.check(unsafe { nyb200_use_own_stream(e.h) })?;
        Ok(e)
    }

    /// Status code -> NyError (`crates/ny-core/src/error.rs:18`; codes in include/nyb200.h).
    fn check(&self, st: i32) -> Result<()> {
        if st == 0 {
            return Ok(());
        }
        let msg = unsafe { CStr::from_ptr(nyb200_last_error(self.h)) }.to_string_lossy().into_owned();
        Err(match st {
            1 => NyError::UnsupportedOp(msg),
            2 => NyError::shape_mismatch(vec![], vec![]),
            3 => NyError::InvalidSpec(msg),
            4 => NyError::NumericalInstability(msg),
            5 => NyError::DeadlineExceeded(msg),
            6 => NyError::CpuMemoryExceeded(msg),
            _ => NyError::InternalError(msg),
        })
    }
}

impl Drop for B200Engine {
    fn drop(&mut self) {
        unsafe { nyb200_destroy(self.h) }
    }
}

/// Flattens a backward-order `GpuCrownLayer` list into the C mirror.  The borrowed slices stay alive in the caller's
/// `layers` for the duration of the FFI call.  Kinds the library declines are passed through with their tag so that it
/// answers `UnsupportedOp` itself (one place decides what is supported).
fn c_layers(layers: &[GpuCrownLayer]) -> Vec<CrownLayer> {
    let null = ptr::null::<f32>();
    layers
        .iter()
        .map(|l| match l {
            GpuCrownLayer::Linear { weight, bias, out_features, in_features, .. } => CrownLayer {
                kind: 0,
                weight: weight.as_ptr(),
                bias: bias.as_ref().map_or(null, |b| b.as_ptr()),
                out_features: *out_features as i32,
                in_features: *in_features as i32,
                lower_slope: null, upper_slope: null, lower_intercept: null, upper_intercept: null, upper_neg_slope: null,
                num_neurons: 0,
            },
            GpuCrownLayer::Activation { lower_slope, upper_slope, lower_intercept, upper_intercept, num_neurons } => CrownLayer {
                kind: 1,
                weight: null, bias: null, out_features: 0, in_features: 0,
                lower_slope: lower_slope.as_ptr(),
                upper_slope: upper_slope.as_ptr(),
                lower_intercept: lower_intercept.as_ptr(),
                upper_intercept: upper_intercept.as_ptr(),
                upper_neg_slope: null,
                num_neurons: *num_neurons as i32,
            },
            GpuCrownLayer::ActivationReluDualAlpha { lower_pos_slope, cross_slope, upper_neg_slope, cross_intercept, num_neurons } => CrownLayer {
                kind: 3,
                weight: null, bias: null, out_features: 0, in_features: 0,
                lower_slope: lower_pos_slope.as_ptr(),
                upper_slope: cross_slope.as_ptr(),
                lower_intercept: null,
                upper_intercept: cross_intercept.as_ptr(),
                upper_neg_slope: upper_neg_slope.as_ptr(),
                num_neurons: *num_neurons as i32,
            },
            // declined by the library: Conv2d rows go through the registered-network batch calls instead
            GpuCrownLayer::Conv2d { .. } => CrownLayer { kind: 2, weight: null, bias: null, out_features: 0, in_features: 0,
                lower_slope: null, upper_slope: null, lower_intercept: null, upper_intercept: null, upper_neg_slope: null, num_neurons: 0 },
            GpuCrownLayer::MaxPool2d { .. } => CrownLayer { kind: -1, weight: null, bias: null, out_features: 0, in_features: 0,
                lower_slope: null, upper_slope: null, lower_intercept: null, upper_intercept: null, upper_neg_slope: null, num_neurons: 0 },
        })
        .collect()
}

impl GemmEngine for B200Engine {
    fn backend_provenance(&self) -> &'static str {
        // the library returns a pointer to a string literal
        unsafe { CStr::from_ptr(nyb200_backend_provenance()) }.to_str().unwrap_or("nyb200")
    }

    fn gemm_f32(&self, m: usize, k: usize, n: usize, a: &[f32], b: &[f32]) -> Result<Vec<f32>> {
        if a.len() != m * k || b.len() != k * n {
            return Err(NyError::shape_mismatch(vec![m, k, n], vec![a.len(), b.len()]));
        }
        let mut c = vec![0f32; m * n];
        self.check(unsafe { nyb200_gemm_f32(self.h, m as i32, k as i32, n as i32, a.as_ptr(), b.as_ptr(), c.as_mut_ptr()) })?;
        Ok(c)
    }

    /// No precision contract (attack / scoring only): always the tensor-core product.  `gemm_f32` above keeps the
    /// round-to-nearest error model the trait promises (the library takes its binary64-accumulating kernel for k < 21).
    fn gemm_f32_fast(&self, m: usize, k: usize, n: usize, a: &[f32], b: &[f32]) -> Result<Vec<f32>> {
        if a.len() != m * k || b.len() != k * n {
            return Err(NyError::shape_mismatch(vec![m, k, n], vec![a.len(), b.len()]));
        }
        let mut c = vec![0f32; m * n];
        self.check(unsafe { nyb200_gemm_f32_fast(self.h, m as i32, k as i32, n as i32, a.as_ptr(), b.as_ptr(), c.as_mut_ptr()) })?;
        Ok(c)
    }

    fn gemm_f64(&self, m: usize, k: usize, n: usize, a: &[f64], b: &[f64]) -> Result<Vec<f64>> {
        if a.len() != m * k || b.len() != k * n {
            return Err(NyError::shape_mismatch(vec![m, k, n], vec![a.len(), b.len()]));
        }
        let mut c = vec![0f64; m * n];
        self.check(unsafe { nyb200_gemm_f64(self.h, m as i32, k as i32, n as i32, a.as_ptr(), b.as_ptr(), c.as_mut_ptr()) })?;
        Ok(c)
    }

    fn gemm_f64_triplet(&self, m: usize, k: usize, n: usize, a: [&[f64]; 3], b: [&[f64]; 3]) -> Result<[Vec<f64>; 3]> {
        for i in 0..3 {
            if a[i].len() != m * k || b[i].len() != k * n {
                return Err(NyError::shape_mismatch(vec![m, k, n], vec![a[i].len(), b[i].len()]));
            }
        }
        let mut c = [vec![0f64; m * n], vec![0f64; m * n], vec![0f64; m * n]];
        let pa = [a[0].as_ptr(), a[1].as_ptr(), a[2].as_ptr()];
        let pb = [b[0].as_ptr(), b[1].as_ptr(), b[2].as_ptr()];
        let pc = [c[0].as_mut_ptr(), c[1].as_mut_ptr(), c[2].as_mut_ptr()];
        self.check(unsafe { nyb200_gemm_f64_triplet(self.h, m as i32, k as i32, n as i32, pa.as_ptr(), pb.as_ptr(), pc.as_ptr()) })?;
        Ok(c)
    }

    fn conv_transpose_2d(&self, a_reshaped: &[f32], weight_col: &[f32], p: &ConvTranspose2dParams) -> Result<Vec<f32>> {
        let cp = ConvTransposeParams {
            num_specs: p.num_specs as i32, out_channels: p.out_channels as i32, in_channels: p.in_channels as i32,
            out_h: p.out_h as i32, out_w: p.out_w as i32, in_h: p.in_h as i32, in_w: p.in_w as i32,
            kernel_h: p.kernel_h as i32, kernel_w: p.kernel_w as i32, stride_h: p.stride_h as i32, stride_w: p.stride_w as i32,
            pad_h: p.pad_h as i32, pad_w: p.pad_w as i32,
        };
        let mut out = vec![0f32; p.num_specs * p.in_channels * p.in_h * p.in_w];
        self.check(unsafe { nyb200_conv_transpose_2d(self.h, a_reshaped.as_ptr(), weight_col.as_ptr(), &cp, out.as_mut_ptr()) })?;
        Ok(out)
    }

    fn as_gpu_crown_backward(&self) -> Option<&dyn GpuCrownBackward> {
        Some(self)
    }

    fn as_gpu_ibp_forward(&self) -> Option<&dyn GpuIbpForward> {
        Some(self)
    }
}

impl GpuIbpForward for B200Engine {
    fn ibp_forward_gpu(&self, layers: &[GpuIbpLayer], lo: &[f32], hi: &[f32], shape: &[usize]) -> Result<GpuIbpResult> {
        self.ibp_forward_gpu_sound(layers, lo, hi, shape)
    }

    /// Linear / ReLU chains: the network is registered for the call (weights uploaded once per distinct list in a real
    /// deployment: keep the id in a cache keyed on the Arc pointers), the interval pass runs on the device with
    /// binary64 accumulation and outward casts, and the last layer's bounds are returned.
    fn ibp_forward_gpu_sound(&self, layers: &[GpuIbpLayer], lo: &[f32], hi: &[f32], _shape: &[usize]) -> Result<GpuIbpResult> {
        let mut dims: Vec<i32> = Vec::new();
        let (mut w, mut b, mut hb) = (Vec::<f32>::new(), Vec::<f32>::new(), Vec::<i32>::new());
        let mut expect_relu = false;
        for l in layers {
            match l {
                GpuIbpLayer::Linear { weight, bias, out_features, in_features } => {
                    if dims.is_empty() {
                        dims.push(*in_features as i32);
                    }
                    dims.push(*out_features as i32);
                    w.extend_from_slice(weight);
                    hb.push(bias.is_some() as i32);
                    if let Some(bv) = bias {
                        b.extend_from_slice(bv);
                    }
                    expect_relu = true;
                }
                GpuIbpLayer::ReLU { .. } if expect_relu => expect_relu = false,
                GpuIbpLayer::View { .. } => {}
                _ => return Err(NyError::UnsupportedOp("nyb200: this entry serves Linear/ReLU chains (Conv2d: register the network)".into())),
            }
        }
        if dims.len() < 2 || lo.len() != dims[0] as usize {
            return Err(NyError::shape_mismatch(vec![dims.first().copied().unwrap_or(0) as usize], vec![lo.len()]));
        }
        let mut id = 0i32;
        self.check(unsafe {
            nyb200_net_create(self.h, hb.len() as i32, dims.as_ptr(), w.as_ptr(), if b.is_empty() { ptr::null() } else { b.as_ptr() }, hb.as_ptr(), &mut id)
        })?;
        let n_pre: usize = dims[1..].iter().map(|&d| d as usize).sum();
        let (mut pl, mut pu) = (vec![0f32; n_pre], vec![0f32; n_pre]);
        let st = unsafe { nyb200_ibp_forward(self.h, id, 1, lo.as_ptr(), hi.as_ptr(), 0, pl.as_mut_ptr(), pu.as_mut_ptr()) };
        unsafe { nyb200_net_destroy(self.h, id) };
        self.check(st)?;
        let last = *dims.last().unwrap() as usize;
        Ok(GpuIbpResult { lower: pl[n_pre - last..].to_vec(), upper: pu[n_pre - last..].to_vec() })
    }

    fn provides_sound_gpu_ibp(&self) -> bool {
        true
    }
}

impl GpuCrownBackward for B200Engine {
    fn crown_backward_gpu(&self, layers: &[GpuCrownLayer], spec: &[f32], num_specs: usize, lo: &[f32], hi: &[f32]) -> Result<GpuCrownResult> {
        self.crown_backward_gpu_sound(layers, spec, num_specs, lo, hi)
    }

    fn crown_backward_gpu_sound(&self, layers: &[GpuCrownLayer], spec: &[f32], num_specs: usize, lo: &[f32], hi: &[f32]) -> Result<GpuCrownResult> {
        let cl = c_layers(layers);
        let (mut ol, mut ou) = (vec![0f32; num_specs], vec![0f32; num_specs]);
        self.check(unsafe {
            nyb200_crown_backward(self.h, cl.as_ptr(), cl.len() as i32, spec.as_ptr(), num_specs as i32, ptr::null(), lo.as_ptr(), hi.as_ptr(),
                                  ol.as_mut_ptr(), ou.as_mut_ptr())
        })?;
        Ok(GpuCrownResult { lower_bounds: ol, upper_bounds: ou })
    }

    fn provides_sound_gpu_crown(&self) -> bool {
        true
    }

    fn crown_backward_gpu_seeded(&self, layers: &[GpuCrownLayer], seed: &GpuCrownSeed, lo: &[f32], hi: &[f32]) -> Result<GpuCrownResult> {
        self.crown_backward_gpu_seeded_sound(layers, seed, lo, hi)
    }

    fn crown_backward_gpu_seeded_sound(&self, layers: &[GpuCrownLayer], seed: &GpuCrownSeed, lo: &[f32], hi: &[f32]) -> Result<GpuCrownResult> {
        let cl = c_layers(layers);
        let cs = CrownSeed {
            lower_a: seed.lower_a.as_ptr(), upper_a: seed.upper_a.as_ptr(), lower_b: seed.lower_b.as_ptr(), upper_b: seed.upper_b.as_ptr(),
            num_specs: seed.num_specs as i32, current_dim: seed.current_dim as i32,
        };
        let (mut ol, mut ou) = (vec![0f32; seed.num_specs], vec![0f32; seed.num_specs]);
        self.check(unsafe {
            nyb200_crown_backward(self.h, cl.as_ptr(), cl.len() as i32, ptr::null(), seed.num_specs as i32, &cs, lo.as_ptr(), hi.as_ptr(),
                                  ol.as_mut_ptr(), ou.as_mut_ptr())
        })?;
        Ok(GpuCrownResult { lower_bounds: ol, upper_bounds: ou })
    }

    /// Chain networks only: a segment list with a Residual / ResidualProj member is declined (the registered-network
    /// batch calls serve identity skips).  The seed of this call is the symmetric spec matrix (zero bias).
    fn crown_backward_gpu_resnet_sound_beta_batched(&self, domains: &[GpuResnetBatchedDomainRef<'_>], seed: &GpuCrownSeed) -> Result<Vec<GpuCrownResult>> {
        let s = seed.num_specs;
        let mut keep_layers: Vec<Vec<CrownLayer>> = Vec::with_capacity(domains.len());
        let mut keep_ptrs: Vec<(Vec<*const f32>, Vec<*const f32>)> = Vec::with_capacity(domains.len());
        for d in domains {
            let chain = match d.segments {
                [GpuResnetSegment::Chain(layers)] => layers,
                _ => return Err(NyError::UnsupportedOp("nyb200: beta-batched serves single Chain segments".into())),
            };
            keep_layers.push(c_layers(chain));
            keep_ptrs.push((d.beta_signed.iter().map(|v| v.as_ptr()).collect(), d.node_abs.iter().map(|v| v.as_ptr()).collect()));
        }
        let refs: Vec<DomainRef> = domains
            .iter()
            .enumerate()
            .map(|(i, d)| DomainRef {
                layers: keep_layers[i].as_ptr(),
                n_layers: keep_layers[i].len() as i32,
                input_lower: d.input_lower.as_ptr(),
                input_upper: d.input_upper.as_ptr(),
                beta_signed: keep_ptrs[i].0.as_ptr(),
                frontier_abs: ptr::null(),
                node_abs: keep_ptrs[i].1.as_ptr(),
                splits: ptr::null(),
                n_splits: 0,
            })
            .collect();
        let (mut ol, mut ou) = (vec![0f32; domains.len() * s], vec![0f32; domains.len() * s]);
        self.check(unsafe {
            nyb200_crown_resnet_beta_batched(self.h, refs.as_ptr(), refs.len() as i32, seed.lower_a.as_ptr(), s as i32, ol.as_mut_ptr(), ou.as_mut_ptr())
        })?;
        Ok((0..domains.len())
            .map(|i| GpuCrownResult { lower_bounds: ol[i * s..(i + 1) * s].to_vec(), upper_bounds: ou[i * s..(i + 1) * s].to_vec() })
            .collect())
    }

    fn set_crown_backward_deadline(&self, deadline: Option<std::time::Instant>) {
        let ns = deadline.map_or(-1, |d| d.saturating_duration_since(std::time::Instant::now()).as_nanos() as i64);
        unsafe { nyb200_set_deadline_ns(self.h, ns) };
    }

    fn honors_crown_backward_deadline(&self) -> bool {
        true
    }

    fn clear_crown_working_set(&self) {
        unsafe { nyb200_clear_working_set(self.h) };
    }
}

/// The `_adam` form needs the sparse beta mapping next to the domain refs (`GpuBetaAdamParams`,
/// `crates/ny-core/src/gemm.rs:3014-3090`); a maintainer fills `splits` of every `DomainRef` from its
/// `GpuBetaAdamMapping` list (relu index converted from fold order to forward order: `n_relu - 1 - relu_index`) and
/// calls `nyb200_crown_resnet_beta_batched_adam` with `BetaAdamConfig::from(cfg)`.
impl From<&GpuBetaAdamConfig> for BetaAdamConfig {
    fn from(c: &GpuBetaAdamConfig) -> Self {
        BetaAdamConfig { iterations: c.iterations as i32, beta_lr: c.beta_lr, beta1: c.beta1, beta2: c.beta2, epsilon: c.epsilon, tolerance: c.tolerance }
    }
}

#[allow(dead_code)]
fn _keep(_: *const c_void, _: Arc<()>) {}
