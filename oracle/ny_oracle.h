/*
 * ny_oracle.h -- CPU restatement of ny's bound-propagation path (TEST INFRASTRUCTURE).
 *
 * This library is the parity checker and the timed CPU baseline.  It is never part of
 * the product path: only the test-suite, the smoke check and the benchmark's CPU legs
 * may load it.  Every function cites the reference source (path inside the ny project)
 * whose arithmetic it restates.  The reference is Rust and cannot be compiled in this
 * environment, so this restatement is pinned against the golden values of the
 * reference's own tests (crates/ny-propagate/src/tests/crown/reference.rs).
 *
 * Network model: a sequential ReLU MLP
 *     x -> Linear_0 -> ReLU -> Linear_1 -> ReLU -> ... -> Linear_{L-1}
 * dims[0..L] are the widths; weights are row-major [dims[k+1] x dims[k]] concatenated in
 * `wflat`; biases are concatenated in `bflat` (has_bias[k]==0 means the layer has none and
 * contributes no entries to bflat).  A layer may instead be a Conv2d (see conv_geom): the interval
 * pass and the backward pass then walk the kernel taps directly (im2col order of
 * layers/convolution/conv2d/ops_ibp_fwd.rs and the transposed convolution of conv2d/bound.rs:601-900),
 * which is the reference's algorithm rather than a dense lowering of it.
 */
#ifndef NY_ORACLE_H
#define NY_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int32_t n_linear;        /* L */
    const int32_t *dims;     /* L+1 */
    const float *wflat;
    const float *bflat;
    const int32_t *has_bias; /* L */
    const int32_t *relu_after; /* L entries or NULL (= a ReLU after every Linear but the last);
                                  relu_after[k]==0 means Linear_k feeds Linear_{k+1} directly, which is
                                  how ny's CLI appends specification rows as a final Linear layer */
    const int32_t *conv_geom;  /* NULL (all layers dense) or L blocks of 12 ints
                                  (ic, ih, iw, oc, oh, ow, kh, kw, sh, sw, ph, pw); a block of zeros marks a
                                  dense layer.  A Conv2d layer (NCHW flattened, dilation 1, one group) stores
                                  its kernel [oc x ic*kh*kw] in wflat and a per-channel bias [oc] in bflat;
                                  dims[k] = ic*ih*iw, dims[k+1] = oc*oh*ow.  Supported by the interval pass,
                                  plain CROWN, the beta-CROWN bound and the batch entry points; the gradient
                                  and optimisation entry points return -2 for such a network. */
    const int32_t *skip_from;  /* NULL or L entries: skip_from[k] = j >= 0 adds the post-activation output of layer j
                                  (j <= k - 2, same width) to layer k's output before its ReLU,
                                  pre_k = W_k z + b_k + relu(pre_j): the identity branch of a residual block
                                  (GpuResnetSegment::Residual, crates/ny-core/src/gemm.rs:1640-1669); -1 = none.
                                  Supported by nyo_domain_bounds (mode 1), nyo_beta_crown_bound and the batch entry
                                  point; the other entry points return -2 for such a network. */
} nyo_net;

/* A split constraint on ReLU `relu` (0-based, the ReLU that follows Linear_relu),
 * neuron `neuron`; sign +1 = active (pre-activation >= 0), -1 = inactive. */
typedef struct {
    int32_t relu;
    int32_t neuron;
    int32_t sign;
    float beta;
} nyo_split;

/* scalar helpers (exported for unit tests) */
float nyo_next_up_f32(float x);
float nyo_next_down_f32(float x);
double nyo_certified_affine_sum(float bias, const float *coef, const float *val, int n, int upper);

/* IBP forward: writes pre-activation bounds of every Linear layer, concatenated
 * (sum_{k=1..L} dims[k] floats each).  Returns 0. */
int nyo_ibp_forward(const nyo_net *net, const float *in_lo, const float *in_hi,
                    float *pre_lo, float *pre_hi);

/* Plain CROWN of the sequential engine: IBP, CROWN-IBP intermediate tightening,
 * final backward from identity, concretize, intersect with the forward bound.
 * out_lo/out_hi have dims[L] entries.  If inter_lo/inter_hi are non-NULL they receive the
 * tightened pre-activation bounds (same layout as nyo_ibp_forward). */
int nyo_crown(const nyo_net *net, const float *in_lo, const float *in_hi,
              float *out_lo, float *out_hi, float *inter_lo, float *inter_hi);
/* nyo_crown for a ReLU-split domain (clamps on every layer's tightened bound, multipliers at zero); 1 = infeasible. */
int nyo_crown_split(const nyo_net *net, const float *in_lo, const float *in_hi, const nyo_split *splits, int n_splits,
                    float *out_lo, float *out_hi, float *inter_lo, float *inter_hi);

/* beta-CROWN bound of one BaB domain given its pre-activation bounds
 * (layout as nyo_ibp_forward, only the first L-1 blocks are read), its split list, and
 * per-neuron lower slopes alpha (concatenated over the L-1 ReLUs; NULL = the
 * heuristic [u > -l]).  out_lo/out_hi have dims[L] entries. */
int nyo_beta_crown_bound(const nyo_net *net, const float *in_lo, const float *in_hi,
                         const float *pre_lo, const float *pre_hi,
                         const nyo_split *splits, int n_splits, const float *alpha,
                         float *out_lo, float *out_hi);

/* Per-domain intermediate bounds under a split history.
 * mode 0 ("clamp only", sequential engine): copy the inherited bounds and clamp the split neurons.
 * mode 1 ("constrained forward", graph engine): additionally re-propagate interval bounds
 * downstream and keep the tighter of inherited / re-propagated per element.
 * Returns 1 if the domain is infeasible (a clamp inverted an interval), else 0. */
int nyo_domain_bounds(const nyo_net *net, const float *in_lo, const float *in_hi,
                      const float *inh_lo, const float *inh_hi,
                      const nyo_split *splits, int n_splits, int mode,
                      float *pre_lo, float *pre_hi);

/* Batch driver (a thread pool over domains): nyo_domain_bounds + nyo_beta_crown_bound for D
 * domains sharing net, input box and inherited bounds.  splits is [D x max_splits],
 * n_splits[d] valid entries each.  out_* are [D x dims[L]]; infeasible[d] is set to 1
 * (and the bounds to +inf/-inf... i.e. lower=+inf, upper=-inf) for empty domains.
 * Returns the number of threads used. */
int nyo_bab_bound_batch(const nyo_net *net, const float *in_lo, const float *in_hi,
                        const float *inh_lo, const float *inh_hi,
                        const nyo_split *splits, const int32_t *n_splits, int max_splits,
                        int D, int mode, float *out_lo, float *out_hi, int32_t *infeasible,
                        int n_threads);

/* Lower bounds of the spec rows (binary64, no outward rounding) and the joint gradient of their sum with
 * respect to alpha (n_pre layout, zero for stable or split neurons) and to every split's beta. */
int nyo_joint_gradient(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                       const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                       double *lower_out, float *grad_alpha, float *grad_beta);

/* 1 (default): the certified per-coefficient error channel of the plain-CROWN path is discharged, as in the
 * reference; 0: it is left out (test use: isolates the error chain from the bound). */
void nyo_set_error_channel(int on);
int nyo_joint_gradient_rows(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                            const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                            double *lower_out, float *grad_alpha, float *grad_beta, int only_row);
int nyo_optimize_objective(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                           const float *pre_hi, nyo_split *splits, int n_splits, float *alpha, int iterations,
                           float lr_alpha, float lr_beta, float lr_decay, float clip_beta, int objective, float *best_lo,
                           float *best_hi);
int nyo_beta_crown_bound_dual(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                              const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                              const float *alpha_up, float *out_lo, float *out_hi);
int nyo_upper_gradient(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                       const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                       const float *alpha_up, double *upper_out, float *grad_alpha_up);
int nyo_optimize_dual(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                      const float *pre_hi, nyo_split *splits, int n_splits, float *alpha, int iterations,
                      float lr_alpha, float lr_beta, float lr_decay, float clip_beta, int objective, float *best_lo,
                      float *best_hi, float *alpha_up_out);
/* The same loop with the reference's other update and stopping rules (see the definition). */
typedef struct {
    int32_t iterations;
    float lr_alpha, lr_beta, lr_decay, clip_beta;
    int32_t objective;       /* 0 sum of the rows, 1 smallest row, 2 dual alpha */
    int32_t rule;            /* 0 Adam, 1 plain projected step (the reference default), 2 Adam + AMSGrad */
    float tolerance;         /* > 0: stop when max |gradient| < tolerance */
    int32_t patience;        /* > 0: stop after more than `patience` iterations without improvement */
    float start_save_best;   /* in (0,1): best bounds updated at iteration 0 and after iterations * this */
} nyo_opt_cfg;
int nyo_optimize_ex(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                    const float *pre_hi, nyo_split *splits, int n_splits, float *alpha, const nyo_opt_cfg *cfg,
                    float *best_lo, float *best_hi, float *alpha_up_out, int *iterations_run);
int nyo_select_intercept(const nyo_net *net, const float *pre_lo, const float *pre_hi, const nyo_split *splits,
                         int n_splits, int32_t *relu, int32_t *neuron, float *score);

/* Projected-Adam optimisation of alpha (in [0,1]) and beta (>= 0) with fixed intermediate bounds; keeps the
 * element-wise best sound bounds.  alpha and the beta fields of `splits` are updated in place. */
int nyo_optimize(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo, const float *pre_hi,
                 nyo_split *splits, int n_splits, float *alpha, int iterations, float lr_alpha, float lr_beta,
                 float lr_decay, float clip_beta, float *best_lo, float *best_hi);

/* Largest-width branching choice (first maximum wins, NaN skipped).
 * Returns 1 and fills relu/neuron if an unstable unsplit neuron exists, else 0. */
int nyo_select_largest_width(const nyo_net *net, const float *pre_lo, const float *pre_hi,
                             const nyo_split *splits, int n_splits,
                             int32_t *relu, int32_t *neuron, float *width);

/* Verdict predicates (lower mode): verified iff finite and lower > threshold. */
int nyo_domain_verified(float lower, float upper, float threshold);
int nyo_domain_violated(float lower, float upper, float threshold);

#ifdef __cplusplus
}
#endif
#endif
