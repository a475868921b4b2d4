/*
 * nyb200.h -- C ABI of the B200 (sm_100a) bound-propagation engine.
 *
 * Every entry point takes plain pointers and sizes and returns an int32 status; no C++ or
 * framework types cross this boundary.  The functions are what a Rust (or any FFI) binding of
 * ny's engine plugin traits would bind; each comment names the reference interface it stands in
 * for (paths inside the ny project).  Host pointers unless a comment says "device".
 *
 * Threading: an engine handle serialises its own calls (as ny-cuda does behind a mutex,
 * crates/ny-cuda/src/lib.rs:1402-1420); distinct handles are independent.
 *
 * There is no CPU fallback: a call on a machine without a usable CUDA device fails with
 * NYB200_ERR_UNSUPPORTED from nyb200_create and nothing else can be called.
 */
#ifndef NYB200_H
#define NYB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: one per ny_core::NyError variant the engine boundary uses
 * (crates/ny-core/src/error.rs:18).  UNSUPPORTED is a decline, never fatal. */
#define NYB200_OK 0
#define NYB200_ERR_UNSUPPORTED 1 /* NyError::UnsupportedOp      */
#define NYB200_ERR_SHAPE 2       /* NyError::ShapeMismatch      */
#define NYB200_ERR_INVALID 3     /* NyError::InvalidSpec        */
#define NYB200_ERR_NUMERICAL 4   /* NyError::NumericalInstability */
#define NYB200_ERR_DEADLINE 5    /* NyError::DeadlineExceeded   */
#define NYB200_ERR_OOM 6         /* NyError::CpuMemoryExceeded / device allocation failure */
#define NYB200_ERR_INTERNAL 7    /* NyError::InternalError      */

typedef struct nyb200_engine nyb200_engine;

/* One ReLU split of a BaB domain: `relu` is the 0-based index of the ReLU layer (the one
 * after Linear_relu), `neuron` its flat neuron index, `sign` +1 active / -1 inactive and
 * `beta` the Lagrange multiplier (>= 0).  Mirrors NeuronConstraint + BetaEntry
 * (crates/ny-propagate/src/beta_crown/state/beta.rs:20-40). */
typedef struct {
    int32_t relu;
    int32_t neuron;
    int32_t sign;
    float beta;
} nyb200_split;

/* Arithmetic used for the A*W contraction of the backward pass. */
#define NYB200_PATH_F64 0   /* binary64 FMA accumulation of exact fp32 products */
#define NYB200_PATH_TF32X3 1 /* tcgen05 3xTF32 split products, chunked TMEM accumulators */

/* ---- lifecycle ---------------------------------------------------------------------------
 * Engine construction/provenance: GemmEngine::backend_provenance (crates/ny-core/src/gemm.rs:313)
 * and the CLI's factory seams (crates/ny-cli/src/main.rs:577-700). */
int32_t nyb200_create(int32_t device_ordinal, nyb200_engine **out);
void nyb200_destroy(nyb200_engine *e);
const char *nyb200_backend_provenance(void);
const char *nyb200_last_error(const nyb200_engine *e);
/* Launch all work of this engine on the given cudaStream_t (NULL = the default stream). */
int32_t nyb200_set_stream(nyb200_engine *e, void *cuda_stream);
/* Gives the engine a non-blocking stream of its own (created on first use, destroyed with the engine) and makes it the
 * engine's stream.  Several engines on one GPU, each with its own stream and its own batches, overlap on the device:
 * batches are independent, so one batch's latency-bound interval pass runs beside another's tensor-bound chain, and
 * one's transfers beside another's kernels (ny_b200/pool.py drives that; the reference's counterpart is its per-thread
 * engine handles, crates/ny-core/src/gemm.rs:568-578). */
int32_t nyb200_use_own_stream(nyb200_engine *e);
/* The persistent kernels (one CTA per SM, tiles dealt out statically) leave n SMs unused.  For callers that run a
 * collective on another stream beside them (the per-round min-reduce of a sharded search): a collective's CTA that
 * takes an SM keeps one CTA of a full-width persistent kernel waiting until another retires, which stretches that
 * kernel by its whole per-CTA share.  Default 0. */
int32_t nyb200_set_reserved_sms(nyb200_engine *e, int32_t n);
/* Programmatic dependent launch of the engine's kernels (default on): a kernel is scheduled while its predecessor in
 * the stream is still running and waits for it after its own set-up, which hides launch latency, CTA scheduling and
 * tensor-memory allocation (1 % of a step with one batch in flight).  With several engines on one GPU it costs more than
 * it gives: the early CTAs of a full-width kernel hold their SMs while they wait, and another engine's kernel that
 * could have run there does not (three batches in flight: 0.957 ms per step without against 0.973 ms with).
 * ny_b200/pool.py switches it off for pools of more than one engine. */
int32_t nyb200_set_launch_overlap(nyb200_engine *e, int32_t on);
/* Select the contraction arithmetic (NYB200_PATH_*).  Default NYB200_PATH_TF32X3; NYB200_PATH_F64 is the
 * slower binary64 reference arithmetic on the same device. */
int32_t nyb200_set_path(nyb200_engine *e, int32_t path);
/* Layer fusion of the NYB200_PATH_TF32X3 backward pass.  On (default): where the network allows it (Linear layers
 * without skips, hidden widths <= 256 and multiples of 4) the contractions of all hidden layers and their ReLU
 * relaxations run as one kernel that keeps a tile of coefficient rows on the SM from the specification rows down to
 * the first layer's input; only the first layer's (wide) contraction and the concretisation follow as separate
 * launches.  Off: one contraction launch and one relaxation launch per layer.  Both compute the same quantities
 * with the same per-coefficient arithmetic; they differ in the accumulation order of the tensor-core sums (and its
 * certified rounding charge), i.e. by a few ulps of the coefficients.  No counterpart in the reference, whose
 * engines launch per layer (crates/ny-cuda/src/sound_crown.rs:348-376). */
int32_t nyb200_set_fusion(nyb200_engine *e, int32_t on);
/* Adaptive precision of the NYB200_PATH_TF32X3 path.  Every rounding of that path is charged to the
 * bounds as a penalty; when, for some domain of a batch, that penalty exceeds `tol` times
 * max(|bound|, 1% of the domain's largest bound) -- which happens for narrow boxes, where a bound is much
 * smaller than the terms it is made of -- the batch is evaluated again with binary64 contractions before
 * results are returned, so the returned bounds stay within the parity tolerance of the reference's
 * binary64 CPU path.  Default 5e-5; 0 disables the re-run (bounds remain sound, only looser).
 * nyb200_batch_refined reports how many domains of the last run triggered it (0 = fast path only). */
int32_t nyb200_set_refine_tolerance(nyb200_engine *e, float tol);
int32_t nyb200_batch_refined(nyb200_engine *e, int32_t *n_domains);
/* ---- device-resident BaB frontier (the "resident frontier" extension; no counterpart in the reference's traits, whose
 * search loop keeps its domains on the host: crates/ny-propagate/src/beta_crown/engine/core.rs:492-735).
 * nyb200_frontier_create: the open set starts as the root domain (no splits).  spec [S x out], thresholds [S] and
 * owner [S] (the clause a row belongs to, 0 .. n_clauses-1; S <= 64, n_clauses <= 32): a domain is decided when it is
 * infeasible or when every clause has a row whose lower bound exceeds its threshold.  in_lo / in_hi: the shared box;
 * inh_lo / inh_hi [sum_{k>=1} dims[k]]: inherited (root) pre-activation bounds.  max_depth: longest split history the
 * ring can hold; capacity: domains.
 * nyb200_frontier_round: pops up to `batch` domains from the front, bounds them (constrained forward pass, one bound
 * per domain, multipliers zero), decides, picks the split neuron of every open domain with the given score
 * (NYB200_BRANCH_*), appends both children at the back (active child first).  stats_out [6]: bounded, verified,
 * infeasible, stuck (undecided with no neuron left: the batch then stays in the frontier and nothing is appended),
 * open domains afterwards, deepest history bounded; *min_lower the smallest lower bound among the round's feasible
 * domains.  The order of domains is the host loop's, so a search through these calls bounds the same domains. */
int32_t nyb200_frontier_create(nyb200_engine *e, int32_t net_id, const float *spec, const float *thresholds,
                               const int32_t *owner, int32_t S, int32_t n_clauses, const float *in_lo, const float *in_hi,
                               const float *inh_lo, const float *inh_hi, int32_t max_depth, int64_t capacity);
int32_t nyb200_frontier_round(nyb200_engine *e, int32_t batch, int32_t branching, int64_t *stats_out, float *min_lower);
void nyb200_frontier_destroy(nyb200_engine *e);
/* The same round with every domain's slopes and split multipliers optimised (cfg as for nyb200_batch_optimize; declared
 * below) and warm starts: the children inherit the parent's optimised slopes (kept in a ring of [capacity x neurons]
 * floats that the first such round allocates) and carry its optimised multipliers in their split records; a batch
 * starts warm when every one of its domains has slopes of its own (the rule of the host loop, ny_b200/bab.py, which
 * follows beta_crown/engine/core.rs:600-700).  Records that arrive through nyb200_frontier_give / _upload have none. */
struct nyb200_opt_config;
int32_t nyb200_frontier_round_optimized(nyb200_engine *e, int32_t batch, int32_t branching, const struct nyb200_opt_config *cfg,
                                        int64_t *stats_out, float *min_lower);
/* Which domains of a round are re-evaluated with binary64 contractions.  0 (default): the engine's rule (every domain
 * whose rounding charge is visible at nyb200_set_refine_tolerance, so that the bounds stay within the parity bar of the
 * binary64 path).  1: only the domains whose verdict the charge could change - some row's certified lower bound misses
 * its threshold by less than twice the row's charge; the others keep the tensor-path bound, which is sound and at most
 * that charge looser.  The search's verdict is sound either way; with 1 a domain may be split once more than with 0.
 * Applies to the frontier that exists when it is called. */
int32_t nyb200_frontier_set_refinement(nyb200_engine *e, int32_t verdict_only);
/* Sharded search (one process per GPU, each with its own frontier): the shards are levelled by moving records between
 * them, device array to device array (the caller carries them with a point-to-point collective; the reference's
 * domain distribution is host-side, beta_crown/engine/core.rs:560-640).  nyb200_frontier_take removes up to n records
 * from the back of the ring into dev_splits [n x max_depth] (nyb200_split) and dev_nsplits [n], both device memory of
 * this engine's GPU, complete on return; nyb200_frontier_give appends n such records (their contents must be complete:
 * synchronise the stream or collective that wrote them first).  nyb200_frontier_count: open domains held. */
int32_t nyb200_frontier_count(nyb200_engine *e, int64_t *open);
int32_t nyb200_frontier_take(nyb200_engine *e, int64_t n, void *dev_splits, int32_t *dev_nsplits, int64_t *taken);
int32_t nyb200_frontier_give(nyb200_engine *e, int64_t n, const void *dev_splits, const int32_t *dev_nsplits);
/* Dump and resume (the reference's search has no checkpoint; its benchmark sweep resumes from metadata).
 * nyb200_frontier_download copies the open records, front first, into host arrays splits [capacity x max_depth] and
 * nsplits [capacity] and reports their number (call with capacity 0 to learn it); the frontier keeps them.
 * nyb200_frontier_upload replaces the frontier's contents by n host records of row length depth <= max_depth. */
int32_t nyb200_frontier_download(nyb200_engine *e, int64_t capacity, nyb200_split *splits, int32_t *nsplits, int64_t *n_out);
int32_t nyb200_frontier_upload(nyb200_engine *e, int64_t n, int32_t depth, const nyb200_split *splits, const int32_t *nsplits);
/* Non-blocking look at the runs launched so far (no counterpart in the reference, whose calls return finished
 * results): every nyb200_batch_run ends with a one-thread kernel that publishes, to mapped host memory, the run's
 * sequence number, the tensor pipeline's error word and the number of domains flagged for the binary64 re-run.
 * *completed = 1 when the newest run has finished on the device; *attention = 1 when any run since the last
 * finishing call (download, nyb200_batch_refined, ...) flagged a domain - the caller then calls
 * nyb200_batch_refined, which synchronises and re-evaluates; a latched pipeline error is returned as
 * NYB200_ERR_INTERNAL.  A resident loop that launches round after round calls this instead of synchronising each
 * round and learns of a flagged round one or two rounds late, never not at all. */
int32_t nyb200_batch_poll(nyb200_engine *e, int32_t *completed, int32_t *attention);
/* Number of kernels this engine has launched since creation (bench bookkeeping). */
int64_t nyb200_launch_count(const nyb200_engine *e);
/* GpuCrownBackward::clear_crown_working_set (crates/ny-core/src/gemm.rs:3205). */
int32_t nyb200_clear_working_set(nyb200_engine *e);

/* ---- GemmEngine::gemm_f32 (crates/ny-core/src/gemm.rs:325): C[m,n] = A[m,k] * B[k,n], row-major.
 * The trait's precision contract (:318-324) is the error model of round-to-nearest fp32 arithmetic,
 * |c - a.b| <= gamma_k sum|a||b|: on NYB200_PATH_TF32X3 the tcgen05 3xTF32 product is used where its certified rate is
 * below gamma_k (k >= 21), the binary64-accumulating kernel for shorter contractions and on NYB200_PATH_F64.
 * nyb200_gemm_f32_fast is GemmEngine::gemm_f32_fast (:337, no precision contract, attack and scoring only): always the
 * tensor-core product on NYB200_PATH_TF32X3.  gemm_interval_sound (:663) stays the trait's default over gemm_f32. */
int32_t nyb200_gemm_f32(nyb200_engine *e, int32_t m, int32_t k, int32_t n, const float *a, const float *b,
                        float *c_out);
int32_t nyb200_gemm_f32_fast(nyb200_engine *e, int32_t m, int32_t k, int32_t n, const float *a, const float *b,
                             float *c_out);

/* ---- network residency -------------------------------------------------------------------
 * Stands in for the Arc<[f32]> pointer-identity cache key of GpuCrownLayer::Linear
 * (crates/ny-core/src/gemm.rs:1524-1547): weights are uploaded once and named by an id.
 * Sequential ReLU MLP: dims[0..n_linear]; weights row-major [dims[k+1] x dims[k]] concatenated;
 * has_bias[k]==0 layers contribute nothing to bflat. */
int32_t nyb200_net_create(nyb200_engine *e, int32_t n_linear, const int32_t *dims, const float *wflat,
                          const float *bflat, const int32_t *has_bias, int32_t *net_id);
/* Sequential network of Linear and Conv2d layers, every layer but the last followed by a ReLU: the
 * Linear / Conv2d members of GpuCrownLayer (crates/ny-core/src/gemm.rs:1524-1600) and of the IBP layer
 * enum (crates/ny-core/src/gemm_gpu_ibp.rs:31-67).  Tensors are NCHW flattened; a Conv2d layer has
 * dilation 1 and one group, weights W_col [out_channels x in_channels*kernel_h*kernel_w] row-major and an
 * optional per-channel bias [out_channels] (expanded on the device).  A Linear layer has weights
 * [out_features x in_features] and bias [out_features].  A global average pool followed by a Linear layer is
 * registered as that one Linear layer with the pool folded into its weights (W[i][c] / (H*W) repeated over the
 * pixels: the backward broadcast A/(H*W) of layers/pooling/average.rs:347,457).  wflat / bflat concatenate the layers in order;
 * layer k's in_features must equal layer k-1's out_features (= out_channels*out_h*out_w for a conv). */
#define NYB200_LAYER_LINEAR 0
#define NYB200_LAYER_CONV2D 1
typedef struct nyb200_layer_desc {
    int32_t kind;
    int32_t in_features, out_features;
    int32_t has_bias;
    /* Conv2d only (ConvTranspose2dParams, crates/ny-core/src/gemm.rs:150-178) */
    int32_t in_channels, in_h, in_w, out_channels, out_h, out_w;
    int32_t kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w;
    /* Residual connection (GpuResnetSegment::Residual, crates/ny-core/src/gemm.rs:1640-1669): 0 = none;
     * j + 1 = the post-activation output of layer j (j <= this layer - 2, same width as this layer's output)
     * is added to this layer's output before its ReLU: pre = W z + b + relu(pre_j).  Blocks may nest, overlap
     * or start at the same layer.  A projection block (ResidualProj, :1658-1669) is registered as the sequential
     * layers the host mirror's lower_projection_block produces.  Supported by the interval pass, the bound batch entry points, the parameter optimisation and the
     * attack, and the CROWN-IBP pipeline. */
    int32_t skip_from;
} nyb200_layer_desc;
int32_t nyb200_net_create_layers(nyb200_engine *e, int32_t n_layers, const nyb200_layer_desc *layers,
                                 const float *wflat, const float *bflat, int32_t *net_id);
int32_t nyb200_net_destroy(nyb200_engine *e, int32_t net_id);

/* ---- GpuIbpForward::ibp_forward_gpu_sound (crates/ny-core/src/gemm_gpu_ibp.rs:78-135) ------
 * Interval forward pass for D boxes.  in_lo/in_hi are [D x dims[0]] (box_stride = dims[0]) or a
 * single shared box (box_stride = 0).  pre_lo/pre_hi receive the pre-activation bounds of every
 * Linear layer, [D x sum_{k>=1} dims[k]]. */
int32_t nyb200_ibp_forward(nyb200_engine *e, int32_t net_id, int32_t D, const float *in_lo, const float *in_hi,
                           int32_t box_stride, float *pre_lo, float *pre_hi);

/* ---- beta-CROWN bound of a batch of BaB domains --------------------------------------------
 * One call = for every domain: intermediate bounds under its splits, alpha/beta ReLU relaxation,
 * CROWN backward of the spec rows, concretisation on the input box.  It fuses the host
 * preparation and the engine call of process_gpu_batched Phase 2
 * (crates/ny-propagate/src/beta_crown/engine/graph/gpu_bab/batched_gpu.rs:89,
 *  engine/graph/propagation/batched.rs:1695-1708 ->
 *  GpuCrownBackward::crown_backward_gpu_resnet_sound_beta_batched, crates/ny-core/src/gemm.rs:3944)
 * and returns what compute_bounds_with_alpha_beta returns per domain
 * (crates/ny-propagate/src/beta_crown/engine/optimization/bound_compute.rs:90).
 *
 *   spec          [S x dims[L]] specification rows (appended as a bias-free Linear layer by ny's CLI)
 *   in_lo/in_hi   input box, shared (box_stride 0) or per domain (box_stride dims[0])
 *   inh_lo/inh_hi inherited pre-activation bounds [sum_{k>=1} dims[k]] (root or parent bounds)
 *   splits        [D x max_splits], n_splits[d] valid entries per domain
 *   mode          0 clamp-only intermediate bounds (sequential engine, engine/domain/child.rs:51-118)
 *                 1 constrained forward re-propagation (graph engine, constraints/mod.rs:184-760)
 *   alpha         NULL (heuristic [u > -l]) or lower slopes laid out like the pre-activation bounds,
 *                 [D x sum_{k>=1} dims[k]] (the last layer's block is ignored)
 *   out_lo/out_hi [D x S]; an infeasible domain gets lower=+inf, upper=-inf and infeasible[d]=1
 */
int32_t nyb200_bab_bound_batch(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                               const float *in_hi, int32_t box_stride, const float *inh_lo, const float *inh_hi,
                               const nyb200_split *splits, const int32_t *n_splits, int32_t max_splits, int32_t D,
                               int32_t mode, const float *alpha, float *out_lo, float *out_hi,
                               int32_t *infeasible);

/* ---- plain CROWN with CROWN-IBP intermediate bounds ---------------------------------------------
 * GpuCrownBackward::crown_backward_gpu_sound(layers, spec, num_specs, in_lo, in_hi)
 * (crates/ny-core/src/gemm.rs:3357) with the intermediate bounds the reference's `crown` pipeline collects
 * (crates/ny-propagate/src/network/core/sequential/crown.rs:168-330, network/ibp/crown_ibp.rs:32-420): every
 * layer that feeds a ReLU is bounded by a partial CROWN pass with the plain-CROWN relaxation
 * (activations/relu/mod.rs:105-132) and merged with its IBP and forward bounds; the spec rows are bounded by
 * the full pass and tightened (crown/tighten.rs:126-190).  D boxes in lock-step: in_lo/in_hi [D x dims[0]]
 * with box_stride = dims[0], or one box with box_stride = 0 and D = 1.  out_lo/out_hi [D x S];
 * inter_lo/inter_hi (may be NULL) receive the tightened pre-activation bounds [D x sum_{k>=1} dims[k]].
 * Linear and Conv2d layers, identity skips included. */
int32_t nyb200_crown_bounds(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                            const float *in_hi, int32_t box_stride, int32_t D, float *out_lo, float *out_hi,
                            float *inter_lo, float *inter_hi);
/* The same pipeline for ReLU-split BaB domains (the per-domain CROWN-tightened intermediate bounds that the graph
 * engine's constrained forward pass stands in for, crates/ny-propagate/src/beta_crown/engine/graph/propagation/
 * beta.rs:921-929; collection as above): D domains, one shared box (box_stride = 0) or one box each, every domain with
 * its own split list.  The interval pass runs under the domains' clamps, every layer's tightened bound is clamped
 * (active l = max(l, 0), inactive u = min(u, 0)) before its relaxation is taken, the split multipliers are ignored
 * (plain CROWN carries none).  infeasible [D]: 1 where a clamp empties an interval (bounds of such a domain are
 * meaningless).  inter_lo / inter_hi are what a caller hands to nyb200_batch_set_inherited to bound the same domains
 * with tighter relaxations.  Costs one partial pass of 2 n_k rows per domain and hidden layer: a tool for hundreds of
 * domains, not for the 4096-domain batch.  Default error convention only. */
int32_t nyb200_crown_bounds_split(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                                  const float *in_hi, int32_t box_stride, const nyb200_split *splits,
                                  const int32_t *n_splits, int32_t max_splits, int32_t D, float *out_lo, float *out_hi,
                                  float *inter_lo, float *inter_hi, int32_t *infeasible);
/* Convention for the certified rounding error of nyb200_crown_bounds.
 *   NYB200_ERRCH_IMMEDIATE (default): every rounding is discharged at the layer where it occurs, against the interval
 *     of the variable the coefficient multiplies.  Sound and tighter than the reference on deep networks (by about
 *     2e-3 of the bound at depth 6), hence NOT identical to it there.
 *   NYB200_ERRCH_REFERENCE: the reference's own channel - a per-coefficient error matrix
 *     err' = |cast| + gamma_K |A||W| + err |W| carried through every layer (LinearBounds::lower_a_err / upper_a_err,
 *     crates/ny-propagate/src/bounds/linear.rs:320-347; layers/linear/crown_single.rs:2092-2103; ReLU carry
 *     layers/common/crown_dense.rs:41-290) and discharged at the input box (bounds/concretize.rs:443-466), in
 *     binary64 whatever nyb200_set_path says.  Returns the reference's CPU CROWN bounds to within 1e-4 relative.
 *     Linear layers without residual connections only (NYB200_ERR_UNSUPPORTED otherwise). */
#define NYB200_ERRCH_IMMEDIATE 0
#define NYB200_ERRCH_REFERENCE 1
int32_t nyb200_set_error_channel(nyb200_engine *e, int32_t mode);
/* Input-level linear coefficients of the last nyb200_crown_bounds call (LinearBounds::lower_a / upper_a of the
 * reference's CROWN result, used by the input-split heuristic, beta_crown/engine/input_split.rs:111-260):
 * lower_a / upper_a [D x S x dims[0]], either may be NULL.  The rows stay on the device only until the next call
 * that uses the batch workspace (upload, attack, another CROWN call); after that NYB200_ERR_INVALID. */
int32_t nyb200_crown_input_coeffs(nyb200_engine *e, float *lower_a, float *upper_a);

/* ---- resident batch (extension: keeps the domain batch in HBM between calls) ----------------
 * upload copies the same arguments as nyb200_bab_bound_batch to the device; run launches the
 * whole bound evaluation asynchronously on the engine stream with no host<->device traffic;
 * download copies the results back (synchronises the stream).  The reference keeps operands
 * resident only within one call (crates/ny-core/src/gemm.rs:568-578); this is the frontier
 * residency a BaB driver needs to reach the memory roofline. */
int32_t nyb200_batch_upload(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                            const float *in_hi, int32_t box_stride, const float *inh_lo, const float *inh_hi,
                            const nyb200_split *splits, const int32_t *n_splits, int32_t max_splits, int32_t D,
                            int32_t mode, const float *alpha);
/* Verdict-only refinement for the uploaded batch (the per-batch counterpart of nyb200_frontier_set_refinement, for
 * search loops that keep their domains on the host): with thresholds [S] set, the runs of this batch re-evaluate in
 * binary64 only the domains in which some row's certified lower bound misses its threshold by less than twice the
 * row's rounding charge; all other bounds stay the tensor path's (sound, at most that charge looser than the binary64
 * path's).  NULL clears it; the next nyb200_batch_upload clears it too.  No counterpart in the reference, whose device
 * paths carry their error bounds without a binary64 re-evaluation. */
int32_t nyb200_batch_set_thresholds(nyb200_engine *e, const float *thresholds, int32_t S);
/* Per-domain inherited bounds for the resident batch: inh_lo / inh_hi [D x sum_{k>=1} dims[k]] replace the shared
 * vector given at upload (e.g. the tightened intermediates of nyb200_crown_bounds_split for the same domains).  The
 * next run intersects every domain's re-propagated bounds with its own row (mode 1) or takes the row as it is (mode
 * 0).  No counterpart in the reference's trait, whose domain references carry their bounds as baked slopes. */
int32_t nyb200_batch_set_inherited(nyb200_engine *e, const float *inh_lo, const float *inh_hi);
int32_t nyb200_batch_run(nyb200_engine *e);
int32_t nyb200_batch_download(nyb200_engine *e, float *out_lo, float *out_hi, int32_t *infeasible);
/* Smallest lower bound over all feasible domains and rows of the last run (the per-round global
 * lower bound that the multi-GPU driver min-reduces).  Synchronises the stream. */
int32_t nyb200_batch_min_lower(nyb200_engine *e, float *min_lower);
/* Device pointer to that value (float, valid until the next run) for an in-stream collective. */
int32_t nyb200_batch_min_lower_device(nyb200_engine *e, void **dev_ptr);
/* Pre-activation bounds of the last run, [D x sum_{k>=1} dims[k]] (what BabDomain::layer_bounds
 * holds, crates/ny-propagate/src/beta_crown/domain.rs). */
int32_t nyb200_batch_download_pre_bounds(nyb200_engine *e, float *pre_lo, float *pre_hi);
/* Largest-width branching choice per domain of the last run (first maximum wins, NaN skipped,
 * split neurons excluded): select_largest_width_neuron,
 * crates/ny-propagate/src/beta_crown/engine/branching/sequential.rs:49-104.
 * relu[d] = -1 when the domain has no unstable unsplit neuron. */
int32_t nyb200_batch_select_branch(nyb200_engine *e, int32_t *relu, int32_t *neuron, float *width);
/* Same with the score chosen: NYB200_BRANCH_WIDTH (u - l, the sequential engine's default, as above) or
 * NYB200_BRANCH_INTERCEPT ((-l*u)/(u-l) in fp32: PickedDomains::select_branch_batched,
 * crates/ny-propagate/src/batched_domain/domain_list/picked.rs:153-233).  `score` receives the winning value. */
#define NYB200_BRANCH_WIDTH 0
#define NYB200_BRANCH_INTERCEPT 1
/* NYB200_BRANCH_BABSR: the BaBSR score (select_babsr_neuron / compute_babsr_scores,
 * beta_crown/engine/branching/sequential.rs:106-198,784-882; score kernel branching/score.rs:28-97): per domain the
 * specification rows are carried backwards through the Linear layers with the ReLUs' upper slopes, and a neuron's score is
 * the mean over rows of |min(b c (r0 - 1), b c r0) + min(c, 0) r1| with r0 = max(u,0)/(max(u,0) - min(l,0)),
 * r1 = -min(l,0) r0, b the producing layer's bias.  Linear layers only (NYB200_ERR_UNSUPPORTED otherwise).
 * nyb200_batch_download_branch_scores returns the scores of the last BaBSR selection, [D x n_pre], -1 for neurons that
 * are not candidates (stable or split) and for the output block; backup (may be NULL) receives the "backup" score
 * of the filtered heuristics (select_fsb_neuron, sequential.rs:200-358), the mean intercept term min(c, 0) r1 (<= 0;
 * +1 for non-candidates). */
#define NYB200_BRANCH_BABSR 2
int32_t nyb200_batch_select_branch_scored(nyb200_engine *e, int32_t kind, int32_t *relu, int32_t *neuron, float *score);
int32_t nyb200_batch_download_branch_scores(nyb200_engine *e, float *scores, float *backup);

/* ---- alpha/beta optimisation of the resident batch ---------------------------------------------
 * Projected-Adam ascent on every domain's lower slopes alpha (unstable unsplit neurons, kept in [0,1]:
 * update_alphas_adam, crates/ny-propagate/src/bounds/alpha/shared.rs:106-146) and split multipliers beta
 * (kept >= 0, gradient clipped: crates/ny-propagate/src/beta_crown/state/beta.rs:314-441), with the
 * intermediate bounds of the uploaded batch fixed, all domains in lock-step on the device
 * (the role of crown_backward_gpu_resnet_sound_beta_batched_adam and crown_joint_alpha_gradient_resident,
 * crates/ny-core/src/gemm.rs:4042,4095).  Iteration t evaluates the sound bounds with the current
 * parameters, folds them into the element-wise best (network/alpha_crown_loop.rs:928-936), then - except
 * on the last iteration - steps along the joint gradient of sum_s lower[d][s]
 * (crates/ny-core/src/joint_alpha_grad.rs:22-50) with learning rate lr * lr_decay^(t-1).
 * iterations = 1 is exactly nyb200_batch_run.  Asynchronous on the engine stream; nyb200_batch_download
 * then returns the best bounds, nyb200_batch_download_params the final parameters.  On the fast path,
 * when the last iterate's rounding charge is visible at nyb200_set_refine_tolerance, the final parameters
 * are evaluated once more with binary64 contractions and folded into the best bounds. */
typedef struct nyb200_opt_config {
    int32_t iterations;  /* >= 1 */
    float lr_alpha;      /* 0 freezes alpha */
    float lr_beta;       /* 0 freezes beta */
    float lr_decay;      /* per-iteration factor, the reference uses 0.98 */
    float beta1, beta2, epsilon; /* Adam moments; zeros select 0.9, 0.999, 1e-8 */
    float clip_beta;     /* > 0: beta gradients are clipped to [-clip, clip] (reference: 10) */
    int32_t objective;   /* 0: sum over the spec rows of the lower bounds (joint_alpha_gradient);
                            1: the row whose current lower bound is smallest (optimize_joint_bounds,
                            beta_crown/engine/optimization/optimize_loop.rs:77-333);
                            2: dual alpha (ReLULayer::propagate_linear_with_alpha,
                            activations/relu/mod.rs:570-1128): as 0, and the upper rows get their own slopes
                            alpha_up for negative coefficients, started at alpha and descending the sum of the
                            upper bounds */
    int32_t rule;        /* update rule of alpha and beta.  0: projected Adam (above).
                            1: the plain projected step that is the reference's default (use_adaptive = false):
                               beta <- max(0, beta + lr g) (BetaState::gradient_step, beta_crown/state/beta.rs:272-305),
                               alpha <- clamp(alpha + lr g, 0, 1); no moments, no gradient clip.
                            2: Adam with AMSGrad's running maximum of the second moment (beta.rs:369-376; the resident
                               contract GpuBetaAdamConfig, crates/ny-core/src/gemm.rs:2960-2993) */
    float tolerance;     /* > 0: a domain stops once max |gradient| over its parameters (clipped beta gradients, raw
                            alpha gradients) is below it: the reference's beta_tolerance
                            (beta_crown/engine/optimization/optimize_loop.rs:272-279).  Evaluated per domain on the device;
                            a stopped domain keeps its parameters while the others continue in lock-step. */
    int32_t patience;    /* > 0: a domain stops once its objective's best value has not improved for more than `patience`
                            iterations (patience_exhausted_after_iteration, optimize_loop.rs:45-57) */
    float start_save_best; /* in (0, 1): the element-wise best bounds are only updated at the first iteration, after
                            iterations * start_save_best iterations and at the last one, and for a domain that has
                            stopped (AlphaCrownConfig::should_save_best, bounds/alpha_config.rs:1085-1091, used at
                            network/alpha_crown_loop.rs:928-936; the reference's 0.5).  0: every iteration. */
} nyb200_opt_config;
int32_t nyb200_batch_optimize(nyb200_engine *e, const nyb200_opt_config *cfg);
/* After nyb200_batch_optimize: evaluations[d] = number of bound evaluations domain d took part in before it stopped
 * (tolerance or patience), the stopping iteration's update included; equal to `iterations` for a domain that never
 * stopped.  A stop takes effect after the update of its iteration; the parameters it leaves are evaluated once more
 * and folded into the best bounds (the reference returns without that evaluation: this can only be tighter). */
int32_t nyb200_batch_download_opt_evaluations(nyb200_engine *e, int32_t *evaluations);
/* alpha [D x sum_{k>=1} dims[k]] (meaningful on unstable unsplit neurons) and beta [D x max_splits]
 * (same order as the uploaded split lists) after the last run.  Either pointer may be NULL. */
int32_t nyb200_batch_download_params(nyb200_engine *e, float *alpha, float *beta);
/* The upper path's slopes [D x sum_{k>=1} dims[k]] after the last run (equal to alpha unless objective 2 ran). */
int32_t nyb200_batch_download_alpha_upper(nyb200_engine *e, float *alpha_up);

/* ---- PGD attack batched over restarts ----------------------------------------------------------
 * All K restarts advance in lock-step (PgdAttacker::attack_batched,
 * crates/ny-propagate/src/pgd_attack/attacker/batched.rs:33-215) with the exact gradient of the objective
 * (the role of crown_point_vjp_batched, crates/ny-core/src/gemm.rs:4180-4222).  The property holds where every
 * row spec[s] . f(x) > 0; a restart's objective is its smallest row (the worst conjunct,
 * ny-cli commands/beta_crown/verify/graph_pgd.rs:655-685), which the attack minimises.  Step rule
 * (AdamClippingState::step, pgd_attack/adam_state.rs:46-88): Adam moments of the gradient, direction
 * sign(m / (sqrt(v / bc2) + epsilon)) with sign(+0) = +1 and 0 for non-finite values, uniform step
 * step_size * lr_decay^(t-1) / bc1, projection onto the box (NaN -> lower end).  x0 [K x dims[0]] are the
 * starting points (the caller draws them; the reference seeds one generator per restart).  Every step's point
 * competes for the restart's best objective; after the last step the best point of every restart is evaluated
 * once more with binary64 contractions and that value is what is returned ("re-validated by an independent
 * forward").  Outputs: best_margin [K], best_x [K x dims[0]] (may be NULL), *counterexample = index of the
 * restart with the smallest validated objective if that objective is <= 0, else -1.
 * The attack can only produce counterexample candidates; it never affects a bound. */
typedef struct nyb200_pgd_config {
    int32_t steps;
    float step_size;              /* initial L-inf step (config 5 uses 0.25 * eps) */
    float lr_decay;               /* per-step factor; 0 selects the reference's 0.99 */
    float beta1, beta2, epsilon;  /* zeros select 0.9, 0.999, 1e-8 */
} nyb200_pgd_config;
int32_t nyb200_pgd_attack(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                          const float *in_hi, const float *x0, int32_t K, const nyb200_pgd_config *cfg,
                          float *best_margin, float *best_x, int32_t *counterexample);

/* ---- verdicts of the last run ------------------------------------------------------------------
 * Per domain, lower mode (the property holds where every spec row stays above `threshold`), with the reference's
 * predicates (domain_is_verified_for_mode / domain_is_violation_for_mode,
 * crates/ny-propagate/src/beta_crown/config/beta_config.rs:1552-1610): VERIFIED when every row has finite,
 * non-inverted bounds and lower > threshold (strict); VIOLATED when some row has finite, non-inverted bounds and
 * upper < threshold; INFEASIBLE for an empty domain; UNKNOWN otherwise (a non-finite threshold verifies and
 * violates nothing). */
#define NYB200_VERDICT_UNKNOWN 0
#define NYB200_VERDICT_VERIFIED 1
#define NYB200_VERDICT_VIOLATED 2
#define NYB200_VERDICT_INFEASIBLE 3
int32_t nyb200_batch_verdicts(nyb200_engine *e, float threshold, int32_t *status);

/* ---- stand-alone operators of the GemmEngine trait ------------------------------------------------
 * nyb200_gemm_f64 replaces GemmEngine::gemm_f64 (crates/ny-core/src/gemm.rs:356): C = A B for row-major binary64
 * matrices, host buffers, every output element one chain of fused multiply-adds over k in increasing order
 * (deterministic; |error| <= gamma_k |A||B|).
 * nyb200_conv_transpose_2d replaces GemmEngine::conv_transpose_2d (gemm.rs:556; parameters
 * ConvTranspose2dParams, gemm.rs:150-177): the Conv2d CROWN backward of one group.  a_reshaped is
 * [(num_specs*out_h*out_w) x out_channels] row-major, weight_col [out_channels x (in_channels*kernel_h*kernel_w)],
 * out [num_specs x (in_channels*in_h*in_w)].  The product and the col2im scatter run as one device pass; every
 * output element is accumulated in binary64 and rounded to fp32 once. */
int32_t nyb200_gemm_f64(nyb200_engine *e, int32_t m, int32_t k, int32_t n, const double *a, const double *b,
                        double *c_out);
typedef struct nyb200_conv_transpose_params {
    int32_t num_specs, out_channels, in_channels, out_h, out_w, in_h, in_w;
    int32_t kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w;
} nyb200_conv_transpose_params;
int32_t nyb200_conv_transpose_2d(nyb200_engine *e, const float *a_reshaped, const float *weight_col,
                                 const nyb200_conv_transpose_params *params, float *out);

/* ---- cooperative deadline (GpuCrownBackward::set_crown_backward_deadline, gemm.rs:4260-4279) ------
 * ns_from_now >= 0 arms a deadline that many nanoseconds after the call (monotonic clock); a negative value
 * clears it.  While armed, every multi-launch call (interval pass, backward pass, CROWN-IBP collection,
 * optimisation, attack) polls the clock between its units of work (one layer, one iteration, one step); past the
 * deadline it stops enqueuing, waits for the stream, invalidates the run's results and returns
 * NYB200_ERR_DEADLINE.  A launch in flight is never interrupted.  The caller clears the deadline afterwards. */
int32_t nyb200_set_deadline_ns(nyb200_engine *e, int64_t ns_from_now);

/* ---- joint gradient of the uploaded batch (crown_joint_alpha_gradient_resident, gemm.rs:4095;
 * crown_backward_gpu_resnet_sound_beta_batched_grad, gemm.rs:3999) --------------------------------
 * One bound evaluation at the batch's current parameters plus the adjoint pass, no parameter update.
 * objective 0: gradient of the sum of every domain's lower bounds; 1: of the domain's smallest lower bound.
 * grad [D x n_pre]: for an unstable unsplit neuron d(objective)/d(alpha); for a split neuron
 * d(objective)/d(beta) of its multiplier (beta >= 0); zero elsewhere.  The bounds of that evaluation are then
 * available through nyb200_batch_download. */
int32_t nyb200_batch_gradient(nyb200_engine *e, int32_t objective, float *grad);

/* ---- exact point gradients for K attack restarts (crown_point_vjp_batched[_resnet], gemm.rs:4207,4246) ----
 * grads[k] = spec_rows[k] . d f / d x at restart k, with the ReLU derivative taken from 0/1 masks.
 * Exactly one of x [K x dims[0]] (the masks are those of the concrete forward pass at x, [pre > 0]) and
 * masks [K x n_pre] (caller-supplied, a value > 0 passes the gradient; the last dims[L] entries of a row are
 * ignored) is non-NULL.  spec_rows [K x dims[L]], grads [K x dims[0]]; values [K] (optional, only with x)
 * receives spec_rows[k] . f(x_k).  Attack-only arithmetic: it never enters a bound. */
int32_t nyb200_point_vjp_batched(nyb200_engine *e, int32_t net_id, int32_t K, const float *x, const float *masks,
                                 const float *spec_rows, float *grads, float *values);

/* ---- reference-shaped calls ------------------------------------------------------------------------
 * The operands of ny's own trait methods, for a binding that wants a drop-in without touching its caller: layer
 * lists in BACKWARD order (output -> input; crates/ny-cuda/src/sound_crown.rs:1159-1260 walks them that way), whose
 * Activation members carry relaxation slopes the CALLER baked.  The split-list calls above derive the relaxation
 * on the device from 128 bytes per domain and are the fast route; these take about 24 bytes per neuron per domain
 * through host memory and exist for parity with the reference's interface.  Supported members: Linear and
 * Activation (GpuCrownLayer::{Linear, Activation, ActivationReluDualAlpha with equal slopes},
 * crates/ny-core/src/gemm.rs:1524-1645), strictly alternating; Conv2d / MaxPool2d members and Residual segments are
 * declined with NYB200_ERR_UNSUPPORTED (the trait's "decline -> CPU fallback"), never approximated. */
#define NYB200_CROWN_LINEAR 0
#define NYB200_CROWN_ACTIVATION 1
#define NYB200_CROWN_CONV2D 2
#define NYB200_CROWN_RELU_DUAL_ALPHA 3
typedef struct nyb200_crown_layer {
    int32_t kind;
    /* Linear: weight [out_features x in_features] row-major, bias [out_features] or NULL */
    const float *weight, *bias;
    int32_t out_features, in_features;
    /* Activation: per-neuron relaxation, [num_neurons] each (lower_intercept may be NULL = zeros).
     * ActivationReluDualAlpha: lower_slope = lower_pos_slope, upper_slope = cross_slope,
     * upper_intercept = cross_intercept, upper_neg_slope as named. */
    const float *lower_slope, *upper_slope, *lower_intercept, *upper_intercept, *upper_neg_slope;
    int32_t num_neurons;
} nyb200_crown_layer;
/* GpuCrownSeed (gemm.rs:1684-1691): an asymmetric frontier that starts the pass mid-network. */
typedef struct nyb200_crown_seed {
    const float *lower_a, *upper_a; /* [num_specs x current_dim] */
    const float *lower_b, *upper_b; /* [num_specs] or NULL (zeros) */
    int32_t num_specs, current_dim;
} nyb200_crown_seed;
/* GpuCrownBackward::crown_backward_gpu_sound (gemm.rs:3357) with spec [num_specs x out_features of layers[0]] and
 * seed == NULL, or ::crown_backward_gpu_seeded_sound (gemm.rs:3387) with a seed (spec ignored; the suffix may open
 * with the Activation behind which the frontier sits, current_dim = its num_neurons).  One input box
 * in_lo / in_hi [in_features of the last member].  Computed in the reference's own error convention (per-coefficient
 * error matrices carried to the box, binary64: layers/linear/crown_single.rs:2092-2103, bounds/concretize.rs:443-466),
 * so out_lo / out_hi [num_specs] are the reference's CPU CROWN bounds for the same slopes to within 1e-4 relative. */
int32_t nyb200_crown_backward(nyb200_engine *e, const nyb200_crown_layer *layers, int32_t n_layers, const float *spec,
                              int32_t num_specs, const nyb200_crown_seed *seed, const float *in_lo, const float *in_hi,
                              float *out_lo, float *out_hi);
/* GpuResnetBatchedDomainRef (gemm.rs:2939-2952) for a network that is one Chain segment: the domain's layer list
 * (shared weight tensors - the same pointers in every domain - and this domain's baked slopes), its input box, per
 * Activation in fold (backward) order its signed multipliers beta * sign (beta_signed[r], [num_neurons], NULL = none)
 * and its pre-node abs-max bounds (node_abs[r], [num_neurons]).  frontier_abs is accepted for signature parity and not
 * read: the rounding charges are discharged against node_abs and the box.  splits / n_splits name the multipliers the
 * _adam call optimises (GpuBetaAdamMapping, gemm.rs:2996-3012: relu = 0-based ReLU index in FORWARD order, neuron,
 * sign); the plain call ignores them. */
typedef struct nyb200_domain_ref {
    const nyb200_crown_layer *layers;
    int32_t n_layers;
    const float *input_lower, *input_upper;
    const float *const *beta_signed;
    const float *const *frontier_abs;
    const float *const *node_abs;
    const nyb200_split *splits;
    int32_t n_splits;
} nyb200_domain_ref;
/* GpuCrownBackward::crown_backward_gpu_resnet_sound_beta_batched (gemm.rs:3944): D domains, one shared spec
 * [num_specs x output width]; out_lo / out_hi [D x num_specs].  Same kernels and arithmetic as nyb200_bab_bound_batch
 * (tensor path with its certified rounding charge, binary64 re-evaluation when that charge shows); a heterogeneous or
 * non-finite batch is refused as a whole (gemm.rs:3941-3943). */
int32_t nyb200_crown_resnet_beta_batched(nyb200_engine *e, const nyb200_domain_ref *domains, int32_t D, const float *spec,
                                         int32_t num_specs, float *out_lo, float *out_hi);
/* GpuBetaAdamConfig (gemm.rs:2960-2993): projected-Adam ascent on the multipliers only, AMSGrad second moments,
 * at most `iterations` bound evaluations, a domain stops when its largest |gradient| falls below `tolerance`. */
typedef struct nyb200_beta_adam_config {
    int32_t iterations;
    float beta_lr, beta1, beta2, epsilon, tolerance;
} nyb200_beta_adam_config;
/* ::crown_backward_gpu_resnet_sound_beta_batched_adam (gemm.rs:4042): returns the element-wise best bounds over the
 * evaluated iterates and, in out_beta [D x max_splits] (may be NULL), the final multipliers in the order of each
 * domain's split mapping. */
int32_t nyb200_crown_resnet_beta_batched_adam(nyb200_engine *e, const nyb200_domain_ref *domains, int32_t D, const float *spec,
                                              int32_t num_specs, const nyb200_beta_adam_config *cfg, float *out_lo,
                                              float *out_hi, float *out_beta, int32_t max_splits);
/* GemmEngine::gemm_f64_triplet (gemm.rs:523): three same-shape binary64 products C_i = A_i B_i (the centre, magnitude
 * and propagated-error products of sound CROWN, crates/ny-cuda/src/sound_crown.rs:348-376), queued on one stream and
 * synchronised once; each obeys nyb200_gemm_f64's contract.  An operand pointer that repeats is uploaded once. */
int32_t nyb200_gemm_f64_triplet(nyb200_engine *e, int32_t m, int32_t k, int32_t n, const double *const a[3],
                                const double *const b[3], double *const c_out[3]);

/* ---- interval forward pass of ONE box without any device allocation ------------------------------
 * No counterpart in the reference: an addition for hosts that cannot let a library allocate device
 * memory at call time (a service that gave the whole GPU to its own arena at start-up, or a BaB loop
 * that cannot afford the device-wide synchronisation an allocation implies).  Same arithmetic and
 * output layout as nyb200_ibp_forward with D = 1, but in_lo/in_hi [dims[0]] and pre_lo/pre_hi
 * [sum_{k>=1} dims[k]] are DEVICE pointers owned by the caller, and the intermediate intervals live in
 * a fixed array inside the library image (about 128 KB per GPU, held from first use until exit).
 *   - Linear layers without residual connections only: a network registered with a Conv2d layer or a
 *     skip_from is refused with NYB200_ERR_UNSUPPORTED before anything is launched;
 *   - every layer width, the input included, must be <= 8192, otherwise NYB200_ERR_UNSUPPORTED;
 *   - all calls on a GPU share that array: calls that overlap on the device (other streams or engines)
 *     race and their results are undefined; calls on one stream are safe back to back;
 *   - the first call on a GPU resolves the array's device address: make it outside stream capture;
 *   - the call returns after the engine stream has drained (it reads one status word back). */
int32_t nyb200_ibp_forward_noalloc(nyb200_engine *e, int32_t net_id, const float *dev_in_lo, const float *dev_in_hi,
                                   float *dev_pre_lo, float *dev_pre_hi);

/* Kernel-only timing of the last nyb200_batch_run calls: average milliseconds per run of the
 * named phase ("forward", "backward", "total") measured with CUDA events on the engine stream
 * since the last reset.  With nyb200_timing_enable(e, 1) every per-layer launch of the A*W contraction kernel
 * is additionally bracketed by its own event pair and reported as phase "gemm" (average milliseconds
 * per run, summed over that run's launches; n_runs counts runs), and the fused backward chain launch of a run as
 * phase "chain". */
int32_t nyb200_timing_enable(nyb200_engine *e, int32_t per_kernel);
int32_t nyb200_timing_reset(nyb200_engine *e);
int32_t nyb200_timing_read(nyb200_engine *e, const char *phase, double *avg_ms, int32_t *n_runs);

#ifdef __cplusplus
}
#endif
#endif
