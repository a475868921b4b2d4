// Internal declarations shared by the engine's translation units (not part of the C ABI).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/nyb200.h"

namespace nyb {

constexpr int kMaxLinear = 32;

// Per-domain flag bits written by the kernels.
constexpr int kFlagInfeasible = 1;  // a split clamp inverted an interval: the domain is empty
constexpr int kFlagDegraded = 2;    // NaN / infinite pre-activation bound: bounds degrade to [-inf, +inf]
constexpr int kFlagInvalid = 4;     // split entry out of range
constexpr int kFlagLooseFwd = 8;    // fast-path interval pass: rounding slack visible against an unstable neuron's width
constexpr int kFlagLoose = 16;      // fast-path backward pass: rounding penalty visible against the bound

// Device-side view of a registered network (passed by value to kernels).
struct NetView {
    int L;                        // number of Linear layers
    int dims[kMaxLinear + 1];     // widths
    int pre_off[kMaxLinear + 1];  // offset of Linear_k's output block inside a [n_pre] row
    int n_pre;                    // sum_{k>=1} dims[k]
    int nps;                      // row stride of the per-domain device arrays: n_pre rounded up to 4
    const float *W[kMaxLinear];   // device, row-major [dims[k+1] x dims[k]]
    const float *b[kMaxLinear];   // device or nullptr
};

// Geometry of a Conv2d layer (NCHW flattened, dilation 1, one group).
struct ConvGeom {
    int ic, ih, iw, oc, oh, ow, kh, kw, sh, sw, ph, pw;
};

// Per-layer operands of the tcgen05 contraction: W split into TF32 high/low parts, transposed to
// [N x kpad] (K contiguous, zero padded to a multiple of 32) with one TMA tensor map each.
// Concretisation fused into the epilogue of the last contraction (k_umma_tf32x3): every epilogue thread routes its
// slice of the finished coefficient row against the input box (sign-routed binary64 products, as k_concretize) and
// leaves the slice's sum and magnitude sum in its own slot; k_concretize_fused adds a row's slots in a fixed order.
struct ConcFuse {
    int on = 0;
    int store = 0;            // also write the coefficient rows (a later call reads them)
    int R = 0, S = 0, slots = 0;
    const float *in_lo = nullptr, *in_hi = nullptr;
    long box_ds = 0;
    double *part = nullptr;   // [M x slots x 2]
    int *bad = nullptr;       // [M], cleared by the caller
};

struct UmmaLayer {
    float *wh = nullptr, *wl = nullptr;
    int K = 0, N = 0, kpad = 0;
    int chain = 0;  // K stages per tensor-memory accumulation chain for this operand; 0 = the kernel's default
    alignas(64) unsigned char tm_hi[128];
    alignas(64) unsigned char tm_lo[128];
};

struct Net {
    NetView v;
    std::vector<float *> owned;
    int max_dim = 0;
    std::vector<int> kind;        // per layer: NYB200_LAYER_LINEAR or NYB200_LAYER_CONV2D
    std::vector<ConvGeom> geom;   // per layer; meaningful for conv layers
    std::vector<int> skip;        // per layer: index of the layer whose post-activation output is added, or -1
    bool is_conv(int k) const { return !kind.empty() && kind[k] == NYB200_LAYER_CONV2D; }
    int skip_of(int k) const { return skip.empty() ? -1 : skip[k]; }
    bool has_skip() const { for (int j : skip) if (j >= 0) return true; return false; }
    std::vector<UmmaLayer> umma;  // filled on first use of the tcgen05 path
    std::vector<UmmaLayer> umma_fwd;  // interval forward operands [W+ | W-] per layer (entry 0 unused)
    std::vector<float *> wt;          // W_k^T, row-major [dims[k] x dims[k+1]] (adjoint pass; built on first use)
    std::vector<UmmaLayer> umma_adj;  // tcgen05 operands of the adjoint pass (from wt)
};

struct DevBuf {
    void *p = nullptr;
    size_t bytes = 0;
};

struct Batch {
    bool valid = false;
    int net_id = -1;
    int S = 0, R = 0, D = 0, mode = 0, box_stride = 0, max_splits = 0;
    bool has_alpha = false;
    bool ran = false;
    bool dual_alpha = false; // the upper rows use their own slopes (workspace "alpha_up")
    bool optimized = false;  // the last run was a parameter optimisation: results are the best-so-far bounds
    bool finished = false;  // results of the last run have been checked (and refined if needed)
    int refined = 0;        // domains that triggered the binary64 re-run of the last batch
    int opt_iterations = 0; // iterations of the last parameter optimisation
    int inh_stride = 0;     // 0: one inherited-bound vector for all domains; nps: one row per domain (nyb200_batch_set_inherited)
    bool external_tables = false;  // relaxation tables, abs-max tables and q were uploaded by a reference-shaped call:
                                   // nothing may re-derive them with an interval pass
    // Left behind by the last plain-CROWN call: the input-level coefficient rows of its final pass
    // ([crown_D * 2 * crown_S x crown_lda], per box S lower rows then S upper rows), until any call reuses the workspace.
    const float *crown_a = nullptr;
    int crown_lda = 0, crown_D = 0, crown_S = 0, crown_n0 = 0;
    const float *decision_thr = nullptr;   // device [S]: verdict-only refinement (nyb200_batch_set_thresholds, the frontier)
};

struct Timing {
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};  // start, after forward, end
    double fwd_ms = 0, bwd_ms = 0, tot_ms = 0, gemm_ms = 0, chain_ms = 0;
    int runs = 0;
    bool pending = false;
    bool per_kernel = false;
    std::vector<cudaEvent_t> kev;  // start/stop pairs around the contraction launches of the last run
    int kev_used = 0;
    cudaEvent_t cev[2] = {nullptr, nullptr};  // around the fused chain launch of the last run
    bool cev_used = false;
};

}  // namespace nyb

namespace nyb { struct ResidentFrontier; void frontier_free(ResidentFrontier *f); }
using nyb::ResidentFrontier;

struct nyb200_engine {
    int device = 0;
    cudaStream_t stream = nullptr;
    int reserve_sms = 0;                          // see nyb200_set_reserved_sms
    bool launch_overlap = true;                   // see nyb200_set_launch_overlap
    cudaStream_t own_stream = nullptr;            // created by nyb200_use_own_stream, destroyed with the engine
    int path = NYB200_PATH_TF32X3;
    float refine_tol = 5e-5f;  // see nyb200_set_refine_tolerance
    int error_channel = NYB200_ERRCH_IMMEDIATE;  // see nyb200_set_error_channel
    bool fuse_chain = true;                       // see nyb200_set_fusion
    std::string err;
    std::mutex mu;
    std::map<int, nyb::Net> nets;
    int next_net = 1;
    int64_t launches = 0;
    int64_t deadline_ns = -1;  // monotonic-clock deadline of the cooperative cancellation, or -1
    nyb::Batch batch;
    nyb::Timing timing;
    std::map<std::string, nyb::DevBuf> ws;  // named grow-only device workspace
    std::map<uint64_t, int> boundary_nets;   // networks registered on behalf of the reference-shaped calls, by weight key
    // Status words of the batch runs in mapped pinned host memory, written by the last kernel of every run:
    // [0] sequence number of the newest completed run, [1] pipeline error word seen by any run since the last finish,
    // [2] domains flagged for the binary64 re-evaluation by any run since the last finish.  See nyb200_batch_poll.
    struct ResidentFrontier *frontier = nullptr;   // nyb200_frontier_* (nyb200_frontier.cu)
    struct ResidentFrontier *frontier_spare = nullptr;   // the last destroyed frontier's device arrays, reused by the next
    // Pinned host staging: small inputs of an upload are gathered here so that their copies are truly asynchronous,
    // and the results of a run are fetched here ahead of the one synchronisation that ends it (a copy into pageable
    // memory is staged by the driver and blocks).  in: [0, kStageIn), out: the rest (grow-only).
    unsigned char *stage = nullptr;
    size_t stage_bytes = 0;
    cudaEvent_t stage_in_done = nullptr;   // the last upload's copies out of the input region
    bool stage_out_valid = false;          // the output region holds the resident batch's final results
    int *status_host = nullptr;
    int *status_dev = nullptr;
    int run_seq = 0;
};

// Programmatic dependent launch.  A kernel launched through launch_pdl may be scheduled while its predecessor in the
// stream is still running (the predecessor says when by pdl_trigger, at the latest by finishing); it must call pdl_wait
// before its first access to memory that any earlier kernel of the stream writes or reads, which returns once the
// predecessor has completed and its writes are visible.  What overlaps is the launch latency, the scheduling of the
// CTAs and whatever the kernel does before pdl_wait (barrier set-up, tensor-memory allocation).  Both calls do nothing
// in a kernel that was launched the ordinary way.  With several engines on one GPU the early-scheduled CTAs of a
// full-width kernel hold their SMs' shared memory while they wait, which keeps other engines' kernels off those SMs:
// nyb200_set_launch_overlap(e, 0) launches the ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, nyb200_engine *e, Args &&...args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = e->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = e->launch_overlap ? 1 : 0;   // off: an ordinary launch (see nyb200_set_launch_overlap)
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

namespace nyb { constexpr size_t kStageIn = 1 << 20; }

#define NYB_TRY(expr)                      \
    do {                                   \
        int _st = (expr);                  \
        if (_st != NYB200_OK) return _st;  \
    } while (0)
#define NYB_CUDA(e, call) NYB_TRY(nyb::check_cuda((e), (call), #call))
#define NYB_WS(var, type, e, name, bytes)                          \
    type var = (type)nyb::ws_get((e), (name), (bytes));                 \
    if (!var) return NYB200_ERR_OOM;

namespace nyb {

// Returns a device buffer of at least `bytes` under `name` (grow-only); nullptr on failure.
void *ws_get(nyb200_engine *e, const char *name, size_t bytes);
int set_err(nyb200_engine *e, int code, const std::string &msg);
int check_cuda(nyb200_engine *e, cudaError_t st, const char *what);

// ---- kernel launchers (nyb200_kernels.cu) ----
void launch_scatter_splits(nyb200_engine *e, const NetView &nv, const nyb200_split *sp, const int *ns, int max_splits,
                           int D, signed char *code, float *sbeta, int *flags);
// Interval mat-vec of Linear_k for Deff boxes (binary64 accumulation, outward rounded).
void launch_ibp_linear(nyb200_engine *e, const NetView &nv, int k, int Deff, const float *zl, const float *zu,
                       long in_dstride, float *raw_lo, float *raw_hi, float *q, long out_dstride);
// Per-domain finish of Linear_k's output: intersect / clamp / relaxation tables / post-activation.
void launch_ibp_finish(nyb200_engine *e, const NetView &nv, int k, int D, int mode, const float *raw_lo,
                       const float *raw_hi, long raw_dstride, const float *inh_lo, const float *inh_hi, long inh_dstride,
                       const signed char *code, const float *sbeta, const float *alpha, float *pre_lo, float *pre_hi,
                       float *zl, float *zu, float4 *tab, float *zabs, int *flags, const float *F = nullptr, int ldf = 0,
                       double eps = 0.0, float *q = nullptr, float fwd_tol = 0.f,
                       float *cj = nullptr, float cj_eps = 0.f, float cj_kappa = 0.f);
void launch_seed(nyb200_engine *e, const float *spec, int S, int nL, int D, int lda, float *A);
// A [D*2n x lda] = per domain the n x n identity for the lower rows, then again for the upper rows.
void launch_seed_identity(nyb200_engine *e, int n, int D, int lda, float *A);
// In-place ReLU relaxation of A [M x n] (ReLU r) or identity pass (r < 0), accumulating the row sums.
// With Asrc != nullptr the rows are read from Asrc (row stride lds) and the result written to A.
void launch_relax(nyb200_engine *e, const NetView &nv, int r, int lin_k, int M, int R, int S, float *A, int lda,
                  const float4 *tab, const float *zabs, const float *q, long q_dstride, double eps_gemm, double *rb,
                  double *rabs, double *rpen, const float *Asrc, int lds, const float *aup = nullptr);
// C[M x N] = A[M x K] * W_k (binary64 accumulation), cast error charged to rpen.
void launch_gemm_f64(nyb200_engine *e, int M, int N, int K, const float *A, int lda, const float *B, int ldb, float *C,
                     int ldc, int R, const float *zin_lo, const float *zin_hi, long zin_dstride, double *rpen);
void launch_concretize(nyb200_engine *e, int M, int R, int S, int n0, const float *A, int lda, const float *in_lo,
                       const float *in_hi, long box_dstride, const double *rb, const double *rabs, const double *rpen,
                       int *flags, float *out_lo, float *out_hi, float *min_lower, float loose_tol);
// Per (domain, spec row): domain flags and the repair rule applied to the bounds, global minimum folded.
void launch_finalize(nyb200_engine *e, int D, int S, const int *flags, float *out_lo, float *out_hi, float *min_lower);
void launch_verdicts(nyb200_engine *e, int D, int S, const float *out_lo, const float *out_hi, const int *flags,
                     float threshold, int *status);
// dst row i = src row idx[i] (gather) or dst row idx[i] = src row i (scatter); rows of `row_words` 32-bit words.
void launch_gather_rows(nyb200_engine *e, void *dst, const void *src, const int *idx, int n_rows, long row_words);
void launch_scatter_rows(nyb200_engine *e, void *dst, const void *src, const int *idx, int n_rows, long row_words);
// min over feasible domains and rows of out_lo (the value the concretisation folds), recomputed from scratch
void launch_min_lower(nyb200_engine *e, int D, int S, const float *out_lo, const int *flags, float *min_lower);
void launch_select_branch(nyb200_engine *e, const NetView &nv, int D, const float *pre_lo, const float *pre_hi,
                          const signed char *code, int *relu, int *neuron, float *width, int kind);
void launch_fill_f64(nyb200_engine *e, double *p, size_t n, double v);
void launch_fill_f32(nyb200_engine *e, float *p, size_t n, float v);

// ---- resident batch (nyb200_api.cu) ----
// Device addresses of the resident batch's arrays (all inside the engine's named workspace).
struct BatchPtrs {
    float *spec, *in_lo, *in_hi, *inh_lo, *inh_hi, *alpha;
    nyb200_split *splits;
    int *nsplits, *flags;
    signed char *code;
    float *sbeta, *raw_lo, *raw_hi, *q, *pre_lo, *pre_hi, *zl, *zu, *zabs;
    float4 *tab;
    float *A0, *A1;
    double *rb, *rabs, *rpen;
    int *row_bad;
    float *out_lo, *out_hi, *min_lower;
    int lda;
    float *a_final = nullptr;  // set by run_backward: the coefficients on the input box, [D*R x lda]
    bool keep_final = false;   // the caller reads a_final afterwards: the last contraction must store its rows
    float *cj = nullptr;       // charge weights of the fused chain, when the interval pass already wrote them
    float *alpha_up = nullptr; // dual alpha: the upper path's own lower slopes [D x nps], or null (shared with the lower path)
};
int batch_ptrs(nyb200_engine *e, const Net &net, const Batch &b, BatchPtrs &p);
int find_net(nyb200_engine *e, int net_id, Net **out);
void free_net(Net &net);
// Interval forward pass for the resident batch.  fwd_mode: 0 clamp-only, 1 constrained, 2 plain IBP.
int run_forward(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int fwd_mode);
// Backward pass + concretisation.  With ckpt != nullptr, ckpt[r] (row stride ld_ckpt) receives the
// coefficients entering ReLU r before its relaxation is applied.
// top >= 0 starts the pass at Linear_top's output with identity rows (b.S = dims[top + 1]) instead of the spec.
int run_backward(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, float *const *ckpt, int ld_ckpt, int top = -1);
// The same pass in the reference's error convention (per-coefficient error matrices carried to the input box,
// binary64 arithmetic; nyb200_ref.cu).
// seed: optional asymmetric starting rows (GpuCrownSeed, crates/ny-core/src/gemm.rs:1684-1691), device pointers:
// lower_a / upper_a [S x dims[L]], bias [2S] (lower biases, then upper biases)
struct RefSeed { const float *lower_a = nullptr, *upper_a = nullptr, *bias = nullptr; bool relu_first = false; };
int run_backward_ref(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int top, const RefSeed *seed = nullptr);
int create_net(nyb200_engine *e, int32_t n_layers, const nyb200_layer_desc *ld, const float *wflat, const float *bflat, int32_t *net_id);
int finish_batch_public(nyb200_engine *e);
int run_batch_public(nyb200_engine *e);
void launch_dgemm(nyb200_engine *e, int m, int n, int k, const double *a, const double *b, double *c);
int prepare_backward_operands(nyb200_engine *e, Net &net);
// ---- fused backward chain (nyb200_chain.cu) ----
bool chain_eligible(const Net &net, int L);
double chain_eps(int K);
float chain_cj_eps(const Net &net, int L, int block);   // rounding rate folded into the charge weights of table block `block`
float chain_kappa();
int launch_chain(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int L, bool identity_seed, bool shared_box,
                 float *A_out, double eps0, int *derr);
int prepare_transposed(nyb200_engine *e, Net &net, bool tensor);
int conv_forward_tensor(nyb200_engine *e, Net &net, int k, int rows, const float *Z, int ldz, float *out, int ldo, int *derr);
void fold_timing(Timing &t);
cudaEvent_t next_kev(Timing &t);

// ---- plain CROWN with CROWN-IBP intermediate bounds (nyb200_crown.cu) ----
int crown_bounds(nyb200_engine *e, int net_id, const float *spec, int S, const float *in_lo, const float *in_hi,
                 int box_stride, int D, float *out_lo, float *out_hi, float *inter_lo, float *inter_hi);

// ---- parameter optimisation (nyb200_optimize.cu) ----
// grad_host != nullptr: one evaluation plus the adjoint pass, gradients [D x n_pre] to the host, no update
int optimize_batch(nyb200_engine *e, const nyb200_opt_config &cfg, float *grad_host = nullptr);
int babsr_select(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int *relu, int *neuron, float *best,
                 float **score_dev);
// Cooperative cancellation: true once the armed deadline has passed.
bool deadline_passed(const nyb200_engine *e);
// What a multi-launch call does when the deadline has passed: drain the stream, drop the run, report.
int deadline_abort(nyb200_engine *e, const char *where);
#define NYB_DEADLINE(e, where) \
    do { if (nyb::deadline_passed(e)) return nyb::deadline_abort((e), (where)); } while (0)
int refine_optimized(nyb200_engine *e, Net &net, Batch &b, BatchPtrs &p);
int download_params(nyb200_engine *e, float *alpha, float *beta);

// ---- residual connections (nyb200_kernels.cu) ----
// raw_lo/raw_hi block `off` += the interval [zl, zu] block `src_off`, rounded outward.
void launch_skip_interval(nyb200_engine *e, int D, int n, long stride, float *raw_lo, float *raw_hi, int off,
                          const float *zl, const float *zu, int src_off);
// A[M x n] += S[M x n]; the rounding of every sum is measured exactly and charged against the magnitude of the
// skipped variable (zl/zu at `src_off`), or ignored when rpen is null.
void launch_skip_coeff(nyb200_engine *e, int M, int n, float *A, int lda, const float *S, int lds, int R,
                       const float *zl, const float *zu, long stride, int src_off, double *rpen);

// ---- Conv2d layers (nyb200_conv.cu) ----
void launch_ibp_conv(nyb200_engine *e, const NetView &nv, const ConvGeom &g, int k, int Deff, const float *zl,
                     const float *zu, long in_dstride, float *raw_lo, float *raw_hi, float *q, long out_dstride);
// C[M x ic*ih*iw] = transposed convolution of A[M x oc*oh*ow] (binary64 accumulation, cast error charged to rpen).
// With `cols` (M * oh*ow * ic*kh*kw doubles of scratch) it runs as an im2col-space binary64 GEMM plus a gather,
// without it as one direct gather kernel.
void launch_conv_transpose(nyb200_engine *e, const ConvGeom &g, int M, const float *A, int lda, float *C, int ldc,
                           const float *W, int R, const float *zin_lo, const float *zin_hi, long zin_dstride,
                           double *rpen, double *cols);
// Sums the tap-major im2col-space products cols[(m * taps + tap) * plane + (oy, ox)] into C[m, (ci, y, x)]
// (binary64 sums of the fp32 entries, one cast: charged through the layer's rounding rate).
void launch_col2im(nyb200_engine *e, const ConvGeom &g, int M, const float *cols, float *C, int ldc);
// Forward convolutions on the tensor path: operand Wf [ic x oc*kh*kw] (or [W+ | W-] with `split`), the per-pixel
// products through launch_umma(a_plane = ih*iw), then one of the gathers.
int prepare_conv_forward_operand(nyb200_engine *e, const float *W, const ConvGeom &g, bool split, UmmaLayer *out);
void launch_ibp_conv_gather(nyb200_engine *e, const NetView &nv, const ConvGeom &g, int k, int D, const float *cols, double eps,
                            float *raw_lo, float *raw_hi, float *q, long out_dstride);
void launch_conv_fwd_gather(nyb200_engine *e, const ConvGeom &g, int rows, const float *cols, float *out, int ldo);
void launch_conv_plain(nyb200_engine *e, const ConvGeom &g, int rows, const float *Z, int ldz, const float *W, float *out,
                       int ldo);

// ---- tcgen05 contraction (nyb200_umma.cu) ----
int umma_prepare_layer(nyb200_engine *e, const float *W, int K, int N, UmmaLayer *out);
// a_plane > 0 selects the transposed-convolution form: GEMM row r = (m, p) with p < a_plane, operand element
// k at A[m * lda + k * a_plane + p], result column n at C[(m * N + n) * a_plane + p] (ldc unused).
int launch_umma(nyb200_engine *e, const UmmaLayer &L, int M, const float *A, int lda, float *C, int ldc, int *err,
                int a_plane = 0, const ConcFuse *cf = nullptr);
void launch_concretize_fused(nyb200_engine *e, int M, int R, int S, int slots, const double *part, const int *bad,
                             const double *rb, const double *rabs, const double *rpen, int *flags, float *out_lo,
                             float *out_hi, float *min_lower, float loose_tol);
double umma_eps(int K, int chain = 0);
// Builds the forward-pass operand of Linear_k: the [n_in x 2 n_out] matrix (W+^T | W-^T).
int umma_prepare_forward_layer(nyb200_engine *e, const float *W, int n_in, int n_out, UmmaLayer *out);
// raw_lo/raw_hi/q of Linear_k from the two products Fl = zl * (W+|W-), Fu = zu * (W+|W-) (zl >= 0).
void launch_ibp_combine(nyb200_engine *e, int D, int n_out, const float *Fl, const float *Fu, int ldf, const float *bias,
                        double eps, float *raw_lo, float *raw_hi, float *q, long out_ds);

}  // namespace nyb
