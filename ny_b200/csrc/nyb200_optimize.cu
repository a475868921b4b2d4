// Projected-Adam optimisation of the relaxation parameters of the resident batch: every domain's lower
// slopes alpha and split multipliers beta, all domains in lock-step.
//
// One iteration is
//   1. the sound backward pass (nyb200_api.cu: run_backward) with the current parameters, which also
//      keeps, per ReLU, the coefficients that entered its relaxation (the "checkpoints");
//   2. an element-wise best-so-far fold of the bounds (network/alpha_crown_loop.rs:928-936);
//   3. the reverse adjoint of crates/ny-core/src/joint_alpha_grad.rs:22-50 over the lower rows:
//        Z^0[s, j]   = x_lo[j] if A^0[s, j] >= 0 else x_hi[j]
//        Zpre_k      = Z^k W_k^T + b_k                                  (tcgen05 or binary64 contraction)
//        d/d alpha_i = sum_s Zpre_k[s, i] * max(Apre_k[s, i], 0)        (unstable, unsplit neurons)
//        d/d beta_i  = -sign_i * sum_s Zpre_k[s, i]                     (split neurons)
//        Z^{k+1}     = Zpre_k * sigma + tau,  (sigma, tau) = (alpha, 0) if Apre >= 0 else (us, ui)
//      fused with the Adam step of each parameter (bounds/alpha/shared.rs:106-146 for alpha,
//      beta_crown/state/beta.rs:314-441 for beta), because a parameter's gradient is complete inside
//      the one thread that owns its (domain, neuron) pair.
// The gradient only proposes the next parameters; its arithmetic carries no rounding bookkeeping.  Every
// bound that is ever reported comes from step 1.
#include <string.h>

#include "nyb200_internal.cuh"

namespace nyb {

namespace {

struct AdamStep {
    float lr_alpha, lr_beta, beta1, beta2, epsilon, bc1, bc2, clip_beta;
    int rule;  // 0 Adam, 1 plain projected step, 2 Adam + AMSGrad
};

// Per-domain optimisation state (workspace "opt_state", D entries each).
struct OptState {
    int *stopped;        // 0 = running, t = stopped by the rules after the update of iteration t
    unsigned *maxg;      // bit pattern of max |gradient| of the iteration in flight (non-negative floats order as integers; NaN sorts above inf)
    float *best_obj;     // best objective value so far
    int *no_improve;     // iterations without improvement
};

__device__ __forceinline__ float nan_max(float a, float b) { return (isnan(a) || isnan(b)) ? NAN : fmaxf(a, b); }

__global__ void k_transpose(const float *__restrict__ W, int n_out, int n_in, float *__restrict__ WT) {
    __shared__ float tile[32][33];
    int o0 = blockIdx.y * 32, i0 = blockIdx.x * 32;
    for (int r = threadIdx.y; r < 32; r += 8) {
        int o = o0 + r, i = i0 + threadIdx.x;
        tile[r][threadIdx.x] = (o < n_out && i < n_in) ? W[(long)o * n_in + i] : 0.f;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += 8) {
        int i = i0 + r, o = o0 + threadIdx.x;
        if (i < n_in && o < n_out) WT[(long)i * n_out + o] = tile[threadIdx.x][r];
    }
}

// Z[d*Zr + s][j] = the box corner row (d, s) concretises on: lower rows (s < S) take x_lo where the coefficient
// is >= 0, upper rows (S <= s < Zr, present with the dual alpha: Zr = 2S) take x_hi there.
__global__ void k_adjoint_seed(int D, int S, int R, int Zr, int n0, const float *__restrict__ A, int lda,
                               const float *__restrict__ in_lo, const float *__restrict__ in_hi, long box_ds,
                               float *__restrict__ Z, int ldz) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * Zr * n0) return;
    int j = (int)(t % n0);
    long ds = t / n0;
    int d = (int)(ds / Zr), s = (int)(ds % Zr);
    float a = A[((long)d * R + s) * lda + j];
    bool take_lo = (a >= 0.f) == (s < S);
    Z[ds * ldz + j] = take_lo ? in_lo[(long)d * box_ds + j] : in_hi[(long)d * box_ds + j];
}

// One thread per (domain, neuron) of ReLU `k`: adds the bias, harvests the parameter gradient over the
// domain's S lower rows, maps Zpre to the post-activation adjoint in place, then takes the Adam step of the
// parameter this neuron owns (alpha if unstable and unsplit, beta if split, none otherwise) and writes it
// into the relaxation table the next backward pass reads.
__global__ void __launch_bounds__(256)
k_adjoint_relu(int n, int off, int D, int S, int R, int Zr, long nps, float *__restrict__ Z, int ldz,
               const float *__restrict__ bias, const float *__restrict__ Apre, int ldc, float4 *__restrict__ tab,
               const signed char *__restrict__ code, const float *__restrict__ pre_lo,
               const float *__restrict__ pre_hi, float *__restrict__ mom, float *__restrict__ var,
               const int *__restrict__ only_row, float *__restrict__ aup, float *__restrict__ mom_up,
               float *__restrict__ var_up, float *__restrict__ grad_out, AdamStep h, const int *__restrict__ stopped,
               unsigned *__restrict__ maxg, float *__restrict__ vmax, float *__restrict__ vmax_up) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * n) return;
    int d = (int)(t / n), i = (int)(t % n);
    const bool frozen = stopped && stopped[d] != 0;  // a stopped domain keeps its parameters
    long o = (long)d * nps + off + i;
    float4 tb = tab[o];
    float bk = bias ? bias[i] : 0.f;
    float g_alpha = 0.f, g_sum = 0.f;
    const int pick = only_row ? only_row[d] : -1;  // objective: one row of the domain, or the sum over its rows
    for (int s = 0; s < S; ++s) {
        long zr = ((long)d * Zr + s) * ldz + i;
        float g = Z[zr] + bk;
        float ap = Apre[((long)d * R + s) * ldc + i];
        if (pick < 0 || s == pick) {
            g_alpha = fmaf(g, fmaxf(ap, 0.f), g_alpha);
            g_sum += g;
        }
        bool pos = ap >= 0.f;
        Z[zr] = fmaf(g, pos ? tb.x : tb.y, pos ? 0.f : tb.z);
    }
    int c = code[o];
    float l = pre_lo[o], u = pre_hi[o];
    if (Zr > S) {
        // dual alpha: the upper rows' adjoint; a >= 0 takes the chord, a < 0 the upper path's own slope, whose
        // gradient is sum_s Zpre * min(Apre, 0); the sum of the upper bounds descends
        float au = aup[o], g_up = 0.f;
        for (int s = S; s < Zr; ++s) {
            long zr = ((long)d * Zr + s) * ldz + i;
            float g = Z[zr] + bk;
            float ap = Apre[((long)d * R + s) * ldc + i];
            g_up = fmaf(g, fminf(ap, 0.f), g_up);
            bool pos = ap >= 0.f;
            Z[zr] = fmaf(g, pos ? tb.y : au, pos ? tb.z : 0.f);
        }
        if ((c == 0) && (l < 0.f) && (u > 0.f) && h.lr_alpha > 0.f && !frozen) {
            float a, m = 0.f, v = 0.f;
            if (h.rule == 1) a = au - h.lr_alpha * g_up;
            else {
                m = h.beta1 * mom_up[o] + (1.f - h.beta1) * g_up;
                v = h.beta2 * var_up[o] + (1.f - h.beta2) * g_up * g_up;
                float vu = v;
                if (h.rule == 2) { vu = nan_max(vmax_up[o], v); vmax_up[o] = vu; }
                a = au - h.lr_alpha * (m / h.bc1) / (sqrtf(vu / h.bc2) + h.epsilon);
            }
            a = fminf(fmaxf(a, 0.f), 1.f);
            if (isnan(a)) { a = 0.5f; m = 0.f; v = 0.f; if (h.rule == 2) vmax_up[o] = 0.f; }
            aup[o] = a;
            if (h.rule != 1) { mom_up[o] = m; var_up[o] = v; }
        }
    }
    if (grad_out)  // export: the slope's gradient of an unstable unsplit neuron, the multiplier's of a split one
        grad_out[o] = ((c == 0) && (l < 0.f) && (u > 0.f)) ? g_alpha : (c != 0 ? (c > 0 ? -g_sum : g_sum) : 0.f);
    bool is_alpha = (c == 0) && (l < 0.f) && (u > 0.f) && h.lr_alpha > 0.f;
    bool is_beta = (c != 0) && h.lr_beta > 0.f;
    if ((!is_alpha && !is_beta) || frozen) return;
    float g = is_alpha ? g_alpha : (c > 0 ? -g_sum : g_sum);
    if (is_beta && h.rule != 1 && h.clip_beta > 0.f) g = fminf(fmaxf(g, -h.clip_beta), h.clip_beta);
    if (maxg) atomicMax(&maxg[d], __float_as_uint(fabsf(g)));  // the domain's convergence measure (NaN wins, as in the reference)
    float m = 0.f, v = 0.f, step;
    if (h.rule == 1) step = g;
    else {
        m = h.beta1 * mom[o] + (1.f - h.beta1) * g;
        v = h.beta2 * var[o] + (1.f - h.beta2) * g * g;
        float vu = v;
        if (h.rule == 2) { vu = nan_max(vmax[o], v); vmax[o] = vu; }
        step = (m / h.bc1) / (sqrtf(vu / h.bc2) + h.epsilon);
    }
    if (is_alpha) {
        float a = tb.x + h.lr_alpha * step;
        a = fminf(fmaxf(a, 0.f), 1.f);
        if (isnan(a)) { a = 0.5f; m = 0.f; v = 0.f; if (h.rule == 2) vmax[o] = 0.f; }
        tb.x = a;
    } else {
        float sgn = c > 0 ? 1.f : -1.f;
        float b = fabsf(tb.w) + h.lr_beta * step;
        if (isnan(b) || isinf(b)) { b = 0.f; m = 0.f; v = 0.f; if (h.rule == 2) vmax[o] = 0.f; }
        tb.w = sgn * fmaxf(b, 0.f);
    }
    if (h.rule != 1) { mom[o] = m; var[o] = v; }
    tab[o] = tb;
}

// Y[r, j] += X[r, j]
__global__ void k_add_adjoint(long rows, int n, float *__restrict__ Y, int ldy, const float *__restrict__ X, int ldx) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= rows * n) return;
    long r = t / n;
    int j = (int)(t - r * n);
    Y[r * ldy + j] += X[r * ldx + j];
}

// alpha_up = the lower path's slopes (the table's first component), the starting point of the dual alpha
__global__ void k_init_alpha_up(long n, const float4 *__restrict__ tab, float *__restrict__ aup) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) aup[t] = tab[t].x;
}

// Row with the smallest current lower bound per domain (first minimum wins).
__global__ void k_argmin_row(int D, int S, const float *__restrict__ lo, int *__restrict__ row) {
    int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    int best = 0;
    for (int s = 1; s < S; ++s)
        if (lo[d * S + s] < lo[d * S + best]) best = s;
    row[d] = best;
}

// save: this iteration updates the best bounds of every domain; otherwise only of the domains that have stopped
// (their last parameters are being evaluated for the first time: the forced save of the reference's early exits)
__global__ void k_fold_best(long n, int first, const float *__restrict__ lo, const float *__restrict__ hi,
                            float *__restrict__ best_lo, float *__restrict__ best_hi, int S = 1, int save = 1,
                            const int *__restrict__ stopped = nullptr) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    if (!save && !(stopped && stopped[t / S] != 0)) return;
    float l = lo[t], u = hi[t];
    if (!first) {
        // infeasible domains report (+inf, -inf) and degraded ones (-inf, +inf) on every iteration, so
        // max / min keep those markers
        l = fmaxf(l, best_lo[t]); u = fminf(u, best_hi[t]);
    }
    best_lo[t] = l; best_hi[t] = u;
}

// After the updates of iteration t: per domain, the objective of this iteration's evaluation against the best so far
// (patience), the iteration's largest gradient against the tolerance; a domain that meets a rule is marked stopped.
__global__ void k_opt_rules(int D, int S, int t, int objective, float tolerance, int patience, const float *__restrict__ lo,
                            OptState st) {
    int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const float mg = __uint_as_float(st.maxg[d]);
    st.maxg[d] = 0u;
    if (st.stopped[d] != 0) return;
    float obj = 0.f;
    if (objective == 1) { obj = lo[d * S]; for (int s = 1; s < S; ++s) obj = fminf(obj, lo[d * S + s]); }
    else for (int s = 0; s < S; ++s) { float l = lo[d * S + s]; if (isfinite(l)) obj += l; }
    int ni = st.no_improve[d];
    if (obj > st.best_obj[d]) { st.best_obj[d] = obj; ni = 0; } else ++ni;
    st.no_improve[d] = ni;
    bool stop = (tolerance > 0.f && mg < tolerance) || (patience > 0 && ni > patience);
    if (stop) st.stopped[d] = t;
}

__device__ __forceinline__ void atomic_min_f(float *addr, float v) {
    if (v >= 0.f) atomicMin((int *)addr, __float_as_int(v));
    else atomicMax((unsigned *)addr, __float_as_uint(v));
}

// Publishes the best bounds as the run's result and folds the global minimum lower bound.
__global__ void k_publish_best(int D, int S, const int *__restrict__ flags, const float *__restrict__ best_lo,
                               const float *__restrict__ best_hi, float *__restrict__ out_lo,
                               float *__restrict__ out_hi, float *__restrict__ min_lower) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= D * S) return;
    float l = best_lo[t];
    out_lo[t] = l; out_hi[t] = best_hi[t];
    if (!(flags[t / S] & kFlagInfeasible)) atomic_min_f(min_lower, l);
}

__global__ void k_gather_params(NetView nv, int D, int max_splits, const float4 *__restrict__ tab,
                                const nyb200_split *__restrict__ sp, const int *__restrict__ ns,
                                float *__restrict__ alpha, float *__restrict__ beta) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    long na = (long)D * nv.n_pre, nb = (long)D * max_splits;
    if (t < na) {
        if (alpha) { int d = (int)(t / nv.n_pre), j = (int)(t % nv.n_pre); alpha[t] = tab[(long)d * nv.nps + j].x; }
        return;
    }
    t -= na;
    if (t >= nb || !beta) return;
    int d = (int)(t / max_splits), q = (int)(t % max_splits);
    float b = 0.f;
    if (q < ns[d]) {
        nyb200_split s = sp[t];
        if (s.relu >= 0 && s.relu < nv.L - 1 && s.neuron >= 0 && s.neuron < nv.dims[s.relu + 1])
            b = fabsf(tab[(long)d * nv.nps + nv.pre_off[s.relu] + s.neuron].w);
    }
    beta[t] = b;
}

}  // namespace

// W_k^T (row-major [dims[k] x dims[k+1]]) for every Linear layer, and its tcgen05 operands: what a forward
// product Z * W_k^T needs (the parameter adjoint and the concrete forward pass of the attack).
int prepare_transposed(nyb200_engine *e, Net &net, bool tensor) {
    const NetView &nv = net.v;
    const int L = nv.L;
    if (net.wt.empty()) {
        net.wt.resize(L, nullptr);
        for (int k = 0; k < L; ++k) {
            if (net.is_conv(k)) continue;  // a convolution's forward product runs the convolution itself
            NYB_CUDA(e, cudaMalloc(&net.wt[k], (size_t)nv.dims[k] * nv.dims[k + 1] * 4));
            dim3 grid((nv.dims[k] + 31) / 32, (nv.dims[k + 1] + 31) / 32), blk(32, 8);
            k_transpose<<<grid, blk, 0, e->stream>>>(nv.W[k], nv.dims[k + 1], nv.dims[k], net.wt[k]);
            e->launches++;
        }
    }
    if (tensor && net.umma_adj.empty()) {
        net.umma_adj.resize(L);
        for (int k = 0; k < L; ++k) {
            if (!net.is_conv(k)) NYB_TRY(umma_prepare_layer(e, net.wt[k], nv.dims[k], nv.dims[k + 1], &net.umma_adj[k]));
            else NYB_TRY(prepare_conv_forward_operand(e, nv.W[k], net.geom[k], false, &net.umma_adj[k]));
        }
    }
    return NYB200_OK;
}

// out[rows x oc*oh*ow] = convolution k of the rows of Z (no bias), on the tensor path: per-pixel products, gather.
int conv_forward_tensor(nyb200_engine *e, Net &net, int k, int rows, const float *Z, int ldz, float *out, int ldo, int *derr) {
    const ConvGeom &g = net.geom[k];
    const int plane = g.ih * g.iw, N = g.oc * g.kh * g.kw;
    if ((long)rows * plane > 0x7fffffffL) return set_err(e, NYB200_ERR_UNSUPPORTED, "batch too large for the convolution's product space");
    float *cols = (float *)ws_get(e, "conv_cols", (size_t)rows * plane * N * 4);
    if (!cols) return NYB200_ERR_OOM;
    NYB_TRY(launch_umma(e, net.umma_adj[k], rows * plane, Z, ldz, cols, N, derr, plane));
    launch_conv_fwd_gather(e, g, rows, cols, out, ldo);
    return NYB200_OK;
}

int optimize_batch(nyb200_engine *e, const nyb200_opt_config &cfg, float *grad_host) {
    if (!e->batch.valid) return set_err(e, NYB200_ERR_INVALID, "no batch uploaded");
    if (grad_host && (cfg.objective == 2 || cfg.iterations != 2))
        return set_err(e, NYB200_ERR_INVALID, "gradient export: objective 0 or 1");
    if (cfg.iterations < 1) return set_err(e, NYB200_ERR_INVALID, "iterations must be >= 1");
    if (cfg.objective < 0 || cfg.objective > 2) return set_err(e, NYB200_ERR_INVALID, "objective must be 0, 1 or 2");
    if (!(cfg.lr_alpha >= 0.f) || !(cfg.lr_beta >= 0.f) || !(cfg.lr_decay > 0.f))
        return set_err(e, NYB200_ERR_INVALID, "learning rates must be >= 0 and the decay > 0");
    if (cfg.rule < 0 || cfg.rule > 2) return set_err(e, NYB200_ERR_INVALID, "rule must be 0 (Adam), 1 (plain projected step) or 2 (AMSGrad)");
    if (!(cfg.tolerance >= 0.f) || cfg.patience < 0 || !(cfg.start_save_best >= 0.f) || !(cfg.start_save_best < 1.f))
        return set_err(e, NYB200_ERR_INVALID, "tolerance and patience must be >= 0, start_save_best in [0, 1)");
    Net *net;
    NYB_TRY(find_net(e, e->batch.net_id, &net));
    Batch &b = e->batch;
    b.dual_alpha = cfg.objective == 2 && cfg.iterations > 1 && net->v.L >= 2;  // decides which arrays the batch has
    BatchPtrs p;
    NYB_TRY(batch_ptrs(e, *net, b, p));
    const NetView &nv = net->v;
    const int L = nv.L, D = b.D, S = b.S, R = b.R;
    const long M = (long)D * R, np = nv.nps;
    const bool tensor = e->path == NYB200_PATH_TF32X3;
    const int T = (L >= 2) ? cfg.iterations : 1;
    const bool dual = cfg.objective == 2 && T > 1;
    const int Zr = dual ? R : S;  // adjoint rows per domain
    const float b1 = cfg.beta1 > 0.f ? cfg.beta1 : 0.9f, b2 = cfg.beta2 > 0.f ? cfg.beta2 : 0.999f;
    const float eps = cfg.epsilon > 0.f ? cfg.epsilon : 1e-8f;

    // workspace
    const int ldc = p.lda, ldz = p.lda;
    std::vector<float *> ckpt((size_t)(L > 1 ? L - 1 : 0), nullptr);
    float *z0 = nullptr, *z1 = nullptr, *mom = nullptr, *var = nullptr;
    if (T > 1) {
        NYB_WS(ck, float *, e, "ckpt", (size_t)(L - 1) * M * ldc * 4);
        for (int r = 0; r < L - 1; ++r) ckpt[r] = ck + (size_t)r * M * ldc;
        z0 = (float *)ws_get(e, "adj0", (size_t)D * Zr * ldz * 4);
        z1 = (float *)ws_get(e, "adj1", (size_t)D * Zr * ldz * 4);
        mom = (float *)ws_get(e, "adam_m", (size_t)D * np * 4);
        var = (float *)ws_get(e, "adam_v", (size_t)D * np * 4);
        if (!z0 || !z1 || !mom || !var) return NYB200_ERR_OOM;
        NYB_TRY(prepare_transposed(e, *net, tensor));
        NYB_CUDA(e, cudaMemsetAsync(mom, 0, (size_t)D * np * 4, e->stream));
        NYB_CUDA(e, cudaMemsetAsync(var, 0, (size_t)D * np * 4, e->stream));
    }
    float *mom_up = nullptr, *var_up = nullptr;
    if (dual) {
        mom_up = (float *)ws_get(e, "adam_mu", (size_t)D * np * 4);
        var_up = (float *)ws_get(e, "adam_vu", (size_t)D * np * 4);
        if (!mom_up || !var_up) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(mom_up, 0, (size_t)D * np * 4, e->stream));
        NYB_CUDA(e, cudaMemsetAsync(var_up, 0, (size_t)D * np * 4, e->stream));
    }
    NYB_WS(best_lo, float *, e, "best_lo", (size_t)D * S * 4);
    NYB_WS(best_hi, float *, e, "best_hi", (size_t)D * S * 4);
    // per-domain state of the stopping rules; AMSGrad's running maxima
    NYB_WS(opt_words, int *, e, "opt_state", (size_t)D * 16);
    OptState ost;
    ost.stopped = opt_words; ost.maxg = (unsigned *)(opt_words + D); ost.best_obj = (float *)(opt_words + 2 * (size_t)D);
    ost.no_improve = opt_words + 3 * (size_t)D;
    NYB_CUDA(e, cudaMemsetAsync(opt_words, 0, (size_t)D * 16, e->stream));
    launch_fill_f32(e, ost.best_obj, (size_t)D, -INFINITY);
    const bool rules = (cfg.tolerance > 0.f || cfg.patience > 0) && T > 1 && !grad_host;
    float *vmax = nullptr, *vmax_up = nullptr;
    if (cfg.rule == 2 && T > 1) {
        vmax = (float *)ws_get(e, "adam_vmax", (size_t)D * np * 4);
        if (!vmax) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(vmax, 0, (size_t)D * np * 4, e->stream));
        if (dual) {
            vmax_up = (float *)ws_get(e, "adam_vmax_up", (size_t)D * np * 4);
            if (!vmax_up) return NYB200_ERR_OOM;
            NYB_CUDA(e, cudaMemsetAsync(vmax_up, 0, (size_t)D * np * 4, e->stream));
        }
    }
    const int save_from = (int)((float)T * cfg.start_save_best);  // zero-based iteration threshold of should_save_best
    int *only_row = nullptr;
    if (cfg.objective == 1) {
        only_row = (int *)ws_get(e, "opt_row", (size_t)D * 4);
        if (!only_row) return NYB200_ERR_OOM;
    }
    int *derr = nullptr;
    if (tensor) {
        derr = (int *)ws_get(e, "umma_err", 256);
        if (!derr) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(derr, 0, 4, e->stream));
    }
    float *grad_dev = nullptr;
    if (grad_host) {
        grad_dev = (float *)ws_get(e, "par_grad", (size_t)D * np * 4);
        if (!grad_dev) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(grad_dev, 0, (size_t)D * np * 4, e->stream));
    }

    Timing &tm = e->timing;
    fold_timing(tm);
    cudaEventRecord(tm.ev[0], e->stream);
    if (!b.external_tables) NYB_TRY(run_forward(e, *net, b, p, b.mode));
    if (dual) {
        long na = (long)D * np;
        k_init_alpha_up<<<(unsigned)((na + 255) / 256), 256, 0, e->stream>>>(na, p.tab, p.alpha_up);
        e->launches++;
    }
    cudaEventRecord(tm.ev[1], e->stream);
    const long nres = (long)D * S;
    const unsigned gres = (unsigned)((nres + 255) / 256);
    for (int t = 1; t <= T; ++t) {
        NYB_DEADLINE(e, "optimisation");
        const bool last = (t == T);
        NYB_TRY(run_backward(e, *net, b, p, last ? nullptr : ckpt.data(), ldc));
        const int save = (t == 1 || (t - 1) > save_from || last || !(cfg.start_save_best > 0.f)) ? 1 : 0;
        k_fold_best<<<gres, 256, 0, e->stream>>>(nres, t == 1, p.out_lo, p.out_hi, best_lo, best_hi, S, save, ost.stopped);
        e->launches++;
        if (last) break;
        if (only_row) {
            k_argmin_row<<<(unsigned)((D + 255) / 256), 256, 0, e->stream>>>(D, S, p.out_lo, only_row);
            e->launches++;
        }
        AdamStep h;
        float decay = powf(cfg.lr_decay, (float)(t - 1));
        h.lr_alpha = cfg.lr_alpha * decay; h.lr_beta = cfg.lr_beta * decay;
        h.beta1 = b1; h.beta2 = b2; h.epsilon = eps; h.clip_beta = cfg.clip_beta; h.rule = cfg.rule;
        h.bc1 = fmaxf(1.f - powf(b1, (float)t), 1.1920929e-7f);
        h.bc2 = fmaxf(1.f - powf(b2, (float)t), 1.1920929e-7f);
        long nseed = (long)D * Zr * nv.dims[0];
        k_adjoint_seed<<<(unsigned)((nseed + 255) / 256), 256, 0, e->stream>>>(D, S, R, Zr, nv.dims[0], p.a_final, p.lda, p.in_lo,
                                                                              p.in_hi, (long)b.box_stride, z0, ldz);
        e->launches++;
        float *zc = z0, *zn = z1;
        // adjoints of relu(pre_k) that a later layer's identity branch still needs, one buffer per open source layer
        struct OpenAdj { float *buf; int src; };
        std::vector<OpenAdj> open_adj;
        auto adj_slot = [&](size_t slot) -> float * {
            const std::string name = slot == 0 ? std::string("adj_skip") : "adj_skip_" + std::to_string(slot);
            return (float *)ws_get(e, name.c_str(), (size_t)D * Zr * ldz * 4);
        };
        for (int k = 0; k < L - 1; ++k) {
            int K = nv.dims[k], N = nv.dims[k + 1];
            if (net->is_conv(k) && tensor) NYB_TRY(conv_forward_tensor(e, *net, k, D * Zr, zc, ldz, zn, ldz, derr));
            else if (net->is_conv(k)) launch_conv_plain(e, net->geom[k], D * Zr, zc, ldz, nv.W[k], zn, ldz);
            else if (tensor) NYB_TRY(launch_umma(e, net->umma_adj[k], D * Zr, zc, ldz, zn, ldz, derr));
            else launch_gemm_f64(e, D * Zr, N, K, zc, ldz, net->wt[k], N, zn, ldz, 1, nullptr, nullptr, 0, nullptr);
            if (net->skip_of(k) >= 0) {
                // residual block: pre_k = W z + b + relu(pre_j), so the adjoint of relu(pre_j) joins here
                for (size_t oi = 0; oi < open_adj.size(); ++oi) {
                    if (open_adj[oi].src != net->skip_of(k)) continue;
                    long tot = (long)D * Zr * N;
                    k_add_adjoint<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>((long)D * Zr, N, zn, ldz, open_adj[oi].buf, ldz);
                    e->launches++;
                    bool later = false;   // does another layer further on take the same branch?
                    for (int kk = k + 1; kk < L - 1; ++kk) later |= net->skip_of(kk) == open_adj[oi].src;
                    if (!later) open_adj.erase(open_adj.begin() + (long)oi);
                    break;
                }
            }
            long nt = (long)D * N;
            k_adjoint_relu<<<(unsigned)((nt + 255) / 256), 256, 0, e->stream>>>(N, nv.pre_off[k], D, S, R, Zr, np, zn, ldz, nv.b[k],
                                                                               ckpt[k], ldc, p.tab, p.code, p.pre_lo,
                                                                               p.pre_hi, mom, var, only_row, p.alpha_up, mom_up, var_up, grad_dev, h,
                                                                               rules ? ost.stopped : nullptr, rules ? ost.maxg : nullptr, vmax, vmax_up);
            e->launches++;
            bool opens = false;  // is this layer's post-activation adjoint skipped forward to a later layer?
            for (int kk = k + 2; kk < L - 1; ++kk) opens |= net->skip_of(kk) == k;
            if (opens) {
                size_t slot = 0;
                for (bool taken = true; taken; ) {
                    taken = false;
                    for (const OpenAdj &o : open_adj) if (o.buf == adj_slot(slot)) { taken = true; ++slot; break; }
                }
                float *zstash = adj_slot(slot);
                if (!zstash) return NYB200_ERR_OOM;
                NYB_CUDA(e, cudaMemcpyAsync(zstash, zn, (size_t)D * Zr * ldz * 4, cudaMemcpyDeviceToDevice, e->stream));
                open_adj.push_back({zstash, k});
            }
            float *tmp = zc; zc = zn; zn = tmp;
        }
        if (grad_host) break;  // gradient export: one evaluation and its adjoint, no second pass
        if (rules) {
            k_opt_rules<<<(unsigned)((D + 255) / 256), 256, 0, e->stream>>>(D, S, t, cfg.objective, cfg.tolerance, cfg.patience, p.out_lo, ost);
            e->launches++;
        }
    }
    b.opt_iterations = T;
    static const float inf_word = INFINITY;
    NYB_CUDA(e, cudaMemcpyAsync(p.min_lower, &inf_word, 4, cudaMemcpyHostToDevice, e->stream));
    k_publish_best<<<gres, 256, 0, e->stream>>>(D, S, p.flags, best_lo, best_hi, p.out_lo, p.out_hi, p.min_lower);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    cudaEventRecord(tm.ev[2], e->stream);
    tm.pending = true;
    b.ran = true;
    b.finished = false;
    b.optimized = true;
    b.refined = 0;
    if (grad_host) {
        if (L >= 2) {
            NYB_CUDA(e, cudaMemcpy2DAsync(grad_host, (size_t)nv.n_pre * 4, grad_dev, (size_t)np * 4, (size_t)nv.n_pre * 4, (size_t)D,
                                          cudaMemcpyDeviceToHost, e->stream));
            NYB_CUDA(e, cudaStreamSynchronize(e->stream));
        } else {
            memset(grad_host, 0, (size_t)D * nv.n_pre * 4);
        }
    }
    return NYB200_OK;
}

// Re-evaluates the final parameters of an optimised batch with binary64 contractions and folds the result
// into the best bounds (called after the fast path flagged a visible rounding charge on the last iterate).
int refine_optimized(nyb200_engine *e, Net &net, Batch &b, BatchPtrs &p) {
    NYB_WS(best_lo, float *, e, "best_lo", (size_t)b.D * b.S * 4);
    NYB_WS(best_hi, float *, e, "best_hi", (size_t)b.D * b.S * 4);
    int saved = e->path;
    e->path = NYB200_PATH_F64;
    int st = run_backward(e, net, b, p, nullptr, 0);
    e->path = saved;
    NYB_TRY(st);
    const long nres = (long)b.D * b.S;
    const unsigned gres = (unsigned)((nres + 255) / 256);
    k_fold_best<<<gres, 256, 0, e->stream>>>(nres, 0, p.out_lo, p.out_hi, best_lo, best_hi);
    static const float inf_word = INFINITY;
    NYB_CUDA(e, cudaMemcpyAsync(p.min_lower, &inf_word, 4, cudaMemcpyHostToDevice, e->stream));
    k_publish_best<<<gres, 256, 0, e->stream>>>(b.D, b.S, p.flags, best_lo, best_hi, p.out_lo, p.out_hi, p.min_lower);
    e->launches += 2;
    NYB_CUDA(e, cudaGetLastError());
    return NYB200_OK;
}

int download_params(nyb200_engine *e, float *alpha, float *beta) {
    if (!e->batch.valid || !e->batch.ran) return set_err(e, NYB200_ERR_INVALID, "no batch has been run");
    Net *net;
    NYB_TRY(find_net(e, e->batch.net_id, &net));
    Batch &b = e->batch;
    BatchPtrs p;
    NYB_TRY(batch_ptrs(e, *net, b, p));
    const NetView &nv = net->v;
    size_t na = (size_t)b.D * nv.n_pre, nb = (size_t)b.D * (size_t)(b.max_splits > 0 ? b.max_splits : 0);
    float *da = nullptr, *db = nullptr;
    if (alpha) { da = (float *)ws_get(e, "par_alpha", na * 4); if (!da) return NYB200_ERR_OOM; }
    if (beta && nb) { db = (float *)ws_get(e, "par_beta", nb * 4); if (!db) return NYB200_ERR_OOM; }
    size_t total = na + nb;
    k_gather_params<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(nv, b.D, b.max_splits, p.tab, p.splits, p.nsplits,
                                                                           da, db);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    if (da) NYB_CUDA(e, cudaMemcpyAsync(alpha, da, na * 4, cudaMemcpyDeviceToHost, e->stream));
    if (db) NYB_CUDA(e, cudaMemcpyAsync(beta, db, nb * 4, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    return NYB200_OK;
}

int download_alpha_upper(nyb200_engine *e, float *alpha_up) {
    if (!e->batch.valid || !e->batch.ran) return set_err(e, NYB200_ERR_INVALID, "no batch has been run");
    Net *net;
    NYB_TRY(find_net(e, e->batch.net_id, &net));
    BatchPtrs p;
    NYB_TRY(batch_ptrs(e, *net, e->batch, p));
    const NetView &nv = net->v;
    size_t w = (size_t)nv.n_pre * 4;
    if (p.alpha_up) {
        NYB_CUDA(e, cudaMemcpy2DAsync(alpha_up, w, p.alpha_up, (size_t)nv.nps * 4, w, (size_t)e->batch.D, cudaMemcpyDeviceToHost, e->stream));
        NYB_CUDA(e, cudaStreamSynchronize(e->stream));
        return NYB200_OK;
    }
    return download_params(e, alpha_up, nullptr);  // shared slopes: the upper path uses the lower path's
}

}  // namespace nyb

extern "C" {

int32_t nyb200_batch_download_alpha_upper(nyb200_engine *e, float *alpha_up) {
    if (!e || !alpha_up) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::download_alpha_upper(e, alpha_up);
}

int32_t nyb200_batch_optimize(nyb200_engine *e, const nyb200_opt_config *cfg) {
    if (!e || !cfg) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::optimize_batch(e, *cfg);
}

int32_t nyb200_batch_download_opt_evaluations(nyb200_engine *e, int32_t *evaluations) {
    if (!e || !evaluations) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    if (!e->batch.valid || !e->batch.optimized) return nyb::set_err(e, NYB200_ERR_INVALID, "no optimisation has been run on this batch");
    const int D = e->batch.D;
    int *w = (int *)nyb::ws_get(e, "opt_state", (size_t)D * 16);
    if (!w) return NYB200_ERR_OOM;
    st = cudaMemcpyAsync(evaluations, w, (size_t)D * 4, cudaMemcpyDeviceToHost, e->stream);
    if (st == cudaSuccess) st = cudaStreamSynchronize(e->stream);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "opt evaluations");
    for (int d = 0; d < D; ++d) evaluations[d] = evaluations[d] > 0 ? evaluations[d] + 1 : e->batch.opt_iterations;
    return NYB200_OK;
}

int32_t nyb200_batch_gradient(nyb200_engine *e, int32_t objective, float *grad) {
    if (!e || !grad) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    nyb200_opt_config cfg = {};
    cfg.iterations = 2;  // one evaluation with checkpoints and its adjoint; the second evaluation is skipped
    cfg.lr_decay = 1.f;
    cfg.objective = objective;
    return nyb::optimize_batch(e, cfg, grad);
}

int32_t nyb200_batch_download_params(nyb200_engine *e, float *alpha, float *beta) {
    if (!e) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::download_params(e, alpha, beta);
}

}  // extern "C"
