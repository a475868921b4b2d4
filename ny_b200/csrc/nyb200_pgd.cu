// PGD attack batched over restarts: concrete forward pass, exact gradient of the worst specification row and
// the AdamClipping step, all K restarts in lock-step on the device.
//
// The forward products Z * W_k^T and the backward products G * W_k run on the same contraction kernels as the
// bound propagation (tcgen05 3xTF32, or binary64 when that path is selected); convolutions use the plain
// forward convolution and the transposed-convolution path.  The attack only proposes points: the value
// returned for each restart comes from a final evaluation of its best point with binary64 contractions.
#include "nyb200_internal.cuh"

namespace nyb {

namespace {

struct PgdStep {
    float step, beta1, beta2, epsilon, bc2;
};

// z += bias; optionally ReLU.  Post-activations are kept: z > 0 afterwards is exactly the gradient mask.
__global__ void k_bias_act(long rows, int n, float *__restrict__ Z, int ld, const float *__restrict__ bias, int relu) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= rows * n) return;
    long r = t / n;
    int j = (int)(t - r * n);
    float v = Z[r * ld + j] + (bias ? bias[j] : 0.f);
    Z[r * ld + j] = relu ? fmaxf(v, 0.f) : v;
}

// Per restart: margins spec[s] . y, the smallest one and its row.  `track`: the step's point competes for the
// restart's best objective (improved[r] tells k_keep_best to copy the point).  `seed`: G[r] = spec[row].
__global__ void k_pgd_objective(int K, int S, int nL, const float *__restrict__ Y, int ldy, const float *__restrict__ spec,
                                float *__restrict__ best, int *__restrict__ improved, float *__restrict__ G, int ldg,
                                float *__restrict__ value_out) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= K) return;
    const float *y = Y + (long)r * ldy;
    float mv = INFINITY;
    int ms = 0;
    bool bad = false;
    for (int s = 0; s < S; ++s) {
        double acc = 0.0;
        for (int j = 0; j < nL; ++j) acc = fma((double)spec[s * nL + j], (double)y[j], acc);
        float m = (float)acc;
        if (isnan(m)) bad = true;
        if (m < mv) { mv = m; ms = s; }
    }
    if (bad) mv = NAN;
    if (value_out) value_out[r] = mv;
    if (best) {
        int imp = (!bad && mv < best[r]) ? 1 : 0;
        if (imp) best[r] = mv;
        improved[r] = imp;
    }
    if (G)
        for (int j = 0; j < nL; ++j) G[(long)r * ldg + j] = spec[ms * nL + j];
}

__global__ void k_keep_best(int K, int n0, const float *__restrict__ X, int ldx, const int *__restrict__ improved,
                            float *__restrict__ best_x) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)K * n0) return;
    int r = (int)(t / n0), j = (int)(t % n0);
    if (improved[r]) best_x[(long)r * n0 + j] = X[(long)r * ldx + j];
}

// G *= [Zpost > 0]
__global__ void k_relu_mask(long rows, int n, float *__restrict__ G, int ldg, const float *__restrict__ Z, int ldz) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= rows * n) return;
    long r = t / n;
    int j = (int)(t - r * n);
    if (!(Z[r * ldz + j] > 0.f)) G[r * ldg + j] = 0.f;
}

// AdamClipping step (pgd_attack/adam_state.rs:46-88), descending the objective.  A restart whose gradient
// holds a NaN skips the step (attacker/batched.rs:93-104): rows flagged in nan_row are left alone.
__global__ void k_pgd_step(int K, int n0, float *__restrict__ X, int ldx, const float *__restrict__ G, int ldg,
                           float *__restrict__ mom, float *__restrict__ var, const float *__restrict__ lo,
                           const float *__restrict__ hi, const int *__restrict__ nan_row, PgdStep h) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)K * n0) return;
    int r = (int)(t / n0), j = (int)(t % n0);
    if (nan_row[r]) return;
    float g = G[(long)r * ldg + j];
    float m = h.beta1 * mom[t] + (1.f - h.beta1) * g;
    float v = h.beta2 * var[t] + (1.f - h.beta2) * g * g;
    mom[t] = m; var[t] = v;
    float denom = sqrtf(v / h.bc2) + h.epsilon;
    float dir = 0.f;
    if (isfinite(denom) && isfinite(m)) {
        float q = m / denom;
        dir = isnan(q) ? 0.f : copysignf(1.f, q);  // sign(+0) = +1, sign(-0) = -1
    }
    float x = X[(long)r * ldx + j] - dir * h.step;
    float l = lo[j], u = hi[j];
    x = isnan(x) ? l : fminf(fmaxf(x, l), u);
    X[(long)r * ldx + j] = x;
}

__global__ void k_nan_rows(int K, int n0, const float *__restrict__ G, int ldg, int *__restrict__ nan_row) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= K) return;
    int bad = 0;
    for (int j = lane; j < n0; j += 32) bad |= isnan(G[(long)warp * ldg + j]) ? 1 : 0;
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) nan_row[warp] = bad;
}

// Y[r, j] += X[r, j]
__global__ void k_add_rows(long rows, int n, float *__restrict__ Y, int ldy, const float *__restrict__ X, int ldx) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= rows * n) return;
    long r = t / n;
    int j = (int)(t - r * n);
    Y[r * ldy + j] += X[r * ldx + j];
}

// out[r] = X[r, :] . Y[r, :], one warp per row, binary64 accumulation
__global__ void k_row_dot(int rows, int n, const float *__restrict__ X, int ldx, const float *__restrict__ Y, int ldy,
                          float *__restrict__ out) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    double acc = 0.0;
    for (int j = lane; j < n; j += 32) acc = fma((double)X[(long)warp * ldx + j], (double)Y[(long)warp * ldy + j], acc);
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[warp] = (float)acc;
}

__global__ void k_fill_f32(float *p, long n, float v) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) p[t] = v;
}

}  // namespace

// Concrete forward pass of `rows` points X [rows x ldx] through the network; act[k] receives layer k's
// post-activation output (row stride ld), act[L-1] the network output.
static int pgd_forward(nyb200_engine *e, Net &net, bool tensor, int rows, const float *X, int ldx, float *const *act, int ld,
                       int *derr) {
    const NetView &nv = net.v;
    const float *cur = X;
    int ldc = ldx;
    for (int k = 0; k < nv.L; ++k) {
        int K = nv.dims[k], N = nv.dims[k + 1];
        if (net.is_conv(k) && tensor) NYB_TRY(conv_forward_tensor(e, net, k, rows, cur, ldc, act[k], ld, derr));
        else if (net.is_conv(k)) launch_conv_plain(e, net.geom[k], rows, cur, ldc, nv.W[k], act[k], ld);
        else if (tensor) NYB_TRY(launch_umma(e, net.umma_adj[k], rows, cur, ldc, act[k], ld, derr));
        else launch_gemm_f64(e, rows, N, K, cur, ldc, net.wt[k], N, act[k], ld, 1, nullptr, nullptr, 0, nullptr);
        long tot = (long)rows * N;
        if (net.skip_of(k) >= 0) {  // residual: the block's input joins before the bias and the ReLU
            k_add_rows<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>(rows, N, act[k], ld, act[net.skip_of(k)], ld);
            e->launches++;
        }
        k_bias_act<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>(rows, N, act[k], ld, nv.b[k], k < nv.L - 1 ? 1 : 0);
        e->launches++;
        cur = act[k];
        ldc = ld;
    }
    return NYB200_OK;
}

// Exact gradient chain of K rows: G_k = (G_{k+1} . [mask_k > 0]) W_k from the output down to the input, where
// mask_k is act[k] (a concrete forward pass's activations, or caller-supplied 0/1 masks).  G0 holds the output
// cotangents on entry; *result points at the buffer (G0 or G1) that holds the input gradients.
static int pgd_backward(nyb200_engine *e, Net &net, bool tensor, int K, float *G0, float *G1, float *const *act, int ld,
                        int *derr, float **result) {
    const NetView &nv = net.v;
    const int L = nv.L;
    cudaStream_t st = e->stream;
    double *cols64 = nullptr;
    float *g = G0, *gn = G1;
    struct OpenGrad { float *buf; int src; };   // gradients kept for identity branches (blocks may nest)
    std::vector<OpenGrad> open_grad;
    auto grad_slot = [&](size_t slot) -> float * {
        const std::string name = slot == 0 ? std::string("pgd_skip") : "pgd_skip_" + std::to_string(slot);
        return (float *)ws_get(e, name.c_str(), (size_t)K * ld * 4);
    };
    for (int k = L - 1; k >= 0; --k) {
        int Kd = nv.dims[k + 1], N = nv.dims[k];
        for (size_t oi = 0; oi < open_grad.size();) {  // g is the gradient of relu(pre_k): identity branches join here
            if (open_grad[oi].src != k) { ++oi; continue; }
            long tot = (long)K * Kd;
            k_add_rows<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(K, Kd, g, ld, open_grad[oi].buf, ld);
            e->launches++;
            open_grad.erase(open_grad.begin() + (long)oi);
        }
        if (k < L - 1) {
            long tot = (long)K * Kd;
            k_relu_mask<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(K, Kd, g, ld, act[k], ld);
            e->launches++;
        }
        if (net.skip_of(k) >= 0) {  // the gradient of pre_k also reaches relu(pre_j) directly
            size_t slot = 0;
            for (bool taken = true; taken; ) {
                taken = false;
                for (const OpenGrad &o : open_grad) if (o.buf == grad_slot(slot)) { taken = true; ++slot; break; }
            }
            float *gstash = grad_slot(slot);
            if (!gstash) return NYB200_ERR_OOM;
            NYB_CUDA(e, cudaMemcpyAsync(gstash, g, (size_t)K * ld * 4, cudaMemcpyDeviceToDevice, st));
            open_grad.push_back({gstash, net.skip_of(k)});
        }
        if (net.is_conv(k) && tensor) {
            const ConvGeom &cg = net.geom[k];
            const int plane = cg.oh * cg.ow, taps = cg.ic * cg.kh * cg.kw;
            float *cols = (float *)ws_get(e, "conv_cols", (size_t)K * plane * taps * 4);
            if (!cols) return NYB200_ERR_OOM;
            NYB_TRY(launch_umma(e, net.umma[k], K * plane, g, ld, cols, taps, derr, plane));
            launch_col2im(e, cg, K, cols, gn, ld);
        } else if (net.is_conv(k)) {
            const ConvGeom &cg = net.geom[k];
            cols64 = (double *)ws_get(e, "conv_cols", (size_t)K * cg.oh * cg.ow * cg.ic * cg.kh * cg.kw * 8);
            if (!cols64) return NYB200_ERR_OOM;
            launch_conv_transpose(e, cg, K, g, ld, gn, ld, nv.W[k], 1, nullptr, nullptr, 0, nullptr, cols64);
        } else if (tensor) {
            NYB_TRY(launch_umma(e, net.umma[k], K, g, ld, gn, ld, derr));
        } else {
            launch_gemm_f64(e, K, N, Kd, g, ld, nv.W[k], N, gn, ld, 1, nullptr, nullptr, 0, nullptr);
        }
        float *tmp = g; g = gn; gn = tmp;
    }
    *result = g;
    return NYB200_OK;
}

int pgd_attack(nyb200_engine *e, int net_id, const float *spec, int S, const float *in_lo, const float *in_hi,
               const float *x0, int K, const nyb200_pgd_config &cfg, float *best_margin, float *best_x, int *counterexample) {
    Net *net;
    NYB_TRY(find_net(e, net_id, &net));
    const NetView &nv = net->v;
    if (S <= 0 || K <= 0) return set_err(e, NYB200_ERR_SHAPE, "S and K must be positive");
    if (cfg.steps < 0 || !(cfg.step_size >= 0.f)) return set_err(e, NYB200_ERR_INVALID, "steps and step_size must be >= 0");
    const int L = nv.L, n0 = nv.dims[0], nL = nv.dims[L];
    const bool tensor = e->path == NYB200_PATH_TF32X3;
    const float b1 = cfg.beta1 > 0.f ? cfg.beta1 : 0.9f, b2 = cfg.beta2 > 0.f ? cfg.beta2 : 0.999f;
    const float eps = cfg.epsilon > 0.f ? cfg.epsilon : 1e-8f, decay = cfg.lr_decay > 0.f ? cfg.lr_decay : 0.99f;
    const int ld = (net->max_dim + 7) & ~7;
    e->batch = Batch();  // workspace names are shared with the resident batch

    NYB_TRY(prepare_transposed(e, *net, tensor));
    if (tensor) NYB_TRY(prepare_backward_operands(e, *net));
    NYB_WS(dspec, float *, e, "spec", (size_t)S * nL * 4);
    NYB_WS(dlo, float *, e, "in_lo", (size_t)n0 * 4);
    NYB_WS(dhi, float *, e, "in_hi", (size_t)n0 * 4);
    NYB_WS(X, float *, e, "pgd_x", (size_t)K * ld * 4);
    NYB_WS(acts, float *, e, "pgd_act", (size_t)L * K * ld * 4);
    NYB_WS(G0, float *, e, "pgd_g0", (size_t)K * ld * 4);
    NYB_WS(G1, float *, e, "pgd_g1", (size_t)K * ld * 4);
    NYB_WS(mom, float *, e, "pgd_m", (size_t)K * n0 * 4);
    NYB_WS(var, float *, e, "pgd_v", (size_t)K * n0 * 4);
    NYB_WS(dbest, float *, e, "pgd_best", (size_t)K * 4);
    NYB_WS(dbx, float *, e, "pgd_best_x", (size_t)K * n0 * 4);
    NYB_WS(dimp, int *, e, "pgd_improved", (size_t)K * 4);
    NYB_WS(dnan, int *, e, "pgd_nan", (size_t)K * 4);
    int *derr = nullptr;
    if (tensor) {
        derr = (int *)ws_get(e, "umma_err", 256);
        if (!derr) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(derr, 0, 4, e->stream));
    }
    std::vector<float *> act((size_t)L);
    for (int k = 0; k < L; ++k) act[k] = acts + (size_t)k * K * ld;
    cudaStream_t st = e->stream;
    NYB_CUDA(e, cudaMemcpyAsync(dspec, spec, (size_t)S * nL * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(dlo, in_lo, (size_t)n0 * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(dhi, in_hi, (size_t)n0 * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpy2DAsync(X, (size_t)ld * 4, x0, (size_t)n0 * 4, (size_t)n0 * 4, (size_t)K, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpy2DAsync(dbx, (size_t)n0 * 4, x0, (size_t)n0 * 4, (size_t)n0 * 4, (size_t)K, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemsetAsync(mom, 0, (size_t)K * n0 * 4, st));
    NYB_CUDA(e, cudaMemsetAsync(var, 0, (size_t)K * n0 * 4, st));
    k_fill_f32<<<(K + 255) / 256, 256, 0, st>>>(dbest, K, INFINITY);
    e->launches++;
    const unsigned gk = (unsigned)((K + 255) / 256);
    const long nx = (long)K * n0;
    const unsigned gx = (unsigned)((nx + 255) / 256);

    for (int t = 1; t <= cfg.steps + 1; ++t) {
        NYB_DEADLINE(e, "attack");
        NYB_TRY(pgd_forward(e, *net, tensor, K, X, ld, act.data(), ld, derr));
        const bool last = t == cfg.steps + 1;
        k_pgd_objective<<<gk, 256, 0, st>>>(K, S, nL, act[L - 1], ld, dspec, dbest, dimp, last ? nullptr : G0, ld, nullptr);
        k_keep_best<<<gx, 256, 0, st>>>(K, n0, X, ld, dimp, dbx);
        e->launches += 2;
        if (last) break;
        float *g = nullptr;
        NYB_TRY(pgd_backward(e, *net, tensor, K, G0, G1, act.data(), ld, derr, &g));
        k_nan_rows<<<(unsigned)(((long)K * 32 + 255) / 256), 256, 0, st>>>(K, n0, g, ld, dnan);
        PgdStep h;
        float bc1 = 1.f - powf(b1, (float)t);
        h.bc2 = 1.f - powf(b2, (float)t);
        h.step = cfg.step_size * powf(decay, (float)(t - 1)) / bc1;
        h.beta1 = b1; h.beta2 = b2; h.epsilon = eps;
        k_pgd_step<<<gx, 256, 0, st>>>(K, n0, X, ld, g, ld, mom, var, dlo, dhi, dnan, h);
        e->launches += 2;
    }
    // independent evaluation of every restart's best point with binary64 contractions
    NYB_TRY(prepare_transposed(e, *net, false));
    NYB_TRY(pgd_forward(e, *net, false, K, dbx, n0, act.data(), ld, derr));
    k_pgd_objective<<<gk, 256, 0, st>>>(K, S, nL, act[L - 1], ld, dspec, nullptr, nullptr, nullptr, 0, dbest);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaMemcpyAsync(best_margin, dbest, (size_t)K * 4, cudaMemcpyDeviceToHost, st));
    if (best_x) NYB_CUDA(e, cudaMemcpyAsync(best_x, dbx, (size_t)K * n0 * 4, cudaMemcpyDeviceToHost, st));
    int herr = 0;
    if (derr) NYB_CUDA(e, cudaMemcpyAsync(&herr, derr, 4, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaStreamSynchronize(st));
    if (herr) return set_err(e, NYB200_ERR_INTERNAL, "tcgen05 pipeline wait expired (code " + std::to_string(herr) + ")");
    int arg = -1;
    float mv = INFINITY;
    for (int r = 0; r < K; ++r)
        if (best_margin[r] < mv) { mv = best_margin[r]; arg = r; }
    if (counterexample) *counterexample = (arg >= 0 && mv <= 0.f) ? arg : -1;
    return NYB200_OK;
}


// Exact point gradients of K restarts: spec_rows[k] . df/dx, ReLU derivatives from the forward pass at x or from
// caller-supplied masks.
int point_vjp(nyb200_engine *e, int net_id, int K, const float *x, const float *masks, const float *spec_rows, float *grads,
              float *values) {
    Net *net;
    NYB_TRY(find_net(e, net_id, &net));
    const NetView &nv = net->v;
    if (K <= 0) return set_err(e, NYB200_ERR_SHAPE, "K must be positive");
    if ((x != nullptr) == (masks != nullptr)) return set_err(e, NYB200_ERR_INVALID, "exactly one of x and masks must be given");
    if (values && !x) return set_err(e, NYB200_ERR_INVALID, "values need the points x");
    const int L = nv.L, n0 = nv.dims[0], nL = nv.dims[L];
    const bool tensor = e->path == NYB200_PATH_TF32X3;
    const int ld = (net->max_dim + 7) & ~7;
    e->batch = Batch();  // workspace names are shared with the resident batch
    NYB_TRY(prepare_transposed(e, *net, tensor));
    if (tensor) NYB_TRY(prepare_backward_operands(e, *net));
    NYB_WS(X, float *, e, "pgd_x", (size_t)K * ld * 4);
    NYB_WS(acts, float *, e, "pgd_act", (size_t)L * K * ld * 4);
    NYB_WS(G0, float *, e, "pgd_g0", (size_t)K * ld * 4);
    NYB_WS(G1, float *, e, "pgd_g1", (size_t)K * ld * 4);
    NYB_WS(dval, float *, e, "pgd_best", (size_t)K * 4);
    int *derr = nullptr;
    if (tensor) {
        derr = (int *)ws_get(e, "umma_err", 256);
        if (!derr) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(derr, 0, 4, e->stream));
    }
    std::vector<float *> act((size_t)L);
    for (int k = 0; k < L; ++k) act[k] = acts + (size_t)k * K * ld;
    cudaStream_t st = e->stream;
    NYB_CUDA(e, cudaMemcpy2DAsync(G0, (size_t)ld * 4, spec_rows, (size_t)nL * 4, (size_t)nL * 4, (size_t)K, cudaMemcpyHostToDevice, st));
    if (x) {
        NYB_CUDA(e, cudaMemcpy2DAsync(X, (size_t)ld * 4, x, (size_t)n0 * 4, (size_t)n0 * 4, (size_t)K, cudaMemcpyHostToDevice, st));
        NYB_TRY(pgd_forward(e, *net, tensor, K, X, ld, act.data(), ld, derr));
        if (values) {
            k_row_dot<<<(unsigned)(((long)K * 32 + 255) / 256), 256, 0, st>>>(K, nL, act[L - 1], ld, G0, ld, dval);
            e->launches++;
        }
    } else {
        for (int k = 0; k < L - 1; ++k)  // layer k's mask block of every restart's [n_pre] row
            NYB_CUDA(e, cudaMemcpy2DAsync(act[k], (size_t)ld * 4, masks + nv.pre_off[k], (size_t)nv.n_pre * 4,
                                          (size_t)nv.dims[k + 1] * 4, (size_t)K, cudaMemcpyHostToDevice, st));
    }
    float *g = nullptr;
    NYB_TRY(pgd_backward(e, *net, tensor, K, G0, G1, act.data(), ld, derr, &g));
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaMemcpy2DAsync(grads, (size_t)n0 * 4, g, (size_t)ld * 4, (size_t)n0 * 4, (size_t)K, cudaMemcpyDeviceToHost, st));
    if (values) NYB_CUDA(e, cudaMemcpyAsync(values, dval, (size_t)K * 4, cudaMemcpyDeviceToHost, st));
    int herr = 0;
    if (derr) NYB_CUDA(e, cudaMemcpyAsync(&herr, derr, 4, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaStreamSynchronize(st));
    if (herr) return set_err(e, NYB200_ERR_INTERNAL, "tcgen05 pipeline wait expired (code " + std::to_string(herr) + ")");
    for (long i = 0; i < (long)K * n0; ++i)  // never a silently wrong gradient batch
        if (!(grads[i] == grads[i]) || grads[i] - grads[i] != 0.f) return set_err(e, NYB200_ERR_NUMERICAL, "non-finite point gradient");
    return NYB200_OK;
}

}  // namespace nyb

extern "C" int32_t nyb200_point_vjp_batched(nyb200_engine *e, int32_t net_id, int32_t K, const float *x, const float *masks,
                                            const float *spec_rows, float *grads, float *values) {
    if (!e || !spec_rows || !grads) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::point_vjp(e, net_id, K, x, masks, spec_rows, grads, values);
}

extern "C" int32_t nyb200_pgd_attack(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                                     const float *in_hi, const float *x0, int32_t K, const nyb200_pgd_config *cfg,
                                     float *best_margin, float *best_x, int32_t *counterexample) {
    if (!e || !spec || !in_lo || !in_hi || !x0 || !cfg || !best_margin) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::pgd_attack(e, net_id, spec, S, in_lo, in_hi, x0, K, *cfg, best_margin, best_x, counterexample);
}
