// CUDA kernels of the bound-propagation engine (sm_100a): interval forward pass, ReLU
// relaxation with alpha slopes and beta multipliers, binary64-accumulated A*W contraction,
// concretisation and branching.  The tcgen05 contraction lives in nyb200_umma.cu.
//
// Soundness bookkeeping used by every kernel here.  Each row of the coefficient tensor A
// carries three binary64 scalars:
//   rb    the bias accumulated so far (round-to-nearest sums of exact fp32 x fp32 products),
//   rabs  the sum of the magnitudes of everything added to rb (bounds the rounding of rb),
//   rpen  a non-negative penalty: every rounding committed on a coefficient is immediately
//         multiplied by the largest magnitude the variable it multiplies can take (known from
//         the interval forward pass) and added here.  At the end the lower bound is
//         rb + (concretised A) - rpen - slack, rounded toward -inf; the upper bound mirrors it.
// This is the role the per-coefficient error matrices play in the reference
// (crates/ny-propagate/src/layers/linear/crown_single.rs:2092-2103, discharged at
// bounds/concretize.rs:443-466), but discharged layer by layer against the layer's own interval
// (as the reference's device path does with node_abs/frontier_abs,
// crates/ny-core/src/gemm.rs:2939-2952) so that no |W| chain is ever formed.
#include "nyb200_internal.cuh"
#include "nyb200_relax.cuh"

namespace nyb {

// ---------------------------------------------------------------- device helpers
__device__ __forceinline__ float next_up_f(float x) {  // crates/ny-tensor/src/rounding.rs:17-33
    unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return __uint_as_float(1u);
    return (b & 0x80000000u) ? __uint_as_float(b - 1) : __uint_as_float(b + 1);
}
__device__ __forceinline__ float next_down_f(float x) {  // crates/ny-tensor/src/rounding.rs:47-63
    unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return __uint_as_float(0x80000001u);
    return (b & 0x80000000u) ? __uint_as_float(b + 1) : __uint_as_float(b - 1);
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------- split scatter
__global__ void k_scatter_splits(NetView nv, const nyb200_split *__restrict__ sp, const int *__restrict__ ns,
                                 int max_splits, int D, signed char *__restrict__ code, float *__restrict__ sbeta,
                                 int *__restrict__ flags) {
    pdl_trigger();
    pdl_wait();
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * max_splits) return;
    int d = (int)(t / max_splits), s = (int)(t % max_splits);
    if (s >= ns[d]) return;
    nyb200_split c = sp[t];
    if (c.relu < 0 || c.relu >= nv.L - 1 || c.neuron < 0 || c.neuron >= nv.dims[c.relu + 1] ||
        (c.sign != 1 && c.sign != -1)) {
        atomicOr(&flags[d], kFlagInvalid);
        return;
    }
    long o = (long)d * nv.nps + nv.pre_off[c.relu] + c.neuron;
    code[o] = (signed char)c.sign;
    // A non-finite multiplier is skipped, as relu_backward.rs:156-173 does.
    sbeta[o] = isfinite(c.beta) ? c.beta * (float)c.sign : 0.0f;
}

// ---------------------------------------------------------------- interval mat-vec (Linear IBP)
// lo = W+ zl + W- zu + b, hi = W+ zu + W- zl + b (crates/ny-propagate/src/layers/linear/ibp.rs:489-515),
// q = |W| max(|zl|,|zu|).  Exact fp32 products are accumulated in binary64; the accumulation error is
// bounded by gamma_{K+1} * q (Higham) and removed outward before the directed cast to fp32.
constexpr int IB_M = 64, IB_N = 64, IB_K = 16;
__global__ void __launch_bounds__(256)
k_ibp_linear(int Deff, int n_in, int n_out, const float *__restrict__ W, const float *__restrict__ bias,
             const float *__restrict__ zl, const float *__restrict__ zu, long in_ds, float *__restrict__ raw_lo,
             float *__restrict__ raw_hi, float *__restrict__ q, long out_ds) {
    __shared__ float sL[IB_K][IB_M + 1], sU[IB_K][IB_M + 1], sW[IB_K][IB_N + 1];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int d0 = blockIdx.y * IB_M, o0 = blockIdx.x * IB_N;
    double lo[4][4], hi[4][4], qq[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) lo[i][j] = hi[i][j] = qq[i][j] = 0.0;
    for (int k0 = 0; k0 < n_in; k0 += IB_K) {
        for (int t = threadIdx.x; t < IB_M * IB_K; t += 256) {
            int r = t / IB_K, kk = t % IB_K;
            int d = d0 + r, k = k0 + kk;
            float a = 0.f, b = 0.f;
            if (d < Deff && k < n_in) { a = zl[(long)d * in_ds + k]; b = zu[(long)d * in_ds + k]; }
            sL[kk][r] = a; sU[kk][r] = b;
        }
        for (int t = threadIdx.x; t < IB_N * IB_K; t += 256) {
            int r = t / IB_K, kk = t % IB_K;
            int o = o0 + r, k = k0 + kk;
            sW[kk][r] = (o < n_out && k < n_in) ? W[(long)o * n_in + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < IB_K; ++kk) {
            double zlv[4], zuv[4], zm[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float a = sL[kk][ty * 4 + i], b = sU[kk][ty * 4 + i];
                zlv[i] = a; zuv[i] = b; zm[i] = fmaxf(fabsf(a), fabsf(b));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = sW[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    bool pos = w[j] > 0.0;
                    lo[i][j] = fma(w[j], pos ? zlv[i] : zuv[i], lo[i][j]);
                    hi[i][j] = fma(w[j], pos ? zuv[i] : zlv[i], hi[i][j]);
                    qq[i][j] = fma(fabs(w[j]), zm[i], qq[i][j]);
                }
        }
        __syncthreads();
    }
    const double gam = (double)(n_in + 2) * 1.1102230246251565e-16 * 1.000001;  // gamma_{n+2}, 2^-53
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int d = d0 + ty * 4 + i;
        if (d >= Deff) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int o = o0 + tx * 4 + j;
            if (o >= n_out) continue;
            double bv = bias ? (double)bias[o] : 0.0;
            double slack = gam * (qq[i][j] + fabs(bv));
            double l = lo[i][j] + bv - slack, h = hi[i][j] + bv + slack;
            // fma accumulations are not exact products + exact sums: charge one more ulp each way.
            float lf = __double2float_rd(l), hf = __double2float_ru(h);
            float qf = __double2float_ru(qq[i][j] * (1.0 + gam));
            if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
            raw_lo[(long)d * out_ds + o] = lf;
            raw_hi[(long)d * out_ds + o] = hf;
            q[(long)d * out_ds + o] = qf;
        }
    }
}

// Same arithmetic for a single box (the shared input box of the first layer): one warp per output
// neuron, lanes stride over the inputs, binary64 partial sums reduced with shuffles.
__global__ void __launch_bounds__(256)
k_ibp_linear_vec(int n_in, int n_out, const float *__restrict__ W, const float *__restrict__ bias,
                 const float *__restrict__ zl, const float *__restrict__ zu, float *__restrict__ raw_lo,
                 float *__restrict__ raw_hi, float *__restrict__ q) {
    pdl_trigger();
    pdl_wait();
    int o = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (o >= n_out) return;
    const float *w = W + (long)o * n_in;
    double lo = 0.0, hi = 0.0, qq = 0.0;
    for (int i = lane; i < n_in; i += 32) {
        double wv = w[i], a = zl[i], b = zu[i];
        bool pos = wv > 0.0;
        lo = fma(wv, pos ? a : b, lo);
        hi = fma(wv, pos ? b : a, hi);
        qq = fma(fabs(wv), fmax(fabs(a), fabs(b)), qq);
    }
    lo = warp_sum(lo); hi = warp_sum(hi); qq = warp_sum(qq);
    if (lane == 0) {
        const double gam = (double)(n_in + 2) * 1.1102230246251565e-16 * 1.000001;
        double bv = bias ? (double)bias[o] : 0.0;
        double slack = gam * (qq + fabs(bv));
        float lf = __double2float_rd(lo + bv - slack), hf = __double2float_ru(hi + bv + slack);
        if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
        raw_lo[o] = lf; raw_hi[o] = hf;
        q[o] = __double2float_ru(qq * (1.0 + gam));
    }
}

// The same for a few domains (the binary64 re-evaluation of a flagged subset): the tiled kernel above would start
// a handful of CTAs that walk the whole contraction one after the other; here one warp owns one (domain, output)
// pair and the lanes stride over the inputs.
__global__ void __launch_bounds__(256)
k_ibp_linear_warp(int Deff, int n_in, int n_out, const float *__restrict__ W, const float *__restrict__ bias,
                  const float *__restrict__ zl, const float *__restrict__ zu, long in_ds, float *__restrict__ raw_lo,
                  float *__restrict__ raw_hi, float *__restrict__ q, long out_ds) {
    long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= (long)Deff * n_out) return;
    int d = (int)(warp / n_out), o = (int)(warp - (long)d * n_out);
    const float *w = W + (long)o * n_in, *a_row = zl + (long)d * in_ds, *b_row = zu + (long)d * in_ds;
    double lo = 0.0, hi = 0.0, qq = 0.0;
    for (int i = lane; i < n_in; i += 32) {
        double wv = w[i], a = a_row[i], b = b_row[i];
        bool pos = wv > 0.0;
        lo = fma(wv, pos ? a : b, lo);
        hi = fma(wv, pos ? b : a, hi);
        qq = fma(fabs(wv), fmax(fabs(a), fabs(b)), qq);
    }
    lo = warp_sum(lo); hi = warp_sum(hi); qq = warp_sum(qq);
    if (lane == 0) {
        const double gam = (double)(n_in + 2) * 1.1102230246251565e-16 * 1.000001;
        double bv = bias ? (double)bias[o] : 0.0;
        double slack = gam * (qq + fabs(bv));
        float lf = __double2float_rd(lo + bv - slack), hf = __double2float_ru(hi + bv + slack);
        if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
        raw_lo[(long)d * out_ds + o] = lf; raw_hi[(long)d * out_ds + o] = hf;
        q[(long)d * out_ds + o] = __double2float_ru(qq * (1.0 + gam));
    }
}

// ---------------------------------------------------------------- per-domain finish of a Linear output
// mode 0: bounds = inherited (clamp only: beta_crown/engine/domain/child.rs:51-118);
// mode 1: bounds = re-propagated intersected with inherited (graph/propagation/constraints/mod.rs:738-741);
// mode 2: bounds = re-propagated (plain IBP).
// Then the split clamps (constraints/lookups.rs:160-175), the beta-CROWN relaxation
// (beta_crown/engine/backward/relu_backward.rs:63-101) and the post-activation interval (:428-548).
__global__ void k_ibp_finish(NetView nv, int k, int D, int mode, int last, const float *__restrict__ raw_lo,
                             const float *__restrict__ raw_hi, long raw_ds, const float *__restrict__ inh_lo,
                             const float *__restrict__ inh_hi, long inh_ds, const signed char *__restrict__ code,
                             const float *__restrict__ sbeta, const float *__restrict__ alpha,
                             float *__restrict__ pre_lo, float *__restrict__ pre_hi, float *__restrict__ zl,
                             float *__restrict__ zu, float4 *__restrict__ tab, float *__restrict__ zabs,
                             int *__restrict__ flags, const float *__restrict__ F, int ldf, double eps,
                             float *__restrict__ q, float fwd_tol, float *__restrict__ cj, float cj_eps, float cj_kappa) {
    pdl_trigger();
    pdl_wait();
    int n = nv.dims[k + 1], off = nv.pre_off[k];
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * n) return;
    int d = (int)(t / n), j = (int)(t % n);
    long o = (long)d * nv.nps + off + j;
    float l, u;
    if (F) {
        // Tensor-core forward: F rows [0, D) hold zl (W+|W-), rows [D, 2D) hold zu (W+|W-), valid for
        // 0 <= zl <= zu.  lo = W+ zl + W- zu + b, hi = W+ zu + W- zl + b, q = |W| zu.  Every product carries
        // a rounding of at most eps times the sum of its own term magnitudes, each bounded by q, so both
        // ends move outward by eps * q (q inflated by its own relative error) before the directed cast.
        double pl = F[(long)d * ldf + j], nl = F[(long)d * ldf + n + j];
        double pu = F[(long)(D + d) * ldf + j], nu = F[(long)(D + d) * ldf + n + j];
        double b = nv.b[k] ? (double)nv.b[k][j] : 0.0;
        double qq = (fabs(pu) + fabs(nu)) / (1.0 - 2.0 * eps);
        double slack = eps * qq + 2.3e-16 * (qq + fabs(b));
        l = __double2float_rd(pl + nu + b - slack);
        u = __double2float_ru(pu + nl + b + slack);
        if (isnan(l) || isnan(u)) { l = -INFINITY; u = INFINITY; }
        q[o] = __double2float_ru(qq);
        // The slack widens the interval; where that is visible against the width of an unstable neuron the
        // relaxation built from it (and everything downstream) is visibly looser than the binary64 pass's:
        // such a domain is flagged and the batch re-evaluated with binary64 contractions.
        if (!last && l < 0.f && u > 0.f) {
            if (fwd_tol > 0.f && (float)(2.0 * slack) > fwd_tol * (u - l)) atomicOr(&flags[d], kFlagLooseFwd);
        }
    } else {
        l = raw_lo[(long)d * raw_ds + off + j];
        u = raw_hi[(long)d * raw_ds + off + j];
    }
    const long io = (long)d * inh_ds + off + j;   // inh_ds = 0: the domains share one inherited vector
    if (mode == 0 && inh_lo) { l = inh_lo[io]; u = inh_hi[io]; }
    else if (mode == 1 && inh_lo) {
        float il = inh_lo[io], iu = inh_hi[io];
        if (!(isnan(l) || isnan(u) || isnan(il) || isnan(iu))) {
            float tl = fmaxf(l, il), tu = fminf(u, iu);
            if (tl <= tu) { l = tl; u = tu; } else { l = fminf(l, il); u = fmaxf(u, iu); }
        }
    }
    // charge weight of the fused backward chain for this table entry (the arithmetic of k_chain_prep): the rounding
    // of the contraction that consumes the coefficient, the bias product's and, below, the relaxation's own terms
    float cw = 0.f;
    if (cj) {
        cw = __fmul_ru(cj_eps, q[(long)d * raw_ds + off + j]);
        if (nv.b[k]) cw = __fmaf_ru(cj_kappa, fabsf(nv.b[k][j]), cw);
    }
    if (last) { pre_lo[o] = l; pre_hi[o] = u; if (cj) cj[o] = cw; return; }
    int s = code[o];
    if (s > 0) l = (isnan(l)) ? l : fmaxf(l, 0.f);
    else if (s < 0) u = (isnan(u)) ? u : fminf(u, 0.f);
    if (s != 0 && l > u) atomicOr(&flags[d], kFlagInfeasible);
    pre_lo[o] = l; pre_hi[o] = u;
    float ls, us, ui;
    if (s > 0) { ls = 1.f; us = 1.f; ui = 0.f; }
    else if (s < 0) { ls = 0.f; us = 0.f; ui = 0.f; }
    else if (isnan(l) || isnan(u) || isinf(l) || isinf(u)) {
        // The reference has closed forms for these arms (relu_backward.rs:75-93); a domain that reaches
        // them is returned as [-inf, +inf] here, which every one of those arms also implies or encloses.
        atomicOr(&flags[d], kFlagDegraded);
        ls = 0.f; us = 0.f; ui = 0.f;
    } else if (l >= 0.f) { ls = 1.f; us = 1.f; ui = 0.f; }
    else if (u <= 0.f) { ls = 0.f; us = 0.f; ui = 0.f; }
    else {
        float w = fmaxf(u - l, 1e-8f);  // RELU_RELAX_MIN_WIDTH, relu/mod.rs:24
        us = __fdiv_rn(u, w);
        // The reference uses ui = -l*u/w in round-to-nearest.  The chord is only a valid upper line if
        // us*l + ui >= 0 and us*u + ui >= u, so the intercept is taken as the smallest fp32 that
        // provably satisfies both; it differs from the reference value by at most a few ulps.
        float i1 = __fmul_ru(us, -l);
        float i2 = __fsub_ru(u, __fmul_rd(us, u));
        ui = fmaxf(fmaxf(i1, i2), 0.f);
        if (alpha) { float a = alpha[o]; ls = isnan(a) ? 0.f : fminf(fmaxf(a, 0.f), 1.f); }
        else ls = (u > -l) ? 1.f : 0.f;  // beta_crown/state/alpha/domain.rs:161
    }
    tab[o] = make_float4(ls, us, ui, sbeta[o]);
    const float za = fmaxf(fabsf(l), fabsf(u));
    zabs[o] = za;
    if (cj) cj[o] = __fmaf_ru(1.9073487e-7f /* 1.6 * 2^-23 */ + cj_kappa * 1.001f, za, cw);
    float pl = fmaxf(l, 0.f), pu = fmaxf(u, 0.f);
    if (s > 0) { pu = u; }
    else if (s < 0) { pl = 0.f; pu = 0.f; }
    if (isnan(l)) pl = l;
    if (isnan(u)) pu = u;
    zl[o] = pl; zu[o] = pu;
}

// ---------------------------------------------------------------- seed
__global__ void k_seed(const float *__restrict__ spec, int S, int nL, int D, int lda, float *__restrict__ A) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    long total = (long)D * 2 * S * nL;
    if (t >= total) return;
    int j = (int)(t % nL);
    long m = t / nL;
    int rr = (int)(m % (2 * S));
    A[m * lda + j] = spec[(long)(rr % S) * nL + j];
}

__global__ void k_seed_identity(int n, int D, int lda, float *__restrict__ A) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    long total = (long)D * 2 * n * n;
    if (t >= total) return;
    int j = (int)(t % n);
    long m = t / n;
    A[m * lda + j] = ((int)(m % n) == j) ? 1.f : 0.f;
}

// ---------------------------------------------------------------- ReLU relaxation pass
// One warp per row of A.  With r >= 0 the row is composed with ReLU r's relaxation
// (relu_backward.rs:105-175): lower rows take a*ls (a>0) or a*us and a*ui into the bias (a<0), stepped
// one ulp down; upper rows mirror it, stepped up; then the signed beta is subtracted / added.
// With r < 0 the coefficients are left as they are (seed pass).  In both cases the row then pays for
// the contraction that follows: bias += a'.bias_k, rpen += eps * |a'| . q_k.
__global__ void __launch_bounds__(256)
k_relax(int n, int off, int M, int R, int S, int n_pre, int identity, float *A, int lda, const float *Asrc, int lds,
        const float4 *__restrict__ tab, const float *__restrict__ zabs, const float *__restrict__ q, long q_ds,
        const float *__restrict__ bias_k, const float *__restrict__ aup, double eps, double *__restrict__ rb,
        double *__restrict__ rabs, double *__restrict__ rpen) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    int m = warp, d = m / R;
    bool upper = (m % R) >= S;
    float *row = A + (long)m * lda;
    const float *src = Asrc + (long)m * lds;
    double sb = 0.0, sa = 0.0, sp = 0.0;
    for (int j = lane; j < n; j += 32) {
        float a = src[j];
        float nw = a;
        if (!identity) {
            float4 t = tab[(long)d * n_pre + off + j];
            float za = zabs[(long)d * n_pre + off + j];
            float slope = 0.f, icp = 0.f;
            if (a > 0.f) { slope = upper ? t.y : t.x; icp = upper ? t.z : 0.f; }
            else if (a < 0.f) { slope = upper ? (aup ? aup[(long)d * n_pre + off + j] : t.x) : t.y; icp = upper ? 0.f : t.z; }
            if (a == 0.f || slope == 0.f) nw = 0.f;  // exact product: no outward step needed
            else {
                float p = a * slope;
                nw = upper ? next_up_f(p) : next_down_f(p);
                double gap = fabs((double)a * (double)slope - (double)nw);
                if (!(t.y == 1.f && t.z == 0.f)) sp += gap * (double)za;  // see relax_one: no charge where z >= 0
            }
            if (icp != 0.f) { double c = (double)a * (double)icp; sb += c; sa += fabs(c); }
            if (t.w != 0.f) nw = upper ? nw + t.w : nw - t.w;
            row[j] = nw;
        }
        if (bias_k) { double c = (double)nw * (double)bias_k[j]; sb += c; sa += fabs(c); }
        sp += eps * fabs((double)nw) * (double)q[(long)d * q_ds + off + j];
    }
    sb = warp_sum(sb); sa = warp_sum(sa); sp = warp_sum(sp);
    if (lane == 0) { rb[m] += sb; rabs[m] += sa; rpen[m] += sp; }
}

// Vectorised form of k_relax for 16-byte aligned layouts (n, off, lda, row strides multiples of 4): one
// warp per row, every lane handles float4 groups and issues all loads of a group before using them.
// The kernel is instruction-issue bound, so the per-coefficient work is kept short: the product a*slope is
// rounded as the reference does (to nearest, then one ulp outward), its exact residual is charged as
// the rounding gap, penalties are accumulated in fp32 with upward-directed operations (an upper bound is
// all that is needed) and inflated once at the end; the bias stays in binary64.
template <bool UPPER, bool RELAX, bool BIAS>
__device__ __forceinline__ float relax_one(float a, float4 t, float au, float za, float qv, float bk, float eps, double &sb,
                                           float &sa, float &sp) {
    return relax_coeff<RELAX, BIAS>(UPPER, a, t, au, za, qv, bk, eps, sb, sa, sp);
}

template <bool UPPER, bool RELAX, bool BIAS>
__device__ __forceinline__ void relax_row(int n, int lane, float *row, const float *src, const float4 *__restrict__ tab,
                                          const float *__restrict__ zabs, const float *__restrict__ q,
                                          const float *__restrict__ bias_k, const float *__restrict__ aup, float eps,
                                          double &sb, float &sa, float &sp) {
    for (int j = lane * 4; j < n; j += 128) {
        float4 a = *(const float4 *)(src + j);
        float4 qv = *(const float4 *)(q + j);
        float4 bk = BIAS ? *(const float4 *)(bias_k + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 t0 = make_float4(0.f, 0.f, 0.f, 0.f), t1 = t0, t2 = t0, t3 = t0, za = t0;
        if (RELAX) {
            t0 = tab[j]; t1 = tab[j + 1]; t2 = tab[j + 2]; t3 = tab[j + 3];
            za = *(const float4 *)(zabs + j);
        }
        float4 au = make_float4(t0.x, t1.x, t2.x, t3.x);
        if (RELAX && UPPER && aup) au = *(const float4 *)(aup + j);
        float4 o;
        o.x = relax_one<UPPER, RELAX, BIAS>(a.x, t0, au.x, za.x, qv.x, bk.x, eps, sb, sa, sp);
        o.y = relax_one<UPPER, RELAX, BIAS>(a.y, t1, au.y, za.y, qv.y, bk.y, eps, sb, sa, sp);
        o.z = relax_one<UPPER, RELAX, BIAS>(a.z, t2, au.z, za.z, qv.z, bk.z, eps, sb, sa, sp);
        o.w = relax_one<UPPER, RELAX, BIAS>(a.w, t3, au.w, za.w, qv.w, bk.w, eps, sb, sa, sp);
        if (RELAX) *(float4 *)(row + j) = o;
    }
}

template <bool RELAX, bool BIAS>
__global__ void __launch_bounds__(256, 4)
k_relax_v4(int n, int off, int M, int R, int S, long nps, float *A, int lda, const float *Asrc, int lds,
           const float4 *__restrict__ tab,
           const float *__restrict__ zabs, const float *__restrict__ q, long q_ds, const float *__restrict__ bias_k,
           const float *__restrict__ aup, float eps, double *__restrict__ rb, double *__restrict__ rabs,
           double *__restrict__ rpen) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    int m = warp, d = m / R;
    const bool upper = (m % R) >= S;  // uniform in the warp
    float *row = A + (long)m * lda;
    const float *src = Asrc + (long)m * lds;  // the row itself when the pass runs in place
    const long tb = (long)d * nps + off, qb = (long)d * q_ds + off;
    double sb = 0.0;
    float sa = 0.f, sp = 0.f;
    if (upper) relax_row<true, RELAX, BIAS>(n, lane, row, src, tab + tb, zabs + tb, q + qb, bias_k, aup ? aup + tb : nullptr, eps, sb, sa, sp);
    else relax_row<false, RELAX, BIAS>(n, lane, row, src, tab + tb, zabs + tb, q + qb, bias_k, nullptr, eps, sb, sa, sp);
    double da = (double)sa, dp = (double)sp;
    sb = warp_sum(sb); da = warp_sum(da); dp = warp_sum(dp);
    if (lane == 0) {  // reductions without a dependent read: the row is owned by this warp for this launch
        atomicAdd(&rb[m], sb);
        atomicAdd(&rabs[m], da * 1.000001);
        atomicAdd(&rpen[m], dp * 1.000001);  // covers the single rounding of each fp32 gap / product above
    }
}

// Domain-major form of the same pass.  The relaxation table, the magnitudes and the bias of a column are shared
// by all R rows of a domain; with one warp per row they are fetched R times (36 bytes per coefficient through
// L1 against 8 for the coefficient itself).  Here a warp owns 128 columns of one domain: every lane keeps the
// tables of its 4 columns in registers and walks the domain's rows, so the tables are read once.
template <bool UPPER, bool RELAX, bool BIAS>
__device__ __forceinline__ void relax_dom_rows(int r0, int r1, long m0, int j, float *A, int lda, const float *Asrc, int lds,
                                               const float4 &t0, const float4 &t1, const float4 &t2, const float4 &t3,
                                               const float4 &za, const float4 &qv, const float4 &bk, const float4 &au,
                                               float eps, int lane, bool live, double *__restrict__ rb, double *__restrict__ rabs,
                                               double *__restrict__ rpen) {
    // Rows are taken RB at a time: all their loads are issued before the first is used, so a lane has RB
    // independent 16-byte requests in flight (a warp that walks one row after the other is latency bound).
    constexpr int RB = 5;
    for (int rbase = r0; rbase < r1; rbase += RB) {
        float4 a[RB];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const long m = m0 + rbase + u;
            // lanes past the row's end take part in the reductions with zeros (their tables are zero too)
            a[u] = (live && rbase + u < r1) ? *(const float4 *)(Asrc + m * lds + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            if (rbase + u >= r1) break;  // uniform in the warp
            const long m = m0 + rbase + u;
            double sb = 0.0;
            float sa = 0.f, sp = 0.f;
            float4 o;
            o.x = relax_one<UPPER, RELAX, BIAS>(a[u].x, t0, au.x, za.x, qv.x, bk.x, eps, sb, sa, sp);
            o.y = relax_one<UPPER, RELAX, BIAS>(a[u].y, t1, au.y, za.y, qv.y, bk.y, eps, sb, sa, sp);
            o.z = relax_one<UPPER, RELAX, BIAS>(a[u].z, t2, au.z, za.z, qv.z, bk.z, eps, sb, sa, sp);
            o.w = relax_one<UPPER, RELAX, BIAS>(a[u].w, t3, au.w, za.w, qv.w, bk.w, eps, sb, sa, sp);
            if (RELAX && live) __stcs((float4 *)(A + m * lda + j), o);  // streamed: the next reader is another kernel
            // The magnitude sum only ever enters the bound as 2^-40 * rabs (the slack for the binary64 bias
            // sums), so it is folded into the penalty here instead of being reduced on its own; the penalty
            // is reduced in fp32 (five shuffles) and inflated for the roundings of that reduction.
            sp = __fmaf_ru(sa, 9.1e-13f, sp);
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) sp = __fadd_ru(sp, __shfl_xor_sync(0xffffffffu, sp, o2));
            sb = warp_sum(sb);
            if (lane == 0) {
                atomicAdd(&rb[m], sb);
                atomicAdd(&rpen[m], (double)sp * 1.000002);
            }
        }
    }
}

template <bool RELAX, bool BIAS>
__global__ void __launch_bounds__(256)
k_relax_dom(int n, int off, int D, int R, int S, long nps, float *A, int lda, const float *Asrc, int lds,
            const float4 *__restrict__ tab, const float *__restrict__ zabs, const float *__restrict__ q, long q_ds,
            const float *__restrict__ bias_k, const float *__restrict__ aup, float eps, double *__restrict__ rb,
            double *__restrict__ rabs, double *__restrict__ rpen) {
    const int slabs = (n + 127) >> 7;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long)D * slabs) return;
    const int d = (int)(warp / slabs), slab = (int)(warp - (long)d * slabs);
    const int j = slab * 128 + lane * 4;
    const bool live = j < n;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 t0 = zero, t1 = zero, t2 = zero, t3 = zero, za = zero, qv = zero, bk = zero;
    if (live) {
        const long tb = (long)d * nps + off + j;
        qv = *(const float4 *)(q + (long)d * q_ds + off + j);
        if (BIAS) bk = *(const float4 *)(bias_k + j);
        if (RELAX) {
            t0 = tab[tb]; t1 = tab[tb + 1]; t2 = tab[tb + 2]; t3 = tab[tb + 3];
            za = *(const float4 *)(zabs + tb);
        }
    }
    float4 au = make_float4(t0.x, t1.x, t2.x, t3.x);
    if (RELAX && live && aup) au = *(const float4 *)(aup + (long)d * nps + off + j);
    const long m0 = (long)d * R;
    relax_dom_rows<false, RELAX, BIAS>(0, S, m0, j, A, lda, Asrc, lds, t0, t1, t2, t3, za, qv, bk, au, eps, lane, live, rb, rabs, rpen);
    relax_dom_rows<true, RELAX, BIAS>(S, R, m0, j, A, lda, Asrc, lds, t0, t1, t2, t3, za, qv, bk, au, eps, lane, live, rb, rabs, rpen);
}

// ---------------------------------------------------------------- binary64-accumulated contraction
// C[M x N] = A[M x K] * B[K x N]; the fp32 products are exact in binary64, the running sums round to
// nearest (bounded by eps*|A||B|, charged in k_relax), and the final cast to fp32 is measured exactly,
// sign included, and charged against the interval of the variable the coefficient multiplies.
constexpr int GM = 64, GN = 64, GK = 16;
__global__ void __launch_bounds__(256)
k_gemm_f64(int M, int N, int K, const float *__restrict__ A, int lda, const float *__restrict__ B, int ldb,
           float *__restrict__ C, int ldc, int R, const float *__restrict__ zin_lo, const float *__restrict__ zin_hi,
           long zin_ds, double *__restrict__ rpen) {
    __shared__ float sA[GK][GM + 1], sB[GK][GN + 1];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
    double acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
    for (int k0 = 0; k0 < K; k0 += GK) {
        for (int t = threadIdx.x; t < GM * GK; t += 256) {
            int r = t / GK, kk = t % GK;
            int m = m0 + r, k = k0 + kk;
            sA[kk][r] = (m < M && k < K) ? A[(long)m * lda + k] : 0.f;
        }
        for (int t = threadIdx.x; t < GK * GN; t += 256) {
            int kk = t / GN, c = t % GN;
            int k = k0 + kk, n = n0 + c;
            sB[kk][c] = (k < K && n < N) ? B[(long)k * ldb + n] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            double a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sB[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        double pen = 0.0;
        if (m < M) {
            int d = m / R;
            const bool upper_row = (m % R) >= (R >> 1);  // a domain's rows: the lower half, then the upper half
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int n = n0 + tx * 4 + j;
                if (n >= N) continue;
                float c = (float)acc[i][j];
                C[(long)m * ldc + n] = c;
                if (rpen) {
                    // The exact coefficient is c + e with e known, and it multiplies z in [zl, zu]: a lower row loses at
                    // most -min(e zl, e zu), an upper row gains at most max(e zl, e zu).  Signed, so the roundings of a
                    // row cancel against one another the way they do in the exact sum (|e| max|z| would add them up).
                    const double e = acc[i][j] - (double)c;
                    const double zl = zin_lo[(long)d * zin_ds + n], zu = zin_hi[(long)d * zin_ds + n];
                    const double a = e * zl, b = e * zu;
                    pen += (upper_row ? fmax(a, b) : fmax(-a, -b)) + 2.9e-14 * fabs(e) * fmax(fabs(zl), fabs(zu));
                }
            }
        }
        if (rpen) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) pen += __shfl_xor_sync(0xffffffffu, pen, o);
            if (tx == 0 && m < M && pen != 0.0) atomicAdd(&rpen[m], pen);
        }
    }
}

// ---------------------------------------------------------------- concretisation
// lb_s = b_s + sum_j A_sj * (A_sj >= 0 ? x_l : x_u) - penalty (bounds/concretize.rs:374-489), one warp
// per row, exact products accumulated in binary64, directed cast.
__global__ void __launch_bounds__(256)
k_concretize(int M, int R, int S, int n0, const float *__restrict__ A, int lda, const float *__restrict__ in_lo,
             const float *__restrict__ in_hi, long box_ds, const double *__restrict__ rb,
             const double *__restrict__ rabs, const double *__restrict__ rpen, float *__restrict__ out_lo,
             float *__restrict__ out_hi) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    int m = warp, d = m / R, rr = m % R;
    bool upper = rr >= S;
    const float *row = A + (long)m * lda;
    const float *xl = in_lo + (long)d * box_ds, *xu = in_hi + (long)d * box_ds;
    double s = 0.0, sa = 0.0;
    bool bad = false;
    auto term = [&](float a, float l, float u) {
        bool nonneg = !(__float_as_uint(a) >> 31) || (__float_as_uint(a) & 0x7fffffffu) == 0;
        float x = (nonneg != upper) ? l : u;
        if (!(fabsf(a) < 1e10f)) bad = true;  // is_crown_coeff_safe, crates/ny-core/src/gemm.rs:127
        if (a != 0.f && x != 0.f) { double c = (double)a * (double)x; s += c; sa += fabs(c); }
    };
    const bool vec = (n0 % 4 == 0) && (lda % 4 == 0) && (box_ds % 4 == 0) &&
                     (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(in_lo) |
                        reinterpret_cast<uintptr_t>(in_hi)) & 15) == 0);
    if (vec) {
#pragma unroll 4
        for (int j = lane * 4; j < n0; j += 128) {
            float4 a = *(const float4 *)(row + j), l = *(const float4 *)(xl + j), u = *(const float4 *)(xu + j);
            term(a.x, l.x, u.x); term(a.y, l.y, u.y); term(a.z, l.z, u.z); term(a.w, l.w, u.w);
        }
    } else {
        for (int j = lane; j < n0; j += 32) term(row[j], xl[j], xu[j]);
    }
    s = warp_sum(s); sa = warp_sum(sa);
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) {
        double tot_abs = sa + rabs[m] + fabs(rb[m]);
        double slack = tot_abs * 9.094947017729282e-13;  // 2^-40 >> (number of binary64 additions) * 2^-53
        float v;
        if (!upper) {
            double x = rb[m] + s - rpen[m] - slack;
            v = (bad || isnan(x)) ? -INFINITY : __double2float_rd(x);
            out_lo[(long)d * S + rr] = v;
        } else {
            double x = rb[m] + s + rpen[m] + slack;
            v = (bad || isnan(x)) ? INFINITY : __double2float_ru(x);
            out_hi[(long)d * S + (rr - S)] = v;
        }
    }
}

__device__ __forceinline__ void atomic_min_float(float *addr, float v) {
    if (v >= 0.f) atomicMin((int *)addr, __float_as_int(v));
    else atomicMax((unsigned *)addr, __float_as_uint(v));
}

// Counts the domains whose accumulated rounding penalty is not small against their bounds: a row is
// "loose" when rpen > tol * max(|bound|, 1% of the domain's largest bound magnitude), or when the row's width is
// smaller than the charges on its two ends.  The host re-runs
// the batch on the binary64 path when the count is non-zero, so that the fast path never returns a
// bound that its own rounding model has visibly loosened.
// thr != null (a search that only needs verdicts, nyb200_frontier_set_refinement): a domain is flagged only when the
// charge could change a verdict, i.e. some row's lower bound misses its threshold by less than twice the row's charge
// (the exact bound lies within that distance above the certified one).
__global__ void k_count_loose(int D, int S, int R, const float *__restrict__ out_lo, const float *__restrict__ out_hi,
                              const double *__restrict__ rpen, int *__restrict__ flags, float tol,
                              int *__restrict__ n_loose, const float *__restrict__ thr) {
    pdl_trigger();
    pdl_wait();
    int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const int f = flags[d];
    if (f & ~(kFlagLooseFwd | kFlagLoose)) return;  // infeasible / degraded / invalid domains are not re-evaluated
    if (thr) {
        bool close = false;
        for (int s = 0; s < S; ++s) {
            const float l = out_lo[d * S + s];
            if (!isfinite(l)) continue;
            const double reach = (double)l + 2.000001 * rpen[(long)d * R + s];
            if (l <= thr[s] && reach > (double)thr[s]) close = true;
        }
        if (close) { atomicAdd(n_loose, 1); flags[d] = f | kFlagLoose; }
        return;
    }
    if (f & kFlagLooseFwd) { atomicAdd(n_loose, 1); return; }
    float scale = 0.f;
    for (int s = 0; s < S; ++s) {
        float l = out_lo[d * S + s], u = out_hi[d * S + s];
        if (isfinite(l)) scale = fmaxf(scale, fabsf(l));
        if (isfinite(u)) scale = fmaxf(scale, fabsf(u));
    }
    bool loose = false;
    for (int s = 0; s < S; ++s) {
        float l = out_lo[d * S + s], u = out_hi[d * S + s];
        if (!isfinite(l) || !isfinite(u)) continue;
        double pl = rpen[(long)d * R + s], pu = rpen[(long)d * R + S + s];
        if (pl > (double)tol * fmaxf(fabsf(l), 0.01f * scale) || pu > (double)tol * fmaxf(fabsf(u), 0.01f * scale)) loose = true;
        // the charge alone keeps the row from inverting (lower > upper marks an empty domain and is published as
        // [-inf, +inf], bounds/concretize.rs:717-880): let the binary64 pass decide
        if ((double)u - (double)l < pl + pu) loose = true;
    }
    if (loose) { atomicAdd(n_loose, 1); flags[d] = f | kFlagLoose; }
}

// ---------------------------------------------------------------- verdicts
// Per domain, lower mode (every spec row must stay above the threshold): verified when every row passes
// domain_is_verified_for_mode (all of lower, upper, threshold finite, lower <= upper, lower > threshold: strict);
// violated when some row passes domain_is_violation_for_mode (finite, not inverted, upper < threshold)
// (beta_crown/config/beta_config.rs:1552-1610).  Infeasible domains are reported as such.
__global__ void k_verdicts(int D, int S, const float *__restrict__ out_lo, const float *__restrict__ out_hi,
                           const int *__restrict__ flags, float threshold, int *__restrict__ status) {
    int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    if (flags[d] & kFlagInfeasible) { status[d] = NYB200_VERDICT_INFEASIBLE; return; }
    bool all_verified = isfinite(threshold), any_violated = false;
    for (int s = 0; s < S; ++s) {
        float l = out_lo[d * S + s], u = out_hi[d * S + s];
        bool sane = isfinite(l) && isfinite(u) && isfinite(threshold);
        if (!(sane && l <= u && l > threshold)) all_verified = false;
        if (sane && l <= u && u < threshold) any_violated = true;
    }
    status[d] = all_verified ? NYB200_VERDICT_VERIFIED : (any_violated ? NYB200_VERDICT_VIOLATED : NYB200_VERDICT_UNKNOWN);
}

// ---------------------------------------------------------------- row gather / scatter (subset re-evaluation)
__global__ void k_move_rows(unsigned *__restrict__ dst, const unsigned *__restrict__ src, const int *__restrict__ idx,
                            int n_rows, long row_words, int scatter) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)n_rows * row_words) return;
    long i = t / row_words, w = t - i * row_words;
    long other = idx[i];
    if (scatter) dst[other * row_words + w] = src[i * row_words + w];
    else dst[i * row_words + w] = src[other * row_words + w];
}

__global__ void k_min_lower(int D, int S, const float *__restrict__ out_lo, const int *__restrict__ flags,
                            float *__restrict__ min_lower) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= D * S) return;
    if (!(flags[t / S] & kFlagInfeasible)) atomic_min_float(min_lower, out_lo[t]);
}

// Per (domain, spec row): apply the domain flags and the reference's repair rule
// (non-finite endpoint or inversion -> [-inf, +inf], concretize.rs:481-488); fold the global minimum.
__global__ void k_finalize(int D, int S, const int *__restrict__ flags, float *__restrict__ out_lo,
                           float *__restrict__ out_hi, float *__restrict__ min_lower) {
    pdl_trigger();
    pdl_wait();
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= D * S) return;
    int d = t / S;
    int f = flags[d];
    float l = out_lo[t], u = out_hi[t];
    if (f & kFlagInfeasible) { l = INFINITY; u = -INFINITY; }
    else if ((f & (kFlagDegraded | kFlagInvalid)) || !isfinite(l) || !isfinite(u) || l > u) { l = -INFINITY; u = INFINITY; }
    out_lo[t] = l; out_hi[t] = u;
    if (!(f & kFlagInfeasible)) atomic_min_float(min_lower, l);
}

// ---------------------------------------------------------------- branching
// select_largest_width_neuron (beta_crown/engine/branching/sequential.rs:49-104): widest unstable,
// unsplit neuron; strict '>' so the first maximum in (relu, neuron) order wins; NaN widths skipped.
__global__ void __launch_bounds__(256)
k_select_branch(NetView nv, int D, const float *__restrict__ pre_lo, const float *__restrict__ pre_hi,
                const signed char *__restrict__ code, int *__restrict__ relu, int *__restrict__ neuron,
                float *__restrict__ width, int kind) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= D) return;
    int d = warp;
    int n_hidden = nv.pre_off[nv.L - 1];
    float best = -1.f;  // every candidate's score is > 0 (width, or -l*u/(u-l) with l < 0 < u)
    int bidx = 0x7fffffff;
    for (int i = lane; i < n_hidden; i += 32) {
        long o = (long)d * nv.nps + i;
        float l = pre_lo[o], u = pre_hi[o];
        if (l >= 0.f || u <= 0.f || code[o] != 0) continue;
        float w = u - l;
        if (isnan(w)) continue;
        if (kind == 1) {  // intercept score of the batched graph engine (batched_domain/domain_list/picked.rs:153-233)
            if (!(w > 0.f)) continue;
            w = __fdiv_rn(-l * u, w);
            if (isnan(w)) continue;
        }
        if (w > best) { best = w; bidx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; }
    }
    if (lane == 0) {
        if (bidx == 0x7fffffff) { relu[d] = -1; neuron[d] = -1; width[d] = 0.f; }
        else {
            int r = 0;
            while (r + 1 < nv.L - 1 && bidx >= nv.pre_off[r + 1]) ++r;
            relu[d] = r; neuron[d] = bidx - nv.pre_off[r]; width[d] = best;
        }
    }
}

__global__ void k_fill_f64(double *p, size_t n, double v) {
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) p[t] = v;
}

// ---------------------------------------------------------------- residual connections
__global__ void k_skip_interval(int D, int n, long stride, float *__restrict__ raw_lo, float *__restrict__ raw_hi, int off,
                                const float *__restrict__ zl, const float *__restrict__ zu, int src_off) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * n) return;
    int d = (int)(t / n), j = (int)(t % n);
    long o = (long)d * stride + off + j, s = (long)d * stride + src_off + j;
    raw_lo[o] = __fadd_rd(raw_lo[o], zl[s]);
    raw_hi[o] = __fadd_ru(raw_hi[o], zu[s]);
}

// A += S (the identity branch of a residual block meets the coefficients that came through the block:
// A_in = backward_F(A) + A, crates/ny-core/src/gemm.rs:1640-1669).  One warp per row; the error of each
// rounded sum is recovered exactly (two-sum) and charged against max|z| of the variable it multiplies.
__global__ void __launch_bounds__(256)
k_skip_coeff(int M, int n, float *__restrict__ A, int lda, const float *__restrict__ S, int lds, int R,
             const float *__restrict__ zl, const float *__restrict__ zu, long stride, int src_off,
             double *__restrict__ rpen) {
    int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (m >= M) return;
    int d = m / R;
    double pen = 0.0;
    for (int j = lane; j < n; j += 32) {
        float a = A[(long)m * lda + j], b = S[(long)m * lds + j];
        float s = a + b;
        float bb = s - a;
        float err = (a - (s - bb)) + (b - bb);  // exact residual of the rounded sum
        A[(long)m * lda + j] = s;
        if (rpen) {
            long o = (long)d * stride + src_off + j;
            pen += fabs((double)err) * (double)fmaxf(fabsf(zl[o]), fabsf(zu[o]));
        }
    }
    if (rpen) {
        pen = warp_sum(pen);
        if (lane == 0 && pen != 0.0) atomicAdd(&rpen[m], pen);
    }
}

// The same with one block per row and four columns per thread and step (rows of tens of thousands of columns, as the
// convolutional layers of a residual network have, keep a single warp busy for thousands of dependent steps).  The
// block's shares of the charge are added in a fixed order, so the row's penalty does not depend on scheduling.
__global__ void __launch_bounds__(256)
k_skip_coeff_v4(int M, int n, float *__restrict__ A, int lda, const float *__restrict__ S, int lds, int R,
                const float *__restrict__ zl, const float *__restrict__ zu, long stride, int src_off,
                double *__restrict__ rpen) {
    __shared__ double part[8];
    const int m = blockIdx.x;
    if (m >= M) return;
    const int d = m / R;
    float4 *a4 = (float4 *)(A + (long)m * lda);
    const float4 *s4 = (const float4 *)(S + (long)m * lds);
    const float4 *l4 = (const float4 *)(zl + (long)d * stride + src_off), *u4 = (const float4 *)(zu + (long)d * stride + src_off);
    double pen = 0.0;
    auto one = [&](float a, float b, float l, float u, float &out) {
        const float s = a + b;
        const float bb = s - a;
        const float err = (a - (s - bb)) + (b - bb);  // exact residual of the rounded sum
        out = s;
        if (rpen) pen += fabs((double)err) * (double)fmaxf(fabsf(l), fabsf(u));
    };
    for (int j = threadIdx.x; j < n / 4; j += 256) {
        const float4 a = a4[j], b = s4[j];
        float4 l = make_float4(0.f, 0.f, 0.f, 0.f), u = l, o;
        if (rpen) { l = l4[j]; u = u4[j]; }
        one(a.x, b.x, l.x, u.x, o.x); one(a.y, b.y, l.y, u.y, o.y); one(a.z, b.z, l.z, u.z, o.z); one(a.w, b.w, l.w, u.w, o.w);
        a4[j] = o;
    }
    if (rpen) {
        pen = warp_sum(pen);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = pen;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < 8; ++w) t += part[w];
            if (t != 0.0) atomicAdd(&rpen[m], t);
        }
    }
}

// ---------------------------------------------------------------- launchers
#define NYB_COUNT(e) ((e)->launches++)

void launch_scatter_splits(nyb200_engine *e, const NetView &nv, const nyb200_split *sp, const int *ns, int max_splits,
                           int D, signed char *code, float *sbeta, int *flags) {
    long total = (long)D * max_splits;
    if (total == 0) return;
    k_scatter_splits<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(nv, sp, ns, max_splits, D, code, sbeta, flags);
    NYB_COUNT(e);
}

void launch_ibp_linear(nyb200_engine *e, const NetView &nv, int k, int Deff, const float *zl, const float *zu,
                       long in_dstride, float *raw_lo, float *raw_hi, float *q, long out_dstride) {
    int n_in = nv.dims[k], n_out = nv.dims[k + 1];
    if (Deff == 1) {
        launch_pdl(k_ibp_linear_vec, dim3((n_out * 32 + 255) / 256), dim3(256), 0, e, n_in, n_out, (const float *)nv.W[k],
                   (const float *)nv.b[k], zl, zu, raw_lo + nv.pre_off[k], raw_hi + nv.pre_off[k], q + nv.pre_off[k]);
        NYB_COUNT(e);
        return;
    }
    dim3 grid((n_out + IB_N - 1) / IB_N, (Deff + IB_M - 1) / IB_M);
    if ((long)grid.x * grid.y < 96) {  // too few tiles to occupy the GPU: one warp per (domain, output)
        long warps = (long)Deff * n_out;
        k_ibp_linear_warp<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, e->stream>>>(
            Deff, n_in, n_out, nv.W[k], nv.b[k], zl, zu, in_dstride, raw_lo + nv.pre_off[k], raw_hi + nv.pre_off[k],
            q + nv.pre_off[k], out_dstride);
        NYB_COUNT(e);
        return;
    }
    k_ibp_linear<<<grid, 256, 0, e->stream>>>(Deff, n_in, n_out, nv.W[k], nv.b[k], zl, zu, in_dstride,
                                               raw_lo + nv.pre_off[k], raw_hi + nv.pre_off[k], q + nv.pre_off[k],
                                               out_dstride);
    NYB_COUNT(e);
}

void launch_ibp_finish(nyb200_engine *e, const NetView &nv, int k, int D, int mode, const float *raw_lo,
                       const float *raw_hi, long raw_dstride, const float *inh_lo, const float *inh_hi, long inh_dstride,
                       const signed char *code, const float *sbeta, const float *alpha, float *pre_lo, float *pre_hi,
                       float *zl, float *zu, float4 *tab, float *zabs, int *flags, const float *F, int ldf, double eps,
                       float *q, float fwd_tol, float *cj, float cj_eps, float cj_kappa) {
    long total = (long)D * nv.dims[k + 1];
    int last = (k == nv.L - 1);
    launch_pdl(k_ibp_finish, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, e, nv, k, D, mode, last, raw_lo, raw_hi,
               raw_dstride, inh_lo, inh_hi, inh_dstride, code, sbeta, alpha, pre_lo, pre_hi, zl, zu, tab, zabs, flags, F, ldf, eps, q, fwd_tol, cj,
               cj_eps, cj_kappa);
    NYB_COUNT(e);
}

void launch_seed(nyb200_engine *e, const float *spec, int S, int nL, int D, int lda, float *A) {
    long total = (long)D * 2 * S * nL;
    k_seed<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(spec, S, nL, D, lda, A);
    NYB_COUNT(e);
}

void launch_skip_interval(nyb200_engine *e, int D, int n, long stride, float *raw_lo, float *raw_hi, int off,
                          const float *zl, const float *zu, int src_off) {
    long tot = (long)D * n;
    k_skip_interval<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>(D, n, stride, raw_lo, raw_hi, off, zl, zu, src_off);
    NYB_COUNT(e);
}

void launch_skip_coeff(nyb200_engine *e, int M, int n, float *A, int lda, const float *S, int lds, int R,
                       const float *zl, const float *zu, long stride, int src_off, double *rpen) {
    const bool vec = n >= 2048 && (n % 4 == 0) && (lda % 4 == 0) && (lds % 4 == 0) && (stride % 4 == 0) && (src_off % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(S) | reinterpret_cast<uintptr_t>(zl) |
                       reinterpret_cast<uintptr_t>(zu)) & 15) == 0;
    if (vec) {
        k_skip_coeff_v4<<<(unsigned)M, 256, 0, e->stream>>>(M, n, A, lda, S, lds, R, zl, zu, stride, src_off, rpen);
    } else {
        long threads = (long)M * 32;
        k_skip_coeff<<<(unsigned)((threads + 255) / 256), 256, 0, e->stream>>>(M, n, A, lda, S, lds, R, zl, zu, stride, src_off, rpen);
    }
    NYB_COUNT(e);
}

void launch_seed_identity(nyb200_engine *e, int n, int D, int lda, float *A) {
    long total = (long)D * 2 * n * n;
    k_seed_identity<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(n, D, lda, A);
    NYB_COUNT(e);
}

void launch_relax(nyb200_engine *e, const NetView &nv, int r, int lin_k, int M, int R, int S, float *A, int lda,
                  const float4 *tab, const float *zabs, const float *q, long q_dstride, double eps_gemm, double *rb,
                  double *rabs, double *rpen, const float *Asrc, int lds, const float *aup) {
    int n = nv.dims[lin_k + 1], off = nv.pre_off[lin_k];
    if (!Asrc) { Asrc = A; lds = lda; }
    long threads = (long)M * 32;
    unsigned grid = (unsigned)((threads + 255) / 256);
    bool aligned = (n % 4 == 0) && (off % 4 == 0) && (lda % 4 == 0) && (nv.nps % 4 == 0) && (q_dstride % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && (lds % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(Asrc) & 15) == 0);
    if (aligned) {
        const float epsf = (float)(eps_gemm * 1.0000002);
        const float *bk = nv.b[lin_k];
#define NYB_RELAX_LAUNCH(RELAX, BIAS) \
    k_relax_v4<RELAX, BIAS><<<grid, 256, 0, e->stream>>>(n, off, M, R, S, (long)nv.nps, A, lda, Asrc, lds, tab, zabs, q, q_dstride, bk, aup, epsf, rb, rabs, rpen)
        const int D = M / R;
        const long dwarps = (long)D * ((n + 127) / 128);
        const unsigned dgrid = (unsigned)((dwarps * 32 + 255) / 256);
#define NYB_RELAX_DOM(RELAX, BIAS) \
    k_relax_dom<RELAX, BIAS><<<dgrid, 256, 0, e->stream>>>(n, off, D, R, S, (long)nv.nps, A, lda, Asrc, lds, tab, zabs, q, q_dstride, bk, aup, epsf, rb, rabs, rpen)
        // domain-major when a domain's rows amortise the table loads and there are enough warps to fill the GPU
        const bool dom = R >= 4 && dwarps >= 2048;
        if (dom) {
            if (r >= 0) { if (bk) NYB_RELAX_DOM(true, true); else NYB_RELAX_DOM(true, false); }
            else { if (bk) NYB_RELAX_DOM(false, true); else NYB_RELAX_DOM(false, false); }
        } else {
            if (r >= 0) { if (bk) NYB_RELAX_LAUNCH(true, true); else NYB_RELAX_LAUNCH(true, false); }
            else { if (bk) NYB_RELAX_LAUNCH(false, true); else NYB_RELAX_LAUNCH(false, false); }
        }
#undef NYB_RELAX_DOM
#undef NYB_RELAX_LAUNCH
    } else
        k_relax<<<grid, 256, 0, e->stream>>>(n, off, M, R, S, nv.nps, r < 0 ? 1 : 0, A, lda, Asrc, lds, tab, zabs, q, q_dstride,
                                             nv.b[lin_k], aup, eps_gemm, rb, rabs, rpen);
    NYB_COUNT(e);
}

void launch_gemm_f64(nyb200_engine *e, int M, int N, int K, const float *A, int lda, const float *B, int ldb, float *C,
                     int ldc, int R, const float *zin_lo, const float *zin_hi, long zin_dstride, double *rpen) {
    dim3 grid((N + GN - 1) / GN, (M + GM - 1) / GM);
    k_gemm_f64<<<grid, 256, 0, e->stream>>>(M, N, K, A, lda, B, ldb, C, ldc, R, zin_lo, zin_hi, zin_dstride, rpen);
    NYB_COUNT(e);
}

void launch_concretize(nyb200_engine *e, int M, int R, int S, int n0, const float *A, int lda, const float *in_lo,
                       const float *in_hi, long box_dstride, const double *rb, const double *rabs, const double *rpen,
                       int *flags, float *out_lo, float *out_hi, float *min_lower, float loose_tol) {
    long threads = (long)M * 32;
    k_concretize<<<(unsigned)((threads + 255) / 256), 256, 0, e->stream>>>(M, R, S, n0, A, lda, in_lo, in_hi, box_dstride,
                                                                           rb, rabs, rpen, out_lo, out_hi);
    NYB_COUNT(e);
    int D = M / R;
    if (loose_tol > 0.f) {
        k_count_loose<<<(D + 255) / 256, 256, 0, e->stream>>>(D, S, R, out_lo, out_hi, rpen, flags, loose_tol,
                                                              (int *)min_lower + 4, e->batch.decision_thr);
        NYB_COUNT(e);
    }
    k_finalize<<<(D * S + 255) / 256, 256, 0, e->stream>>>(D, S, flags, out_lo, out_hi, min_lower);
    NYB_COUNT(e);
}

// Second half of the fused concretisation: a row's slices, left by the last contraction's epilogue, added in slot
// order (so that the result does not depend on which CTA finished first), then the same closing arithmetic as
// k_concretize.
__global__ void k_concretize_fused(int M, int R, int S, int slots, const double *__restrict__ part, const int *__restrict__ badf,
                                   const double *__restrict__ rb, const double *__restrict__ rabs,
                                   const double *__restrict__ rpen, float *__restrict__ out_lo, float *__restrict__ out_hi) {
    pdl_trigger();
    pdl_wait();
    int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const int d = m / R, rr = m % R;
    const bool upper = rr >= S;
    double s = 0.0, sa = 0.0;
    for (int i = 0; i < slots; ++i) { s += part[((long)m * slots + i) * 2]; sa += part[((long)m * slots + i) * 2 + 1]; }
    const bool bad = badf[m] != 0;
    double tot_abs = sa + rabs[m] + fabs(rb[m]);
    double slack = tot_abs * 9.094947017729282e-13;  // 2^-40 >> (number of binary64 additions) * 2^-53
    if (!upper) {
        double x = rb[m] + s - rpen[m] - slack;
        out_lo[(long)d * S + rr] = (bad || isnan(x)) ? -INFINITY : __double2float_rd(x);
    } else {
        double x = rb[m] + s + rpen[m] + slack;
        out_hi[(long)d * S + (rr - S)] = (bad || isnan(x)) ? INFINITY : __double2float_ru(x);
    }
}

void launch_concretize_fused(nyb200_engine *e, int M, int R, int S, int slots, const double *part, const int *bad,
                             const double *rb, const double *rabs, const double *rpen, int *flags, float *out_lo,
                             float *out_hi, float *min_lower, float loose_tol) {
    launch_pdl(k_concretize_fused, dim3((unsigned)((M + 255) / 256)), dim3(256), 0, e, M, R, S, slots, part, bad, rb, rabs,
               rpen, out_lo, out_hi);
    NYB_COUNT(e);
    int D = M / R;
    if (loose_tol > 0.f) {
        launch_pdl(k_count_loose, dim3((D + 255) / 256), dim3(256), 0, e, D, S, R, (const float *)out_lo, (const float *)out_hi,
                   rpen, flags, loose_tol, (int *)min_lower + 4, e->batch.decision_thr);
        NYB_COUNT(e);
    }
    launch_pdl(k_finalize, dim3((D * S + 255) / 256), dim3(256), 0, e, D, S, (const int *)flags, out_lo, out_hi, min_lower);
    NYB_COUNT(e);
}

void launch_finalize(nyb200_engine *e, int D, int S, const int *flags, float *out_lo, float *out_hi, float *min_lower) {
    k_finalize<<<(D * S + 255) / 256, 256, 0, e->stream>>>(D, S, flags, out_lo, out_hi, min_lower);
    NYB_COUNT(e);
}

void launch_verdicts(nyb200_engine *e, int D, int S, const float *out_lo, const float *out_hi, const int *flags,
                     float threshold, int *status) {
    k_verdicts<<<(unsigned)((D + 255) / 256), 256, 0, e->stream>>>(D, S, out_lo, out_hi, flags, threshold, status);
    NYB_COUNT(e);
}

void launch_gather_rows(nyb200_engine *e, void *dst, const void *src, const int *idx, int n_rows, long row_words) {
    long tot = (long)n_rows * row_words;
    if (tot == 0) return;
    k_move_rows<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>((unsigned *)dst, (const unsigned *)src, idx, n_rows, row_words, 0);
    NYB_COUNT(e);
}

void launch_scatter_rows(nyb200_engine *e, void *dst, const void *src, const int *idx, int n_rows, long row_words) {
    long tot = (long)n_rows * row_words;
    if (tot == 0) return;
    k_move_rows<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>((unsigned *)dst, (const unsigned *)src, idx, n_rows, row_words, 1);
    NYB_COUNT(e);
}

void launch_min_lower(nyb200_engine *e, int D, int S, const float *out_lo, const int *flags, float *min_lower) {
    static const float inf_word = INFINITY;
    cudaMemcpyAsync(min_lower, &inf_word, 4, cudaMemcpyHostToDevice, e->stream);
    k_min_lower<<<(unsigned)((D * S + 255) / 256), 256, 0, e->stream>>>(D, S, out_lo, flags, min_lower);
    NYB_COUNT(e);
}

void launch_select_branch(nyb200_engine *e, const NetView &nv, int D, const float *pre_lo, const float *pre_hi,
                          const signed char *code, int *relu, int *neuron, float *width, int kind) {
    long threads = (long)D * 32;
    k_select_branch<<<(unsigned)((threads + 255) / 256), 256, 0, e->stream>>>(nv, D, pre_lo, pre_hi, code, relu, neuron,
                                                                              width, kind);
    NYB_COUNT(e);
}

__global__ void k_fill_f32(float *p, size_t n, float v) {
    size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) p[t] = v;
}
void launch_fill_f32(nyb200_engine *e, float *p, size_t n, float v) {
    k_fill_f32<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(p, n, v);
    NYB_COUNT(e);
}

void launch_fill_f64(nyb200_engine *e, double *p, size_t n, double v) {
    k_fill_f64<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(p, n, v);
    NYB_COUNT(e);
}

}  // namespace nyb
