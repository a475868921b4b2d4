// Reference-compatible certified-error channel for the plain-CROWN backward pass (binary64 arithmetic).
//
// The engine's default discharges every rounding at the layer where it occurs, against the interval of the
// variable the coefficient multiplies (see nyb200_kernels.cu).  The reference instead carries a per-coefficient
// error matrix next to the coefficients,
//     err' = |a64 - fl32(a64)| + gamma_K * (|A| |W|) + err * |W|        (layers/linear/crown_single.rs:2092-2103,
//                                                                        triplet form ny-cuda/src/sound_crown.rs:348-376)
// pushes it through the ReLU relaxation (layers/common/crown_dense.rs:41-290: e * |slope| + gap where the sign of
// the coefficient is certain, e * (|ls| + |us|) + gap where it is not, the intercepts' share folded into the bias)
// and discharges it only at the input box, lb -= sum_j err_j * max(|x_l|, |x_u|) (bounds/concretize.rs:443-466).
// On deep networks that chain grows with the product of the layers' |W| norms and visibly loosens the bound, so
// the two conventions differ by more than 1e-4 there.  This file is the second convention, selectable with
// nyb200_set_error_channel(e, NYB200_ERRCH_REFERENCE): same intermediate-bound pipeline, same relaxation
// tables, but this backward pass, so that the plain-CROWN entry point returns the reference's numbers.
// Linear layers without residual connections only.
#include "nyb200_internal.cuh"

namespace nyb {

namespace {

__device__ __forceinline__ float nup32(float x) {
    unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return __uint_as_float(1u);
    return (b & 0x80000000u) ? __uint_as_float(b - 1) : __uint_as_float(b + 1);
}
__device__ __forceinline__ float ndn32(float x) {
    unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return __uint_as_float(0x80000001u);
    return (b & 0x80000000u) ? __uint_as_float(b + 1) : __uint_as_float(b - 1);
}
constexpr float kMinPos = 1.17549435e-38f;
constexpr float kCoeffMax = 1e10f;  // crates/ny-core/src/gemm.rs:116
__device__ __forceinline__ bool coeff_safe(float v) { return isfinite(v) && fabsf(v) < kCoeffMax; }
// layers/linear/bias.rs:73-142: directed casts that never produce a subnormal
__device__ __forceinline__ float cast_down_ns(double v) {
    if (isnan(v) || v == -INFINITY) return -INFINITY;
    if (v == INFINITY) return INFINITY;
    if (v == 0.0) return 0.f;
    if (fabs(v) < (double)kMinPos) return v < 0.0 ? -kMinPos : 0.f;
    float n = __double2float_rd(v);
    if (n == INFINITY) return 3.4028234663852886e38f;
    return n;
}
__device__ __forceinline__ float cast_up_ns(double v) {
    if (isnan(v) || v == INFINITY) return INFINITY;
    if (v == -INFINITY) return -INFINITY;
    if (v == 0.0) return 0.f;
    if (fabs(v) < (double)kMinPos) return v < 0.0 ? 0.f : kMinPos;
    float n = __double2float_ru(v);
    if (n == -INFINITY) return -3.4028234663852886e38f;
    return n;
}
// layers/linear/bias.rs:146-154
__device__ __forceinline__ float publish_error_up_normal(double v) {
    if (isnan(v) || v < 0.0 || v == INFINITY) return INFINITY;
    if (v == 0.0) return 0.f;
    return nup32(cast_up_ns(v));
}
// layers/linear/bias.rs:158-167: a negative or non-finite stored error counts as infinite
__device__ __forceinline__ double err_or_inf(float v) {
    unsigned b = __float_as_uint(v), mag = b & 0x7fffffffu;
    if ((mag >> 23) == 0xff || ((b >> 31) != 0 && mag != 0)) return INFINITY;
    return (double)v;
}

// One layer of A' = A W with the error matrix: binary64 sums of the exact products, of their magnitudes and
// (upward) of err * |W|.  64 x 64 output tile, 4 x 4 per thread.  A row with an unsafe coefficient or a
// non-finite error is flagged in rowbad (the row is zeroed and its bias made infinite by k_ref_bias).
constexpr int RM = 64, RN = 64, RK = 16;
__global__ void __launch_bounds__(256)
k_ref_linear(int M, int N, int K, const float *__restrict__ A, int lda, const float *__restrict__ E, int lde,
             const float *__restrict__ W, int ldw, float *__restrict__ Ao, int ldo, float *__restrict__ Eo, int ldeo,
             int *__restrict__ rowbad) {
    __shared__ float sA[RK][RM + 1], sE[RK][RM + 1], sW[RK][RN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * RM, n0 = blockIdx.x * RN;
    double acc[4][4], sab[4][4], pe[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = sab[i][j] = pe[i][j] = 0.0;
    for (int k0 = 0; k0 < K; k0 += RK) {
        for (int t = threadIdx.x; t < RM * RK; t += 256) {
            int r = t / RK, kk = t % RK;
            int m = m0 + r, k = k0 + kk;
            bool in = m < M && k < K;
            sA[kk][r] = in ? A[(long)m * lda + k] : 0.f;
            sE[kk][r] = (in && E) ? E[(long)m * lde + k] : 0.f;
        }
        for (int t = threadIdx.x; t < RK * RN; t += 256) {
            int kk = t / RN, c = t % RN;
            int k = k0 + kk, n = n0 + c;
            sW[kk][c] = (k < K && n < N) ? W[(long)k * ldw + n] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RK; ++kk) {
            double a[4], ea[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = sA[kk][ty * 4 + i]; ea[i] = err_or_inf(sE[kk][ty * 4 + i]); }
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = sW[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const double aw = fabs(w[j]);
                    acc[i][j] = fma(a[i], w[j], acc[i][j]);
                    sab[i][j] = fma(fabs(a[i]), aw, sab[i][j]);
                    if (ea[i] != 0.0 && aw != 0.0) pe[i][j] = __dadd_ru(pe[i][j], __dmul_ru(ea[i], aw));
                }
        }
        __syncthreads();
    }
    const double d = (double)K * 1.1102230246251565e-16;  // K * 2^-53
    const double gamma = d >= 1.0 ? INFINITY : d / (1.0 - d);  // crown_single.rs:124-135
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
        bool bad = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = (float)acc[i][j];
            double cast_err = fabs(acc[i][j] - (double)v);
            double prop = E ? (double)publish_error_up_normal(pe[i][j]) : 0.0;
            float err = publish_error_up_normal(cast_err + gamma * sab[i][j] + prop);
            if (coeff_safe(v) && isfinite(err)) { Ao[(long)m * ldo + n] = v; Eo[(long)m * ldeo + n] = err; }
            else { Ao[(long)m * ldo + n] = 0.f; Eo[(long)m * ldeo + n] = 0.f; bad = true; }
        }
        if (bad) rowbad[m] = 1;
    }
}

// Bias of the same layer: b' = b + A . bias_k (directed binary64 sums of the exact products: downward for the
// lower rows, upward for the upper rows), widened by sum_k err_k |bias_k| (crown_single.rs:2142-2166), cast with
// the direction of the row (bias.rs:73-142).  A flagged row is zeroed and its bias made -inf / +inf
// (crown_single.rs:2180-2216).  One warp per row; the warp's partial sums are combined with directed additions.
__global__ void __launch_bounds__(256)
k_ref_bias(int M, int K, int N, int R, int S, const float *__restrict__ A, int lda, const float *__restrict__ E, int lde,
           const float *__restrict__ bias, float *__restrict__ Ao, int ldo, float *__restrict__ Eo, int ldeo,
           int *__restrict__ rowbad, float *__restrict__ rbf) {
    int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (m >= M) return;
    const bool upper = (m % R) >= S;
    double acc = 0.0, ee = 0.0;
    if (bias) {
        for (int k = lane; k < K; k += 32) {
            double a = A[(long)m * lda + k], b = bias[k];
            double t = a * b;  // exact: two fp32 factors
            if (t != 0.0) acc = upper ? __dadd_ru(acc, t) : __dadd_rd(acc, t);
            if (E) {
                double ba = fabs(b);
                if (ba != 0.0) ee = __dadd_ru(ee, __dmul_ru(err_or_inf(E[(long)m * lde + k]), ba));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            double oa = __shfl_xor_sync(0xffffffffu, acc, o), oe = __shfl_xor_sync(0xffffffffu, ee, o);
            acc = upper ? __dadd_ru(acc, oa) : __dadd_rd(acc, oa);
            ee = __dadd_ru(ee, oe);
        }
    }
    const int bad = rowbad[m];
    if (bad) {
        for (int j = lane; j < N; j += 32) { Ao[(long)m * ldo + j] = 0.f; Eo[(long)m * ldeo + j] = 0.f; }
    }
    if (lane == 0) {
        float bnew = rbf[m];
        if (bias) {
            double tot = upper ? __dadd_ru(acc, ee) : __dadd_rd(acc, -ee);
            bnew = upper ? cast_up_ns(__dadd_ru((double)bnew, tot)) : cast_down_ns(__dadd_rd((double)bnew, tot));
        }
        if (bad) bnew = upper ? INFINITY : -INFINITY;
        rbf[m] = bnew;
        rowbad[m] = 0;
    }
}

// Plain-CROWN ReLU step with the error carry (crown_dense.rs:41-290 with compose.rs:84-185): in place on one
// row per warp.  tab = (lower slope, upper slope, upper intercept, lower intercept); ReLU's own lower line has no
// intercept (0 there), caller-baked tables may carry one.
__global__ void __launch_bounds__(256)
k_ref_relu(int M, int n, int R, int S, long nps, int off, float *__restrict__ A, int lda, float *__restrict__ E, int lde,
           const float4 *__restrict__ tab, float *__restrict__ rbf) {
    int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (m >= M) return;
    const bool upper = (m % R) >= S;
    const int d = m / R;
    double b64 = 0.0, berr = 0.0;
    bool nonfinite = false;
    for (int j = lane; j < n; j += 32) {
        const float4 t = tab[(long)d * nps + off + j];
        const float a = A[(long)m * lda + j];
        const float ls = t.x, us = t.y, ui = t.z, li = t.w;
        float c = 0.f;
        double slope = 0.0, icp_used = 0.0;
        if (a > 0.f) {
            const float s = upper ? us : ls;
            const float p = a * s;
            slope = (double)s;
            c = isfinite(p) ? (upper ? nup32(p) : ndn32(p)) : 0.f;
            nonfinite |= !isfinite(p);
            icp_used = upper ? (double)ui : (double)li;
        } else if (a < 0.f) {
            const float s = upper ? ls : us;
            const float p = a * s;
            slope = (double)s;
            c = isfinite(p) ? (upper ? nup32(p) : ndn32(p)) : 0.f;
            nonfinite |= !isfinite(p);
            icp_used = upper ? (double)li : (double)ui;
        }
        b64 += (double)a * icp_used;
        const double gap = (a != 0.f) ? fabs((double)a * slope - (double)c) : 0.0;
        const double ea = (double)E[(long)m * lde + j];
        float eo = 0.f;
        if (gap != 0.0 || ea != 0.0) {
            double sc, ic;
            if (fabs((double)a) > ea) { sc = fabs(slope); ic = fabs(icp_used); }
            else { sc = (double)(fabsf(ls) + fabsf(us)); ic = (double)(fabsf(ui) + fabsf(li)); }
            eo = nup32((float)(ea * sc + gap));
            if (ea != 0.0) berr += ea * ic;
        }
        A[(long)m * lda + j] = c;
        E[(long)m * lde + j] = eo;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        b64 += __shfl_xor_sync(0xffffffffu, b64, o);
        berr += __shfl_xor_sync(0xffffffffu, berr, o);
    }
    nonfinite = __any_sync(0xffffffffu, nonfinite);
    if (nonfinite) {
        for (int j = lane; j < n; j += 32) { A[(long)m * lda + j] = 0.f; E[(long)m * lde + j] = 0.f; }
    }
    if (lane == 0) {
        double v = (double)rbf[m] + b64 + (upper ? berr : -berr);
        float out = (v == 0.0) ? 0.f : (upper ? nup32((float)v) : ndn32((float)v));
        if (nonfinite) out = upper ? INFINITY : -INFINITY;
        rbf[m] = out;
    }
}

// Concretisation with the error discharge (bounds/concretize.rs:374-489): sign-routed sum on the box, minus /
// plus sum_j err_j max(|x_l|, |x_u|), binary64 with an outward slack for the summation, outward cast.
__global__ void __launch_bounds__(256)
k_ref_concretize(int M, int R, int S, int n0, const float *__restrict__ A, int lda, const float *__restrict__ E, int lde,
                 const float *__restrict__ in_lo, const float *__restrict__ in_hi, long box_ds,
                 const float *__restrict__ rbf, float *__restrict__ out_lo, float *__restrict__ out_hi) {
    int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (m >= M) return;
    const int d = m / R, rr = m % R;
    const bool upper = rr >= S;
    const float *xl = in_lo + (long)d * box_ds, *xu = in_hi + (long)d * box_ds;
    double s = 0.0, sa = 0.0, pen = 0.0;
    bool bad = false;
    for (int j = lane; j < n0; j += 32) {
        const float a = A[(long)m * lda + j];
        const bool nonneg = !(__float_as_uint(a) >> 31) || (__float_as_uint(a) & 0x7fffffffu) == 0;
        const float x = (nonneg != upper) ? xl[j] : xu[j];
        if (!coeff_safe(a)) bad = true;
        if (a != 0.f && x != 0.f) { double c = (double)a * (double)x; s += c; sa += fabs(c); }
        const double e = err_or_inf(E[(long)m * lde + j]);
        const double mx = fmax(fabs((double)xl[j]), fabs((double)xu[j]));
        if (e != 0.0 && mx != 0.0) pen = __dadd_ru(pen, __dmul_ru(e, mx));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        sa += __shfl_xor_sync(0xffffffffu, sa, o);
        pen = __dadd_ru(pen, __shfl_xor_sync(0xffffffffu, pen, o));
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) {
        const double b = (double)rbf[m];
        const double slack = (sa + fabs(b)) * (double)(n0 + 2) * 1.1102230246251565e-16 * 1.000001;
        if (!upper) {
            double x = b + s - slack - pen;
            float v = (bad || isnan(x) || b == -INFINITY) ? -INFINITY : ndn32(__double2float_rd(x));
            out_lo[(long)d * S + rr] = v;
        } else {
            double x = b + s + slack + pen;
            float v = (bad || isnan(x) || b == INFINITY) ? INFINITY : nup32(__double2float_ru(x));
            out_hi[(long)d * S + (rr - S)] = v;
        }
    }
}

// rows of A from an asymmetric seed: lower rows take lower_a, upper rows upper_a
__global__ void k_seed_rows(int S, int dim, int D, int lda, const float *__restrict__ la, const float *__restrict__ ua,
                            float *__restrict__ A) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * 2 * S * dim) return;
    int j = (int)(t % dim);
    long m = t / dim;
    int rr = (int)(m % (2 * S));
    A[m * lda + j] = rr < S ? la[(long)rr * dim + j] : ua[(long)(rr - S) * dim + j];
}

}  // namespace

// The backward pass of run_backward in the reference's error convention.  Same arguments; checkpoints are not
// supported (the parameter optimisation keeps the default convention).
int run_backward_ref(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int top, const RefSeed *seed) {
    const NetView &nv = net.v;
    for (int k = 0; k < nv.L; ++k)
        if (net.is_conv(k) || net.skip_of(k) >= 0)
            return set_err(e, NYB200_ERR_UNSUPPORTED, "the reference error channel covers Linear layers without skips only");
    const bool partial = top >= 0;
    const int D = b.D, S = b.S, R = b.R, L = partial ? top + 1 : nv.L;
    const int M = D * R;
    const long np = nv.nps;
    cudaStream_t st = e->stream;
    NYB_WS(E0, float *, e, "ref_E0", (size_t)M * p.lda * 4);
    NYB_WS(E1, float *, e, "ref_E1", (size_t)M * p.lda * 4);
    NYB_WS(rbf, float *, e, "ref_bias", (size_t)M * 4);
    NYB_WS(rowbad, int *, e, "ref_rowbad", (size_t)M * 4);
    NYB_CUDA(e, cudaMemsetAsync(rbf, 0, (size_t)M * 4, st));
    NYB_CUDA(e, cudaMemsetAsync(rowbad, 0, (size_t)M * 4, st));
    static const float init_words[8] = {INFINITY, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    NYB_CUDA(e, cudaMemcpyAsync(p.min_lower, init_words, sizeof(init_words), cudaMemcpyHostToDevice, st));
    float *cur = p.A0, *nxt = p.A1, *ecur = E0, *enxt = E1;
    if (seed) {
        // an asymmetric frontier handed over by the caller: its own lower / upper rows and biases
        long tot = (long)D * 2 * S * nv.dims[L];
        k_seed_rows<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(S, nv.dims[L], D, p.lda, seed->lower_a, seed->upper_a, cur);
        e->launches++;
        if (seed->bias)
            for (int d = 0; d < D; ++d)
                NYB_CUDA(e, cudaMemcpyAsync(rbf + (size_t)d * 2 * S, seed->bias, (size_t)2 * S * 4, cudaMemcpyDeviceToDevice, st));
    } else if (partial) launch_seed_identity(e, S, D, p.lda, cur);
    else launch_seed(e, p.spec, S, nv.dims[L], D, p.lda, cur);
    bool have_err = false;  // the seed carries no error matrix
    const unsigned row_grid = (unsigned)(((long)M * 32 + 255) / 256);
    if (seed && seed->relu_first) {
        // the frontier sits behind the last activation: relax it first, from an exact (all-zero) error matrix
        NYB_CUDA(e, cudaMemsetAsync(ecur, 0, (size_t)M * p.lda * 4, st));
        k_ref_relu<<<row_grid, 256, 0, st>>>(M, nv.dims[L], R, S, np, nv.pre_off[L - 1], cur, p.lda, ecur, p.lda, p.tab, rbf);
        e->launches++;
        have_err = true;
    }
    for (int k = L - 1; k >= 0; --k) {
        NYB_DEADLINE(e, "backward pass");
        const int K = nv.dims[k + 1], N = nv.dims[k];
        dim3 grid((N + RN - 1) / RN, (M + RM - 1) / RM);
        k_ref_linear<<<grid, 256, 0, st>>>(M, N, K, cur, p.lda, have_err ? ecur : nullptr, p.lda, nv.W[k], N, nxt, p.lda, enxt,
                                           p.lda, rowbad);
        k_ref_bias<<<row_grid, 256, 0, st>>>(M, K, N, R, S, cur, p.lda, have_err ? ecur : nullptr, p.lda, nv.b[k], nxt, p.lda,
                                             enxt, p.lda, rowbad, rbf);
        e->launches += 2;
        float *t = cur; cur = nxt; nxt = t;
        t = ecur; ecur = enxt; enxt = t;
        have_err = true;
        if (k > 0) {
            k_ref_relu<<<row_grid, 256, 0, st>>>(M, N, R, S, np, nv.pre_off[k - 1], cur, p.lda, ecur, p.lda, p.tab, rbf);
            e->launches++;
        }
    }
    p.a_final = cur;
    k_ref_concretize<<<row_grid, 256, 0, st>>>(M, R, S, nv.dims[0], cur, p.lda, ecur, p.lda, p.in_lo, p.in_hi,
                                               (long)b.box_stride, rbf, p.out_lo, p.out_hi);
    e->launches++;
    // flags, repair rule and the global minimum as in the default convention (no loose-domain count: nothing here
    // depends on the tensor path's rounding)
    launch_finalize(e, D, S, p.flags, p.out_lo, p.out_hi, p.min_lower);
    NYB_CUDA(e, cudaGetLastError());
    return NYB200_OK;
}

}  // namespace nyb

extern "C" int32_t nyb200_set_error_channel(nyb200_engine *e, int32_t mode) {
    if (!e) return NYB200_ERR_INVALID;
    if (mode != NYB200_ERRCH_IMMEDIATE && mode != NYB200_ERRCH_REFERENCE) return nyb::set_err(e, NYB200_ERR_INVALID, "unknown error-channel mode");
    std::lock_guard<std::mutex> g(e->mu);
    e->error_channel = mode;
    return NYB200_OK;
}
