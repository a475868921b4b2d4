// Conv2d layers of the bound-propagation path (NCHW flattened, dilation 1, one group): the interval forward
// pass, the CROWN backward step as a transposed convolution of the coefficient rows, and the plain forward
// convolution the parameter adjoint needs.  The kernels here accumulate exact fp32 x fp32 products in
// binary64, as the reference does for convolutions ("always recomputed in f64",
// crates/ny-propagate/src/layers/convolution/conv2d/bound.rs:601-900; engine op conv_transpose_2d,
// crates/ny-core/src/gemm.rs:540-566, geometry :150-178), so their rounding model is the binary64 one of
// k_ibp_linear / k_gemm_f64: gamma_{n+2} with n the longest accumulation, and an exactly measured cast error.
// On the tensor-core path the backward step is instead the reference's own decomposition - reshape, GEMM with
// W_col, col2im - with the GEMM on the tcgen05 contraction (reading the coefficient rows channel-strided, so
// the reshape costs nothing) and k_col2im below as the gather; its rounding rate is the contraction's.
// The weights are W_col [oc x ic*kh*kw] row-major (the layout of GpuCrownLayer::Conv2d::weight_col).
#include "nyb200_internal.cuh"

namespace nyb {

namespace {

// Interval image of the convolution for Deff boxes: one thread per (box, output element).
// lo = W+ * zl + W- * zu + b, hi = W+ * zu + W- * zl + b, q = |W| * max(|zl|, |zu|)
// (interval conv: conv2d/bound.rs:86-268).
__global__ void __launch_bounds__(256)
k_ibp_conv(ConvGeom g, int Deff, const float *__restrict__ W, const float *__restrict__ bias,
           const float *__restrict__ zl, const float *__restrict__ zu, long in_ds, float *__restrict__ raw_lo,
           float *__restrict__ raw_hi, float *__restrict__ q, long out_ds) {
    const int n_out = g.oc * g.oh * g.ow, taps = g.ic * g.kh * g.kw;
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)Deff * n_out) return;
    int d = (int)(t / n_out), o = (int)(t % n_out);
    int co = o / (g.oh * g.ow), oy = (o / g.ow) % g.oh, ox = o % g.ow;
    const float *w = W + (long)co * taps;
    const float *a = zl + (long)d * in_ds, *b = zu + (long)d * in_ds;
    double lo = 0.0, hi = 0.0, qq = 0.0;
    for (int ci = 0; ci < g.ic; ++ci)
        for (int ky = 0; ky < g.kh; ++ky) {
            int iy = oy * g.sh - g.ph + ky;
            if (iy < 0 || iy >= g.ih) continue;
            for (int kx = 0; kx < g.kw; ++kx) {
                int ix = ox * g.sw - g.pw + kx;
                if (ix < 0 || ix >= g.iw) continue;
                double wv = w[(ci * g.kh + ky) * g.kw + kx];
                int j = (ci * g.ih + iy) * g.iw + ix;
                double l = a[j], u = b[j];
                bool pos = wv > 0.0;
                lo = fma(wv, pos ? l : u, lo);
                hi = fma(wv, pos ? u : l, hi);
                qq = fma(fabs(wv), fmax(fabs(l), fabs(u)), qq);
            }
        }
    const double gam = (double)(taps + 2) * 1.1102230246251565e-16 * 1.000001;
    double bv = bias ? (double)bias[o] : 0.0;
    double slack = gam * (qq + fabs(bv));
    float lf = __double2float_rd(lo + bv - slack), hf = __double2float_ru(hi + bv + slack);
    if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
    raw_lo[(long)d * out_ds + o] = lf;
    raw_hi[(long)d * out_ds + o] = hf;
    q[(long)d * out_ds + o] = __double2float_ru(qq * (1.0 + gam));
}

// CROWN backward through the convolution: C[m, (ci, y, x)] = sum_{co, ky, kx} A[m, (co, oy, ox)] W[co, ci, ky, kx]
// over the (oy, ox) with oy*sh - ph + ky = y, ox*sw - pw + kx = x (conv2d_transpose_backward_coeff_f64,
// conv2d/ops_transpose_gemm.rs; reshape + GEMM + col2im in the reference, a direct gather here: no scatter,
// no atomics on the coefficients).  One block per row: the row of A is staged in shared memory (when it fits),
// every thread produces output elements from it.  The cast of each binary64 sum to fp32 is measured exactly and
// charged against the magnitude of the variable the coefficient multiplies (rpen), like k_gemm_f64.
__global__ void __launch_bounds__(256)
k_conv_transpose(ConvGeom g, int M, const float *__restrict__ A, int lda, float *__restrict__ C, int ldc,
                 const float *__restrict__ W, int R, const float *__restrict__ zin_lo, const float *__restrict__ zin_hi,
                 long zin_ds, double *__restrict__ rpen, int stage) {
    extern __shared__ float s_row[];
    const int n_out = g.oc * g.oh * g.ow, n_in = g.ic * g.ih * g.iw, taps = g.ic * g.kh * g.kw, plane = g.oh * g.ow;
    int m = blockIdx.x;
    if (m >= M) return;
    const float *arow = A + (long)m * lda;
    if (stage) {
        for (int i = threadIdx.x; i < n_out; i += blockDim.x) s_row[i] = arow[i];
        __syncthreads();
    }
    const float *src = stage ? s_row : arow;
    const int d = m / R;
    double pen = 0.0;
    for (int j = threadIdx.x; j < n_in; j += blockDim.x) {
        int ci = j / (g.ih * g.iw), y = (j / g.iw) % g.ih, x = j % g.iw;
        double acc = 0.0;
        for (int ky = 0; ky < g.kh; ++ky) {
            int ty = y + g.ph - ky;
            if (ty < 0 || ty % g.sh) continue;
            int oy = ty / g.sh;
            if (oy >= g.oh) continue;
            for (int kx = 0; kx < g.kw; ++kx) {
                int tx = x + g.pw - kx;
                if (tx < 0 || tx % g.sw) continue;
                int ox = tx / g.sw;
                if (ox >= g.ow) continue;
                const float *wp = W + (ci * g.kh + ky) * g.kw + kx;
                const float *ap = src + oy * g.ow + ox;
#pragma unroll 4
                for (int co = 0; co < g.oc; ++co) acc = fma((double)ap[co * plane], (double)wp[(long)co * taps], acc);
            }
        }
        float c = (float)acc;
        C[(long)m * ldc + j] = c;
        if (rpen) {
            float zm = fmaxf(fabsf(zin_lo[(long)d * zin_ds + j]), fabsf(zin_hi[(long)d * zin_ds + j]));
            pen += fabs(acc - (double)c) * (double)zm;
        }
    }
    if (rpen) {
        __shared__ double s_pen[8];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pen += __shfl_xor_sync(0xffffffffu, pen, o);
        if ((threadIdx.x & 31) == 0) s_pen[threadIdx.x >> 5] = pen;
        __syncthreads();
        if (threadIdx.x == 0) {
            double tot = 0.0;
            for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += s_pen[i];
            if (tot != 0.0) atomicAdd(&rpen[m], tot);
        }
    }
}

// Quotient of small non-negative integers by a runtime divisor through its float reciprocal (exact for
// n < 2^22: the +0.5 keeps the product away from the integer boundaries the rounding of 1/d could cross).
__device__ __forceinline__ int small_div(int n, float inv_d) { return __float2int_rd(((float)n + 0.5f) * inv_d); }

// col2im as a gather: C[m, (ci, y, x)] = sum over the taps (ky, kx) that reach (y, x) of the im2col-space
// products, the second half of the reference's reshape + GEMM + col2im decomposition (GpuCrownLayer::Conv2d,
// crates/ny-core/src/gemm.rs:1553-1562).  The products arrive tap-major, cols[(m * taps + tap) * plane + (oy, ox)],
// so threads with consecutive x read consecutive words of one tap's plane.  The few fp32 entries of an output
// are summed in binary64 and cast once; that cast (at most 2^-24 of the sum of the term magnitudes) is part of
// the rounding rate the relaxation pass charges for this layer, so nothing is accumulated here.
__global__ void __launch_bounds__(256)
k_col2im(ConvGeom g, const float *__restrict__ cols, float *__restrict__ C, int ldc, float inv_iw, float inv_sh,
         float inv_sw) {
    const int in_plane = g.ih * g.iw, plane = g.oh * g.ow, kk = g.kh * g.kw;
    const int m = blockIdx.x, ci = blockIdx.y;
    const int pix = blockIdx.z * blockDim.x + threadIdx.x;
    if (pix >= in_plane) return;
    const int y = small_div(pix, inv_iw), x = pix - y * g.iw;
    // valid taps: ky = ky0 + i*sh with oy = yq - i, kx = kx0 + i*sw with ox = xq - i
    const int yq = small_div(y + g.ph, inv_sh), ky0 = (y + g.ph) - yq * g.sh;
    const int xq = small_div(x + g.pw, inv_sw), kx0 = (x + g.pw) - xq * g.sw;
    const float *base = cols + ((long)m * g.ic + ci) * kk * plane;
    double acc = 0.0;
    for (int ky = ky0, oy = yq; ky < g.kh && oy >= 0; ky += g.sh, --oy) {
        if (oy >= g.oh) continue;
        for (int kx = kx0, ox = xq; kx < g.kw && ox >= 0; kx += g.sw, --ox) {
            if (ox >= g.ow) continue;
            acc += (double)base[(ky * g.kw + kx) * plane + oy * g.ow + ox];
        }
    }
    C[(long)m * ldc + ci * in_plane + pix] = (float)acc;
}

// Same gather for layers whose outputs have at most 16 taps each (every stride >= kernel / 4): one thread per
// pixel keeps the tap offsets in registers and walks the input channels, four at a time, so that sixteen or
// more independent loads are in flight per thread (the one-output-per-thread form above is latency bound).
__global__ void __launch_bounds__(256)
k_col2im_t16(ConvGeom g, const float *__restrict__ cols, float *__restrict__ C, int ldc, float inv_iw, float inv_sh,
             float inv_sw) {
    const int in_plane = g.ih * g.iw, plane = g.oh * g.ow, kk = g.kh * g.kw;
    const int m = blockIdx.x;
    const int pix = blockIdx.y * blockDim.x + threadIdx.x;
    if (pix >= in_plane) return;
    const int y = small_div(pix, inv_iw), x = pix - y * g.iw;
    const int yq = small_div(y + g.ph, inv_sh), ky0 = (y + g.ph) - yq * g.sh;
    const int xq = small_div(x + g.pw, inv_sw), kx0 = (x + g.pw) - xq * g.sw;
    int off[16];
    int nt = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int ky = ky0 + i * g.sh, oy = yq - i;
        bool vy = ky < g.kh && oy >= 0 && oy < g.oh;
#pragma unroll
        for (int i2 = 0; i2 < 4; ++i2) {
            int kx = kx0 + i2 * g.sw, ox = xq - i2;
            bool v = vy && kx < g.kw && ox >= 0 && ox < g.ow;
            off[i * 4 + i2] = v ? (ky * g.kw + kx) * plane + oy * g.ow + ox : -1;
            nt += v ? 1 : 0;
        }
    }
    const float *base = cols + (long)m * g.ic * kk * plane;
    float *out = C + (long)m * ldc + pix;
    const int cstride = kk * plane;
    for (int ci = 0; ci < g.ic; ci += 4) {
        double acc[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            if (off[t] < 0) continue;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (ci + u < g.ic) acc[u] += (double)base[(long)(ci + u) * cstride + off[t]];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (ci + u < g.ic) out[(long)(ci + u) * in_plane] = (float)acc[u];
    }
}

// Binary64 form of the same decomposition (the path used when binary64 contractions are selected, and by the
// re-evaluation of batches the fast path flags): the im2col-space product as a 64 x 64 x 16 register-tiled
// binary64 GEMM whose rows read the coefficient tensor channel-strided and whose results are kept in binary64,
// tap-major, so that the gather below adds exact products' sums and only the final cast rounds.
constexpr int CG_M = 64, CG_N = 64, CG_K = 16;
__global__ void __launch_bounds__(256)
k_conv_gemm_f64(int Mrows, int N, int K, int plane, const float *__restrict__ A, int lda, const float *__restrict__ B,
                double *__restrict__ cols) {
    __shared__ float sA[CG_K][CG_M + 1], sB[CG_K][CG_N + 1];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.x * CG_M, n0 = blockIdx.y * CG_N;
    double acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
    for (int k0 = 0; k0 < K; k0 += CG_K) {
        for (int t = threadIdx.x; t < CG_M * CG_K; t += 256) {
            int kk = t / CG_M, r = t % CG_M;  // consecutive threads: consecutive rows = consecutive pixels
            int row = m0 + r, k = k0 + kk;
            sA[kk][r] = (row < Mrows && k < K) ? A[(long)(row / plane) * lda + (long)k * plane + (row % plane)] : 0.f;
        }
        for (int t = threadIdx.x; t < CG_K * CG_N; t += 256) {
            int kk = t / CG_N, c = t % CG_N;
            int k = k0 + kk, n = n0 + c;
            sB[kk][c] = (k < K && n < N) ? B[(long)k * N + n] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < CG_K; ++kk) {
            double a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty + 16 * i];
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
        int row = m0 + ty + 16 * i;
        if (row >= Mrows) continue;
        long m = row / plane;
        int p = row % plane;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n < N) cols[(m * N + n) * plane + p] = acc[i][j];
        }
    }
}

// Gather of the binary64 products: one thread per pixel walks the input channels; the cast of each sum to fp32
// is measured and charged against the magnitude of the variable the coefficient multiplies.
__global__ void __launch_bounds__(256)
k_col2im_f64(ConvGeom g, const double *__restrict__ cols, float *__restrict__ C, int ldc, int R,
             const float *__restrict__ zin_lo, const float *__restrict__ zin_hi, long zin_ds, double *__restrict__ rpen,
             float inv_iw, float inv_sh, float inv_sw) {
    const int in_plane = g.ih * g.iw, plane = g.oh * g.ow, kk = g.kh * g.kw;
    const int m = blockIdx.x;
    const int pix = blockIdx.y * blockDim.x + threadIdx.x;
    double pen = 0.0;
    if (pix < in_plane) {
        const int y = small_div(pix, inv_iw), x = pix - y * g.iw;
        const int yq = small_div(y + g.ph, inv_sh), ky0 = (y + g.ph) - yq * g.sh;
        const int xq = small_div(x + g.pw, inv_sw), kx0 = (x + g.pw) - xq * g.sw;
        const double *base = cols + (long)m * g.ic * kk * plane;
        const int d = m / R;
        for (int ci = 0; ci < g.ic; ++ci) {
            const double *bc = base + (long)ci * kk * plane;
            double acc = 0.0;
            for (int ky = ky0, oy = yq; ky < g.kh && oy >= 0; ky += g.sh, --oy) {
                if (oy >= g.oh) continue;
                for (int kx = kx0, ox = xq; kx < g.kw && ox >= 0; kx += g.sw, --ox) {
                    if (ox >= g.ow) continue;
                    acc += bc[(ky * g.kw + kx) * plane + oy * g.ow + ox];
                }
            }
            int j = ci * in_plane + pix;
            float c = (float)acc;
            C[(long)m * ldc + j] = c;
            if (rpen) {
                float zm = fmaxf(fabsf(zin_lo[(long)d * zin_ds + j]), fabsf(zin_hi[(long)d * zin_ds + j]));
                pen += fabs(acc - (double)c) * (double)zm;
            }
        }
    }
    if (rpen) {
        __shared__ double s_pen[8];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pen += __shfl_xor_sync(0xffffffffu, pen, o);
        if ((threadIdx.x & 31) == 0) s_pen[threadIdx.x >> 5] = pen;
        __syncthreads();
        if (threadIdx.x == 0) {
            double tot = 0.0;
            for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += s_pen[i];
            if (tot != 0.0) atomicAdd(&rpen[m], tot);
        }
    }
}

// Plain forward convolution of `rows` vectors (no bias): out[r, o] = sum W[co, ci, ky, kx] Z[r, (ci, iy, ix)].
__global__ void __launch_bounds__(256)
k_conv_plain(ConvGeom g, int rows, const float *__restrict__ Z, int ldz, const float *__restrict__ W,
             float *__restrict__ out, int ldo) {
    const int n_out = g.oc * g.oh * g.ow, taps = g.ic * g.kh * g.kw;
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)rows * n_out) return;
    int r = (int)(t / n_out), o = (int)(t % n_out);
    int co = o / (g.oh * g.ow), oy = (o / g.ow) % g.oh, ox = o % g.ow;
    const float *w = W + (long)co * taps;
    const float *z = Z + (long)r * ldz;
    double acc = 0.0;
    for (int ci = 0; ci < g.ic; ++ci)
        for (int ky = 0; ky < g.kh; ++ky) {
            int iy = oy * g.sh - g.ph + ky;
            if (iy < 0 || iy >= g.ih) continue;
            for (int kx = 0; kx < g.kw; ++kx) {
                int ix = ox * g.sw - g.pw + kx;
                if (ix < 0 || ix >= g.iw) continue;
                acc = fma((double)w[(ci * g.kh + ky) * g.kw + kx], (double)z[(ci * g.ih + iy) * g.iw + ix], acc);
            }
        }
    out[(long)r * ldo + o] = (float)acc;
}

// ---- forward convolutions on the tensor cores -----------------------------------------------------------------
// A convolution is, per input pixel, a product of that pixel's channel vector with every (output channel, tap)
// weight, followed by a gather: y[co, oy, ox] = sum_{ky, kx} P[(iy, ix), (co, ky, kx)] with iy = oy*sh - ph + ky.
// The product P = x[:, pixel] * Wf, Wf [ic x oc*kh*kw], is the same contraction as the transposed convolution's
// (channel-strided operand, tap-major result); only the gather differs.  Any stride is covered (a stride s uses
// one tap in s*s per pixel; the unused products are wasted tensor work, not traffic that matters here).

// Wf[ci][(co, ky, kx)] = W_col[co][(ci, ky, kx)]; with `split`: [max(W, 0) | min(W, 0)], 2*oc*kk columns.
__global__ void k_build_conv_fwd(const float *__restrict__ W, int oc, int ic, int kk, int split, float *__restrict__ out) {
    const int N = (split ? 2 : 1) * oc * kk;
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)ic * N) return;
    int ci = (int)(t / N), n = (int)(t % N);
    int neg = n >= oc * kk;
    int r = n - (neg ? oc * kk : 0);
    int co = r / kk, tap = r % kk;
    float w = W[((long)co * ic + ci) * kk + tap];
    out[t] = split ? (neg ? fminf(w, 0.f) : fmaxf(w, 0.f)) : w;
}

// Interval convolution from the products of the lower-end rows (m = d) and upper-end rows (m = D + d) of a
// non-negative input interval with [W+ | W-]: lo = W+ zl + W- zu + b, hi = W+ zu + W- zl + b, q = |W| zu.
// The taps of an output are summed in binary64; every product carries a rounding of at most eps times the sum of
// its term magnitudes, all bounded by q, so both ends move outward by eps * q before the directed cast (the same
// accounting as the fully connected tensor forward pass).
__global__ void __launch_bounds__(256)
k_ibp_conv_gather(ConvGeom g, int D, const float *__restrict__ cols, const float *__restrict__ bias, double eps,
                  float *__restrict__ raw_lo, float *__restrict__ raw_hi, float *__restrict__ q, long out_ds,
                  float inv_ow, float inv_plane) {
    const int plane_out = g.oh * g.ow, plane_in = g.ih * g.iw, kk = g.kh * g.kw, N = 2 * g.oc * kk;
    const int d = blockIdx.y;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= g.oc * plane_out) return;
    const int co = small_div(o, inv_plane), pix = o - co * plane_out;
    const int oy = small_div(pix, inv_ow), ox = pix - oy * g.ow;
    const float *lo_rows = cols + (long)d * N * plane_in, *hi_rows = cols + (long)(D + d) * N * plane_in;
    const long pos_off = (long)co * kk * plane_in, neg_off = (long)(g.oc + co) * kk * plane_in;
    double pl = 0.0, nl = 0.0, pu = 0.0, nu = 0.0;
    for (int ky = 0; ky < g.kh; ++ky) {
        int iy = oy * g.sh - g.ph + ky;
        if (iy < 0 || iy >= g.ih) continue;
        for (int kx = 0; kx < g.kw; ++kx) {
            int ix = ox * g.sw - g.pw + kx;
            if (ix < 0 || ix >= g.iw) continue;
            long t = (long)(ky * g.kw + kx) * plane_in + iy * g.iw + ix;
            pl += (double)lo_rows[pos_off + t]; nl += (double)lo_rows[neg_off + t];
            pu += (double)hi_rows[pos_off + t]; nu += (double)hi_rows[neg_off + t];
        }
    }
    double b = bias ? (double)bias[o] : 0.0;
    double qq = (fabs(pu) + fabs(nu)) / (1.0 - 2.0 * eps);
    double slack = eps * qq + 2.3e-16 * (qq + fabs(b));
    float l = __double2float_rd(pl + nu + b - slack), u = __double2float_ru(pu + nl + b + slack);
    if (isnan(l) || isnan(u)) { l = -INFINITY; u = INFINITY; }
    raw_lo[(long)d * out_ds + o] = l;
    raw_hi[(long)d * out_ds + o] = u;
    q[(long)d * out_ds + o] = __double2float_ru(qq);
}

// Plain forward convolution from the per-pixel products (no bias).
__global__ void __launch_bounds__(256)
k_conv_fwd_gather(ConvGeom g, const float *__restrict__ cols, float *__restrict__ out, int ldo, float inv_ow,
                  float inv_plane) {
    const int plane_out = g.oh * g.ow, plane_in = g.ih * g.iw, kk = g.kh * g.kw, N = g.oc * kk;
    const int r = blockIdx.y;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= g.oc * plane_out) return;
    const int co = small_div(o, inv_plane), pix = o - co * plane_out;
    const int oy = small_div(pix, inv_ow), ox = pix - oy * g.ow;
    const float *base = cols + ((long)r * N + (long)co * kk) * plane_in;
    double acc = 0.0;
    for (int ky = 0; ky < g.kh; ++ky) {
        int iy = oy * g.sh - g.ph + ky;
        if (iy < 0 || iy >= g.ih) continue;
        for (int kx = 0; kx < g.kw; ++kx) {
            int ix = ox * g.sw - g.pw + kx;
            if (ix < 0 || ix >= g.iw) continue;
            acc += (double)base[(long)(ky * g.kw + kx) * plane_in + iy * g.iw + ix];
        }
    }
    out[(long)r * ldo + o] = (float)acc;
}

}  // namespace

int prepare_conv_forward_operand(nyb200_engine *e, const float *W, const ConvGeom &g, bool split, UmmaLayer *out) {
    const int kk = g.kh * g.kw, N = (split ? 2 : 1) * g.oc * kk;
    float *tmp = nullptr;
    size_t n = (size_t)g.ic * N;
    if (cudaMalloc(&tmp, n * 4) != cudaSuccess) return NYB200_ERR_OOM;
    k_build_conv_fwd<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(W, g.oc, g.ic, kk, split ? 1 : 0, tmp);
    e->launches++;
    int st = umma_prepare_layer(e, tmp, g.ic, N, out);
    if (split) out->chain = 1;  // interval products: see umma_prepare_forward_layer
    cudaStreamSynchronize(e->stream);
    cudaFree(tmp);
    return st;
}

void launch_ibp_conv_gather(nyb200_engine *e, const NetView &nv, const ConvGeom &g, int k, int D, const float *cols, double eps,
                            float *raw_lo, float *raw_hi, float *q, long out_dstride) {
    int n_out = g.oc * g.oh * g.ow;
    dim3 grid((unsigned)((n_out + 255) / 256), (unsigned)D);
    k_ibp_conv_gather<<<grid, 256, 0, e->stream>>>(g, D, cols, nv.b[k], eps, raw_lo + nv.pre_off[k], raw_hi + nv.pre_off[k],
                                                  q + nv.pre_off[k], out_dstride, 1.0f / (float)g.ow,
                                                  1.0f / (float)(g.oh * g.ow));
    e->launches++;
}

void launch_conv_fwd_gather(nyb200_engine *e, const ConvGeom &g, int rows, const float *cols, float *out, int ldo) {
    int n_out = g.oc * g.oh * g.ow;
    dim3 grid((unsigned)((n_out + 255) / 256), (unsigned)rows);
    k_conv_fwd_gather<<<grid, 256, 0, e->stream>>>(g, cols, out, ldo, 1.0f / (float)g.ow, 1.0f / (float)(g.oh * g.ow));
    e->launches++;
}

void launch_ibp_conv(nyb200_engine *e, const NetView &nv, const ConvGeom &g, int k, int Deff, const float *zl,
                     const float *zu, long in_dstride, float *raw_lo, float *raw_hi, float *q, long out_dstride) {
    long total = (long)Deff * nv.dims[k + 1];
    k_ibp_conv<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(g, Deff, nv.W[k], nv.b[k], zl, zu, in_dstride,
                                                                      raw_lo + nv.pre_off[k], raw_hi + nv.pre_off[k],
                                                                      q + nv.pre_off[k], out_dstride);
    e->launches++;
}

void launch_conv_transpose(nyb200_engine *e, const ConvGeom &g, int M, const float *A, int lda, float *C, int ldc,
                           const float *W, int R, const float *zin_lo, const float *zin_hi, long zin_dstride,
                           double *rpen, double *cols) {
    if (cols) {
        const int plane = g.oh * g.ow, taps = g.ic * g.kh * g.kw;
        const long rows = (long)M * plane;
        dim3 grid((unsigned)((rows + CG_M - 1) / CG_M), (unsigned)((taps + CG_N - 1) / CG_N));
        k_conv_gemm_f64<<<grid, 256, 0, e->stream>>>((int)rows, taps, g.oc, plane, A, lda, W, cols);
        dim3 g2((unsigned)M, (unsigned)((g.ih * g.iw + 255) / 256));
        k_col2im_f64<<<g2, 256, 0, e->stream>>>(g, cols, C, ldc, R, zin_lo, zin_hi, zin_dstride, rpen, 1.0f / (float)g.iw,
                                                 1.0f / (float)g.sh, 1.0f / (float)g.sw);
        e->launches += 2;
        return;
    }
    size_t row_bytes = (size_t)g.oc * g.oh * g.ow * sizeof(float);
    int stage = row_bytes <= 48 * 1024 ? 1 : 0;  // larger rows are read through the caches
    k_conv_transpose<<<(unsigned)M, 256, stage ? row_bytes : 0, e->stream>>>(g, M, A, lda, C, ldc, W, R, zin_lo, zin_hi,
                                                                            zin_dstride, rpen, stage);
    e->launches++;
}

void launch_col2im(nyb200_engine *e, const ConvGeom &g, int M, const float *cols, float *C, int ldc) {
    const float inv_iw = 1.0f / (float)g.iw, inv_sh = 1.0f / (float)g.sh, inv_sw = 1.0f / (float)g.sw;
    const unsigned chunks = (unsigned)((g.ih * g.iw + 255) / 256);
    if ((g.kh + g.sh - 1) / g.sh <= 4 && (g.kw + g.sw - 1) / g.sw <= 4) {
        dim3 grid((unsigned)M, chunks);
        k_col2im_t16<<<grid, 256, 0, e->stream>>>(g, cols, C, ldc, inv_iw, inv_sh, inv_sw);
    } else {
        dim3 grid((unsigned)M, (unsigned)g.ic, chunks);
        k_col2im<<<grid, 256, 0, e->stream>>>(g, cols, C, ldc, inv_iw, inv_sh, inv_sw);
    }
    e->launches++;
}

void launch_conv_plain(nyb200_engine *e, const ConvGeom &g, int rows, const float *Z, int ldz, const float *W, float *out,
                       int ldo) {
    long total = (long)rows * g.oc * g.oh * g.ow;
    k_conv_plain<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(g, rows, Z, ldz, W, out, ldo);
    e->launches++;
}

}  // namespace nyb
