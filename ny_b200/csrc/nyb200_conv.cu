// Conv2d layers of the bound-propagation path (NCHW flattened, dilation 1, one group): the interval forward
// pass, the CROWN backward step as a transposed convolution of the coefficient rows, and the plain forward
// convolution the parameter adjoint needs.  All three accumulate exact fp32 x fp32 products in binary64, as
// the reference does for convolutions on every path ("always recomputed in f64",
// crates/ny-propagate/src/layers/convolution/conv2d/bound.rs:601-900; engine op conv_transpose_2d,
// crates/ny-core/src/gemm.rs:540-566, geometry :150-178), so their rounding model is the binary64 one of
// k_ibp_linear / k_gemm_f64: gamma_{n+2} with n the longest accumulation, and an exactly measured cast error.
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

}  // namespace

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
                           double *rpen) {
    size_t row_bytes = (size_t)g.oc * g.oh * g.ow * sizeof(float);
    int stage = row_bytes <= 48 * 1024 ? 1 : 0;  // larger rows are read through the caches
    k_conv_transpose<<<(unsigned)M, 256, stage ? row_bytes : 0, e->stream>>>(g, M, A, lda, C, ldc, W, R, zin_lo, zin_hi,
                                                                            zin_dstride, rpen, stage);
    e->launches++;
}

void launch_conv_plain(nyb200_engine *e, const ConvGeom &g, int rows, const float *Z, int ldz, const float *W, float *out,
                       int ldo) {
    long total = (long)rows * g.oc * g.oh * g.ow;
    k_conv_plain<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(g, rows, Z, ldz, W, out, ldo);
    e->launches++;
}

}  // namespace nyb
