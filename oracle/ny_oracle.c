/*
 * ny_oracle.c -- CPU restatement of ny's IBP / CROWN / beta-CROWN path.
 *
 * TEST INFRASTRUCTURE ONLY (parity checker and timed CPU baseline); see ny_oracle.h.
 * Build with -ffp-contract=off: the double-double code below relies on explicit fma().
 *
 * Reference files restated here (paths inside the ny project, crates/...):
 *   ny-tensor/src/rounding.rs:17-63                       next_up/next_down
 *   ny-core/src/dd.rs:184-340                             two_sum, two_prod, dd_fma, gamma_n_dd
 *   ny-propagate/src/bounds/certified_reduction.rs:26-129 certified_affine_sum_f32
 *   ny-propagate/src/bounds/concretize.rs:26-130,374-489  concretize_row_directed
 *   ny-propagate/src/layers/linear/ibp.rs:464-523         propagate_ibp_1d
 *   ny-propagate/src/layers/linear/bias.rs:38-284         directed bias arithmetic
 *   ny-propagate/src/layers/linear/crown_single.rs:124-135,1931-2226  linear backward
 *   ny-propagate/src/layers/activations/mod.rs:99-121     upper chord
 *   ny-propagate/src/layers/activations/relu/mod.rs:105-132  relu_linear_relaxation
 *   ny-propagate/src/layers/common/compose.rs:84-185      compose_lower/upper
 *   ny-propagate/src/layers/common/crown_dense.rs:41-286  elementwise backward + error
 *   ny-propagate/src/network/ibp/crown_ibp.rs:32-420, crown_partial.rs:147-560,
 *   ny-propagate/src/network/ibp/sparse_merge.rs:118-146, crown_ibp_forward.rs:25-100
 *   ny-propagate/src/network/core/sequential/crown.rs:168-330 (+ crown/tighten.rs)
 *   ny-propagate/src/beta_crown/engine/backward/relu_backward.rs:33-185
 *   ny-propagate/src/beta_crown/engine/optimization/bound_compute.rs:90-167
 *   ny-propagate/src/beta_crown/engine/domain/child.rs:51-118
 *   ny-propagate/src/beta_crown/engine/graph/propagation/constraints/mod.rs:184-760
 *   ny-propagate/src/beta_crown/engine/branching/sequential.rs:49-104
 *   ny-propagate/src/beta_crown/config/beta_config.rs:1552-1610
 */
#include "ny_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

/* ------------------------------------------------------------------ bit helpers */
static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }
static inline uint64_t d2u(double x) { uint64_t u; memcpy(&u, &x, 8); return u; }
static inline double u2d(uint64_t u) { double x; memcpy(&x, &u, 8); return x; }

/* ny-tensor/src/rounding.rs:17-33 */
float nyo_next_up_f32(float x) {
    uint32_t b = f2u(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return u2f(1u);
    return (b & 0x80000000u) ? u2f(b - 1) : u2f(b + 1);
}
/* ny-tensor/src/rounding.rs:47-63 */
float nyo_next_down_f32(float x) {
    uint32_t b = f2u(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return u2f(0x80000001u);
    return (b & 0x80000000u) ? u2f(b + 1) : u2f(b - 1);
}
#define NUP32 nyo_next_up_f32
#define NDN32 nyo_next_down_f32

/* ny-core/src/dd.rs:312-340 */
static inline double nup64(double x) {
    uint64_t b = d2u(x), mag = b & 0x7fffffffffffffffull;
    if (mag >= 0x7ff0000000000000ull) return x;
    if (mag == 0) return u2d(1ull);
    return (b >> 63) ? u2d(b - 1) : u2d(b + 1);
}
static inline double ndn64(double x) {
    uint64_t b = d2u(x), mag = b & 0x7fffffffffffffffull;
    if (mag >= 0x7ff0000000000000ull) return x;
    if (mag == 0) return u2d(0x8000000000000001ull);
    return (b >> 63) ? u2d(b + 1) : u2d(b - 1);
}

#define F32_MIN_POSITIVE 1.17549435e-38f
#define CROWN_COEFF_MAX 1e10f /* ny-core/src/gemm.rs:116 */
static inline int coeff_safe(float v) { return isfinite(v) && fabsf(v) < CROWN_COEFF_MAX; }

/* ------------------------------------------------------------------ bias.rs directed casts */
/* layers/linear/bias.rs:73-105 */
static float f64_to_f32_down_ns(double v) {
    if (isnan(v) || v == -INFINITY) return -INFINITY;
    if (v == INFINITY) return INFINITY;
    if (v == 0.0) return 0.0f;
    if (fabs(v) < (double)F32_MIN_POSITIVE) return signbit(v) ? -F32_MIN_POSITIVE : 0.0f;
    float n = (float)v;
    if (n == INFINITY) return 3.4028234663852886e38f;
    if (n == -INFINITY) return -INFINITY;
    return ((double)n <= v) ? n : NDN32(n);
}
/* layers/linear/bias.rs:110-142 */
static float f64_to_f32_up_ns(double v) {
    if (isnan(v) || v == INFINITY) return INFINITY;
    if (v == -INFINITY) return -INFINITY;
    if (v == 0.0) return 0.0f;
    if (fabs(v) < (double)F32_MIN_POSITIVE) return signbit(v) ? 0.0f : F32_MIN_POSITIVE;
    float n = (float)v;
    if (n == -INFINITY) return -3.4028234663852886e38f;
    if (n == INFINITY) return INFINITY;
    return ((double)n >= v) ? n : NUP32(n);
}
/* layers/linear/bias.rs:146-154 */
static float publish_error_up_normal(double v) {
    if (isnan(v) || v < 0.0 || v == INFINITY) return INFINITY;
    if (v == 0.0) return 0.0f;
    return NUP32(f64_to_f32_up_ns(v));
}
/* layers/linear/bias.rs:158-167 */
static double nonneg_err_or_inf(float v) {
    uint32_t b = f2u(v), mag = b & 0x7fffffffu;
    if ((mag >> 23) == 0xff || ((b >> 31) != 0 && mag != 0)) return INFINITY;
    return (double)v;
}
/* layers/linear/bias.rs:174-204 */
static inline double add_f64_down(double acc, double term) {
    if (isnan(acc) || isnan(term)) return -INFINITY;
    if (term == 0.0) return acc;
    double s = acc + term;
    return isnan(s) ? -INFINITY : ndn64(s);
}
static inline double add_f64_up(double acc, double term) {
    if (isnan(acc) || isnan(term)) return INFINITY;
    if (term == 0.0) return acc;
    double s = acc + term;
    return isnan(s) ? INFINITY : nup64(s);
}

/* ------------------------------------------------------------------ certified reduction */
/* ny-core/src/dd.rs:184-237 */
static inline void two_sum(double a, double b, double *s, double *e) {
    double ss = a + b, bb = ss - a;
    *e = (a - (ss - bb)) + (b - bb);
    *s = ss;
}
static inline void dd_fma(double *hi, double *lo, double a, double b) {
    double p = a * b, e = fma(a, b, -p);
    double s, e2;
    two_sum(*hi, p, &s, &e2);
    double ee = e2 + e + *lo;
    two_sum(s, ee, hi, lo);
}
/* ny-core/src/dd.rs:284-304 with U_DD = 2^-102 */
static double gamma_n_dd(size_t n) {
    const double u = ldexp(1.0, -102);
    double nu_hi = nup64((double)n * u);
    double den = 1.0 - nu_hi;
    if (!(den > 0.0) || !isfinite(nu_hi)) return INFINITY;
    return nup64(nu_hi / den);
}
/* bounds/safe_math.rs:45-53 */
static inline double safe_mul(double a, double x) {
    if (a == 0.0 || x == 0.0) return 0.0;
    if (isnan(a) || isnan(x)) return NAN;
    return a * x;
}

/* bounds/certified_reduction.rs:40-129.  The term sequence is produced by a callback-free
 * gather: the caller supplies parallel arrays. */
double nyo_certified_affine_sum(float bias, const float *coef, const float *val, int n, int upper) {
    double bias64 = (double)bias;
    double hi = bias64, lo = 0.0;
    double abs_sum = fabs(bias64);
    double directed = bias64;
    size_t count = 0;
    int dd_ok = isfinite(bias);
    int exact_zero = (f2u(bias) & 0x7fffffffu) == 0;
    for (int i = 0; i < n; ++i) {
        float c = coef[i], v = val[i];
        ++count;
        double c64 = (double)c, v64 = (double)v;
        double prod = safe_mul(c64, v64);
        int cz = (f2u(c) & 0x7fffffffu) == 0, vz = (f2u(v) & 0x7fffffffu) == 0;
        exact_zero &= (cz || vz);
        double s = directed + prod;
        if (upper) directed = isnan(s) ? INFINITY : nup64(s);
        else directed = isnan(s) ? -INFINITY : ndn64(s);
        if (dd_ok && isfinite(c) && isfinite(v)) {
            dd_fma(&hi, &lo, c64, v64);
            double pm = fabs(prod);
            if (pm != 0.0) abs_sum = nup64(abs_sum + pm);
            dd_ok = isfinite(hi) && isfinite(lo) && isfinite(abs_sum);
        } else {
            dd_ok = 0;
        }
    }
    if (exact_zero) return 0.0;
    if (!dd_ok) return directed;
    double gamma = gamma_n_dd(count);
    double err = (gamma == 0.0 || abs_sum == 0.0) ? 0.0 : nup64(gamma * abs_sum);
    if (upper) return nup64(nup64(hi + lo) + err);
    return ndn64(ndn64(hi + lo) - err);
}

/* bounds/concretize.rs:68-130 */
static float publish_lower(double v) {
    if (isnan(v) || v == -INFINITY) return -INFINITY;
    if (v == INFINITY) return INFINITY;
    if (v == 0.0) return (float)v;
    if (fabs(v) < (double)F32_MIN_POSITIVE) return signbit(v) ? -F32_MIN_POSITIVE : 0.0f;
    float p = NDN32((float)v);
    uint32_t mag = f2u(p) & 0x7fffffffu;
    if (mag != 0 && mag < f2u(F32_MIN_POSITIVE)) return signbit(v) ? -F32_MIN_POSITIVE : 0.0f;
    return p;
}
static float publish_upper(double v) {
    if (isnan(v) || v == INFINITY) return INFINITY;
    if (v == -INFINITY) return -INFINITY;
    if (v == 0.0) return (float)v;
    if (fabs(v) < (double)F32_MIN_POSITIVE) return signbit(v) ? -0.0f : F32_MIN_POSITIVE;
    float p = NUP32((float)v);
    uint32_t mag = f2u(p) & 0x7fffffffu;
    if (mag != 0 && mag < f2u(F32_MIN_POSITIVE)) return signbit(v) ? -0.0f : F32_MIN_POSITIVE;
    return p;
}
static inline int coef_nonneg(float v) { uint32_t b = f2u(v); return (b >> 31) == 0 || (b & 0x7fffffffu) == 0; }
static inline float max_abs_bits(float l, float u) {
    uint32_t a = f2u(l) & 0x7fffffffu, b = f2u(u) & 0x7fffffffu;
    if (a > 0x7f800000u || b > 0x7f800000u) return NAN;
    return u2f(a > b ? a : b);
}
static inline float nonneg_err_or_inf_f32(float v) {
    uint32_t b = f2u(v), mag = b & 0x7fffffffu;
    if ((mag >> 23) == 0xff || ((b >> 31) != 0 && mag != 0)) return INFINITY;
    return v;
}

/* ------------------------------------------------------------------ linear bounds carrier */
/* bounds/linear.rs:320-347 */
typedef struct {
    int rows, n;
    float *la, *ua, *lb, *ub;
    float *le, *ue; /* certified per-coefficient error, or NULL */
} lbounds;

static lbounds lb_alloc(int rows, int n, int with_err) {
    lbounds b;
    b.rows = rows; b.n = n;
    b.la = (float *)calloc((size_t)rows * n, 4);
    b.ua = (float *)calloc((size_t)rows * n, 4);
    b.lb = (float *)calloc(rows, 4);
    b.ub = (float *)calloc(rows, 4);
    b.le = with_err ? (float *)calloc((size_t)rows * n, 4) : NULL;
    b.ue = with_err ? (float *)calloc((size_t)rows * n, 4) : NULL;
    return b;
}
static void lb_free(lbounds *b) {
    free(b->la); free(b->ua); free(b->lb); free(b->ub); free(b->le); free(b->ue);
    memset(b, 0, sizeof(*b));
}
static lbounds lb_identity(int n) {
    lbounds b = lb_alloc(n, n, 0);
    for (int i = 0; i < n; ++i) { b.la[(size_t)i * n + i] = 1.0f; b.ua[(size_t)i * n + i] = 1.0f; }
    return b;
}

/* bounds/concretize.rs:374-489 (identical arithmetic to :717-880) */
/* The reference's plain-CROWN path carries a certified per-coefficient error matrix through every layer
 * (err' = cast error + gamma_n * S + err * |W|, layers/linear/crown_single.rs:2092-2103) and discharges it at
 * concretisation (bounds/concretize.rs:443-466).  The switch below turns the discharge off, for tests that need
 * to separate that error chain (which grows with the product of the layers' |W| norms) from the bound itself.
 * Default on: the reference's behaviour, the one the golden vectors pin. */
static int g_error_channel = 1;
void nyo_set_error_channel(int on) { g_error_channel = on ? 1 : 0; }

static void concretize_row(float lb, float ub, const float *in_l, const float *in_u, int n,
                           const float *la, const float *ua, const float *le, const float *ue,
                           float *tmp_c, float *tmp_v, float *out_l, float *out_u) {
    int lower_deg = (lb == -INFINITY), upper_deg = (ub == INFINITY);
    int lower_of = 0, upper_of = 0;
    if (!lower_deg || !upper_deg) {
        for (int j = 0; j < n; ++j) {
            if (!lower_deg && !coeff_safe(la[j])) lower_of = 1;
            if (!upper_deg && !coeff_safe(ua[j])) upper_of = 1;
            if ((lower_deg || lower_of) && (upper_deg || upper_of)) break;
        }
    }
    double lower64 = 0.0, upper64 = 0.0;
    if (lower_deg || lower_of) lower64 = -INFINITY;
    if (upper_deg || upper_of) upper64 = INFINITY;
    if (!((lower_deg || lower_of) && (upper_deg || upper_of))) {
        for (int j = 0; j < n; ++j) { tmp_c[j] = la[j]; tmp_v[j] = coef_nonneg(la[j]) ? in_l[j] : in_u[j]; }
        double sum_l = nyo_certified_affine_sum(lb, tmp_c, tmp_v, n, 0);
        for (int j = 0; j < n; ++j) { tmp_c[j] = ua[j]; tmp_v[j] = coef_nonneg(ua[j]) ? in_u[j] : in_l[j]; }
        double sum_u = nyo_certified_affine_sum(ub, tmp_c, tmp_v, n, 1);
        if (le && g_error_channel) {
            for (int j = 0; j < n; ++j) { tmp_c[j] = nonneg_err_or_inf_f32(le[j]); tmp_v[j] = max_abs_bits(in_l[j], in_u[j]); }
            double pen = nyo_certified_affine_sum(0.0f, tmp_c, tmp_v, n, 1);
            sum_l = ndn64(sum_l - pen);
        }
        if (ue && g_error_channel) {
            for (int j = 0; j < n; ++j) { tmp_c[j] = nonneg_err_or_inf_f32(ue[j]); tmp_v[j] = max_abs_bits(in_l[j], in_u[j]); }
            double pen = nyo_certified_affine_sum(0.0f, tmp_c, tmp_v, n, 1);
            sum_u = nup64(sum_u + pen);
        }
        if (!(lower_deg || lower_of)) lower64 = isnan(sum_l) ? -INFINITY : sum_l;
        if (!(upper_deg || upper_of)) upper64 = isnan(sum_u) ? INFINITY : sum_u;
    }
    float l = publish_lower(lower64), u = publish_upper(upper64);
    if (!isfinite(l) || !isfinite(u) || l > u) { l = -INFINITY; u = INFINITY; }
    *out_l = l; *out_u = u;
}

static void concretize(const lbounds *b, const float *in_l, const float *in_u, float *out_l, float *out_u) {
    float *tc = (float *)malloc(sizeof(float) * (size_t)(b->n > 0 ? b->n : 1));
    float *tv = (float *)malloc(sizeof(float) * (size_t)(b->n > 0 ? b->n : 1));
    for (int i = 0; i < b->rows; ++i) {
        size_t o = (size_t)i * b->n;
        concretize_row(b->lb[i], b->ub[i], in_l, in_u, b->n, b->la + o, b->ua + o,
                       b->le ? b->le + o : NULL, b->ue ? b->ue + o : NULL, tc, tv, out_l + i, out_u + i);
    }
    free(tc); free(tv);
}

/* ------------------------------------------------------------------ network access */
typedef struct { const float *W; const float *b; int n_in, n_out; const int32_t *g; /* conv geometry or NULL */ } lin_layer;
enum { G_IC, G_IH, G_IW, G_OC, G_OH, G_OW, G_KH, G_KW, G_SH, G_SW, G_PH, G_PW };
static const int32_t *layer_geom(const nyo_net *net, int k) {
    if (!net->conv_geom) return NULL;
    const int32_t *g = net->conv_geom + 12 * (size_t)k;
    return g[G_OC] > 0 ? g : NULL;
}
static int skip_of(const nyo_net *net, int k) { return net->skip_from ? net->skip_from[k] : -1; }
static int net_has_skip(const nyo_net *net) {
    for (int k = 0; k < net->n_linear; ++k) if (skip_of(net, k) >= 0) return 1;
    return 0;
}
static int net_has_conv(const nyo_net *net) {
    for (int k = 0; k < net->n_linear; ++k) if (layer_geom(net, k)) return 1;
    return 0;
}

static lin_layer net_layer(const nyo_net *net, int k) {
    size_t wo = 0, bo = 0;
    for (int i = 0; i < k; ++i) {
        const int32_t *g = layer_geom(net, i);
        wo += g ? (size_t)g[G_OC] * g[G_IC] * g[G_KH] * g[G_KW] : (size_t)net->dims[i] * net->dims[i + 1];
        if (net->has_bias[i]) bo += g ? (size_t)g[G_OC] : (size_t)net->dims[i + 1];
    }
    lin_layer l;
    l.W = net->wflat + wo;
    l.b = net->has_bias[k] ? net->bflat + bo : NULL;
    l.n_in = net->dims[k]; l.n_out = net->dims[k + 1];
    l.g = layer_geom(net, k);
    return l;
}
static inline int relu_after(const nyo_net *net, int k) {
    if (k >= net->n_linear - 1) return 0;
    return net->relu_after ? (net->relu_after[k] != 0) : 1;
}
static size_t pre_offset(const nyo_net *net, int k) { /* offset of Linear_k's output block */
    size_t o = 0;
    for (int i = 0; i < k; ++i) o += (size_t)net->dims[i + 1];
    return o;
}

/* ------------------------------------------------------------------ IBP */
/* layers/convolution/conv2d/bound.rs:86-268 with ops_ibp_fwd.rs:131-395: the interval convolution
 * lower = conv(l, W+) + conv(u, W-) + b, upper = conv(u, W+) + conv(l, W-) + b over the im2col taps
 * (row = output position, column = (ic, ki, kj); taps outside the input contribute zero).  The reference runs
 * the four products as fp32 GEMMs; here they are accumulated in binary64 and cast outward like the Linear
 * layer's, which encloses the reference's values (they differ by fp32 summation noise, ~1e-7 relative). */
static void conv_ibp(const lin_layer *L, const float *xl, const float *xu, float *yl, float *yu) {
    const int32_t *g = L->g;
    const int ic = g[G_IC], ih = g[G_IH], iw = g[G_IW], oc = g[G_OC], oh = g[G_OH], ow = g[G_OW];
    const int kh = g[G_KH], kw = g[G_KW], sh = g[G_SH], sw = g[G_SW], ph = g[G_PH], pw = g[G_PW];
    for (int co = 0; co < oc; ++co)
        for (int oy = 0; oy < oh; ++oy)
            for (int ox = 0; ox < ow; ++ox) {
                double lo = 0.0, hi = 0.0;
                for (int ci = 0; ci < ic; ++ci)
                    for (int ky = 0; ky < kh; ++ky) {
                        int iy = oy * sh + ky - ph;
                        if (iy < 0 || iy >= ih) continue;
                        for (int kx = 0; kx < kw; ++kx) {
                            int ix = ox * sw + kx - pw;
                            if (ix < 0 || ix >= iw) continue;
                            float w = L->W[(((size_t)co * ic + ci) * kh + ky) * kw + kx];
                            double wp = (double)fmaxf(w, 0.0f), wn = (double)fminf(w, 0.0f);
                            if (isnan(w)) { wp = NAN; wn = NAN; }
                            size_t i = ((size_t)ci * ih + iy) * iw + ix;
                            lo += wp * (double)xl[i] + wn * (double)xu[i];
                            hi += wp * (double)xu[i] + wn * (double)xl[i];
                        }
                    }
                if (L->b) { lo += (double)L->b[co]; hi += (double)L->b[co]; }
                float l = NDN32((float)lo), u = NUP32((float)hi);
                if (isnan(l) || isnan(u) || l > u) { l = -INFINITY; u = INFINITY; }
                size_t o = ((size_t)co * oh + oy) * ow + ox;
                yl[o] = l; yu[o] = u;
            }
}

/* layers/linear/ibp.rs:464-523: W+ l + W- u + b accumulated in binary64, cast outward. */
static void linear_ibp(const lin_layer *L, const float *xl, const float *xu, float *yl, float *yu) {
    if (L->g) { conv_ibp(L, xl, xu, yl, yu); return; }
    for (int o = 0; o < L->n_out; ++o) {
        const float *w = L->W + (size_t)o * L->n_in;
        double pl = 0.0, nu = 0.0, pu = 0.0, nl = 0.0;
        for (int i = 0; i < L->n_in; ++i) {
            double wp = (double)fmaxf(w[i], 0.0f), wn = (double)fminf(w[i], 0.0f);
            if (isnan(w[i])) { wp = NAN; wn = NAN; }
            pl += wp * (double)xl[i]; nu += wn * (double)xu[i];
            pu += wp * (double)xu[i]; nl += wn * (double)xl[i];
        }
        double lo = pl + nu, hi = pu + nl;
        if (L->b) { lo += (double)L->b[o]; hi += (double)L->b[o]; }
        float l = NDN32((float)lo), u = NUP32((float)hi);
        /* BoundedTensor::new_repaired(Conservative): NaN or inverted -> [-inf, +inf] */
        if (isnan(l) || isnan(u) || l > u) { l = -INFINITY; u = INFINITY; }
        yl[o] = l; yu[o] = u;
    }
}
/* layers/activations/relu/ibp.rs:14-18 (NaN-propagating max) */
static inline float nanmax(float a, float b) { return (isnan(a) || isnan(b)) ? NAN : (a > b ? a : b); }
static inline float nanmin(float a, float b) { return (isnan(a) || isnan(b)) ? NAN : (a < b ? a : b); }

int nyo_ibp_forward(const nyo_net *net, const float *in_lo, const float *in_hi, float *pre_lo, float *pre_hi) {
    int L = net->n_linear;
    int maxn = 0;
    for (int k = 0; k <= L; ++k) if (net->dims[k] > maxn) maxn = net->dims[k];
    float *zl = (float *)malloc(4 * (size_t)maxn), *zu = (float *)malloc(4 * (size_t)maxn);
    memcpy(zl, in_lo, 4 * (size_t)net->dims[0]); memcpy(zu, in_hi, 4 * (size_t)net->dims[0]);
    for (int k = 0; k < L; ++k) {
        lin_layer Lk = net_layer(net, k);
        size_t o = pre_offset(net, k);
        linear_ibp(&Lk, zl, zu, pre_lo + o, pre_hi + o);
        if (skip_of(net, k) >= 0) {  /* identity branch: + relu(pre_j), whose interval is relu of the stored bounds */
            size_t so = pre_offset(net, skip_of(net, k));
            for (int j = 0; j < Lk.n_out; ++j) {
                pre_lo[o + j] = f64_to_f32_down_ns((double)pre_lo[o + j] + (double)nanmax(pre_lo[so + j], 0.0f));
                pre_hi[o + j] = f64_to_f32_up_ns((double)pre_hi[o + j] + (double)nanmax(pre_hi[so + j], 0.0f));
            }
        }
        int act = relu_after(net, k);
        for (int j = 0; j < Lk.n_out; ++j) {
            zl[j] = act ? nanmax(pre_lo[o + j], 0.0f) : pre_lo[o + j];
            zu[j] = act ? nanmax(pre_hi[o + j], 0.0f) : pre_hi[o + j];
        }
    }
    free(zl); free(zu);
    return 0;
}

/* ------------------------------------------------------------------ linear backward */
/* layers/linear/crown_single.rs:124-135 */
static double gamma_n_f64(size_t n) {
    double d = (double)n * ldexp(1.0, -53);
    return d >= 1.0 ? INFINITY : d / (1.0 - d);
}

/* layers/linear/crown_single.rs:1931-2226.  in: rows x n_out; returns rows x n_in with
 * certified error matrices. */
static lbounds linear_backward(const lin_layer *L, const lbounds *in) {
    int rows = in->rows, K = L->n_out, N = L->n_in;
    lbounds out = lb_alloc(rows, N, 1);
    /* contraction length: out_features for a Linear layer, oc*kh*kw for a Conv2d (bound.rs:633) */
    double gamma = gamma_n_f64(L->g ? (size_t)L->g[G_OC] * L->g[G_KH] * L->g[G_KW] : (size_t)K);
    double *a64 = (double *)malloc(sizeof(double) * (size_t)N);
    double *s64 = (double *)malloc(sizeof(double) * (size_t)N);
    double *p64 = (double *)malloc(sizeof(double) * (size_t)N);
    for (int side = 0; side < 2; ++side) {
        const float *A = side ? in->ua : in->la;
        const float *E = side ? in->ue : in->le;
        const float *Bin = side ? in->ub : in->lb;
        float *Ao = side ? out.ua : out.la, *Eo = side ? out.ue : out.le, *Bo = side ? out.ub : out.lb;
        for (int i = 0; i < rows; ++i) {
            const float *a = A + (size_t)i * K;
            for (int j = 0; j < N; ++j) { a64[j] = 0.0; s64[j] = 0.0; p64[j] = 0.0; }
            if (L->g) {
                /* Conv2d: transposed convolution of the row (layers/convolution/conv2d/bound.rs:601-900,
                 * conv2d_transpose_backward_coeff_f64, ops_transpose_gemm.rs): the coefficient of input element
                 * (ci, iy, ix) collects a[(co, oy, ox)] * W[co, ci, ky, kx] over the taps with iy = oy*sh + ky - ph,
                 * ix = ox*sw + kx - pw; binary64 accumulation with the magnitude sum, the incoming error through
                 * |W| (bound.rs:860-1010). */
                const int32_t *g = L->g;
                const int ic = g[G_IC], ih = g[G_IH], iw = g[G_IW], oc = g[G_OC], oh = g[G_OH], ow = g[G_OW];
                const int kh = g[G_KH], kw = g[G_KW], sh = g[G_SH], sw = g[G_SW], ph = g[G_PH], pw = g[G_PW];
                const float *e = E ? E + (size_t)i * K : NULL;
                for (int co = 0; co < oc; ++co)
                    for (int oy = 0; oy < oh; ++oy)
                        for (int ox = 0; ox < ow; ++ox) {
                            size_t k = ((size_t)co * oh + oy) * ow + ox;
                            double ak = (double)a[k], ek = e ? nonneg_err_or_inf(e[k]) : 0.0;
                            if (ak == 0.0 && ek == 0.0) continue;
                            double aak = fabs(ak);
                            for (int ci = 0; ci < ic; ++ci)
                                for (int ky = 0; ky < kh; ++ky) {
                                    int iy = oy * sh + ky - ph;
                                    if (iy < 0 || iy >= ih) continue;
                                    for (int kx = 0; kx < kw; ++kx) {
                                        int ix = ox * sw + kx - pw;
                                        if (ix < 0 || ix >= iw) continue;
                                        double w = (double)L->W[(((size_t)co * ic + ci) * kh + ky) * kw + kx];
                                        size_t j = ((size_t)ci * ih + iy) * iw + ix;
                                        if (isnan(ak)) a64[j] = NAN;
                                        else if (ak != 0.0) { a64[j] += ak * w; s64[j] += aak * fabs(w); }
                                        if (ek != 0.0 && w != 0.0) p64[j] = add_f64_up(p64[j], ek * fabs(w));
                                    }
                                }
                        }
            } else {
            /* aw_f64_with_abssum (:170): exact products, binary64 accumulation */
            for (int k = 0; k < K; ++k) {
                double ak = (double)a[k];
                const float *w = L->W + (size_t)k * N;
                if (ak != 0.0) {
                    double aak = fabs(ak);
                    for (int j = 0; j < N; ++j) { a64[j] += ak * (double)w[j]; s64[j] += aak * fabs((double)w[j]); }
                } else if (isnan(ak)) {
                    for (int j = 0; j < N; ++j) { a64[j] = NAN; }
                }
            }
            /* incoming_error_product (:1238): upward-directed sum of err * |W| published as f32 */
            if (E) {
                const float *e = E + (size_t)i * K;
                for (int k = 0; k < K; ++k) {
                    double ek = nonneg_err_or_inf(e[k]);
                    if (ek == 0.0) continue;
                    const float *w = L->W + (size_t)k * N;
                    for (int j = 0; j < N; ++j) {
                        double aw = fabs((double)w[j]);
                        if (aw != 0.0) p64[j] = add_f64_up(p64[j], ek * aw);
                    }
                }
            }
            }
            int nonfinite = 0;
            for (int j = 0; j < N; ++j) {
                float v = (float)a64[j];
                double cast_err = fabs(a64[j] - (double)v);
                double prop = E ? (double)publish_error_up_normal(p64[j]) : 0.0;
                float err = publish_error_up_normal(cast_err + gamma * s64[j] + prop);
                if (coeff_safe(v) && isfinite(err)) { Ao[(size_t)i * N + j] = v; Eo[(size_t)i * N + j] = err; }
                else nonfinite = 1;
            }
            /* bias: accumulate_bias_f64 (bias.rs:238-255) + error fold (:2142-2166) + finalize */
            float bnew = Bin[i];
            if (L->b) {
                double acc = 0.0;
                /* a Conv2d bias is per channel: element k belongs to channel k / (oh*ow)
                 * (compute_conv_bias_f64, layers/crown_helpers.rs:748-800) */
                const int plane = L->g ? L->g[G_OH] * L->g[G_OW] : 1;
                for (int k = 0; k < K; ++k) {
                    double t = (double)a[k] * (double)L->b[k / plane];
                    acc = side ? add_f64_up(acc, t) : add_f64_down(acc, t);
                }
                if (E) {
                    const float *e = E + (size_t)i * K;
                    double ee = 0.0;
                    for (int k = 0; k < K; ++k) {
                        double ba = fabs((double)L->b[k / plane]);
                        if (ba == 0.0) continue;
                        ee = add_f64_up(ee, nonneg_err_or_inf(e[k]) * ba);
                    }
                    acc = side ? add_f64_up(acc, ee) : add_f64_down(acc, -ee);
                }
                bnew = side ? f64_to_f32_up_ns(add_f64_up((double)Bin[i], acc))
                            : f64_to_f32_down_ns(add_f64_down((double)Bin[i], acc));
            }
            if (nonfinite) {
                for (int j = 0; j < N; ++j) { Ao[(size_t)i * N + j] = 0.0f; Eo[(size_t)i * N + j] = 0.0f; }
                bnew = side ? INFINITY : -INFINITY;
            }
            Bo[i] = bnew;
        }
    }
    free(a64); free(s64); free(p64);
    return out;
}

/* ------------------------------------------------------------------ ReLU relaxations */
typedef struct { float ls, li, us, ui; } relax_t; /* lower slope/intercept, upper slope/intercept */

/* activations/relu/mod.rs:105-132 + activations/mod.rs:99-121 */
static relax_t relu_relaxation(float l, float u) {
    relax_t r;
    if (isnan(l) || isnan(u)) { r.ls = 0; r.li = -INFINITY; r.us = 0; r.ui = INFINITY; return r; }
    if (l >= 0.0f) { r.ls = 1; r.li = 0; r.us = 1; r.ui = 0; return r; }
    if (u <= 0.0f) { r.ls = 0; r.li = 0; r.us = 0; r.ui = 0; return r; }
    if (isinf(l) && isinf(u)) { r.ls = 0; r.li = 0; r.us = 0; r.ui = INFINITY; return r; }
    if (isinf(u)) { r.ls = 1; r.li = 0; r.us = 1; r.ui = -l; return r; }
    if (isinf(l)) { r.ls = 0; r.li = 0; r.us = 0; r.ui = u; return r; }
    double width = (double)u - (double)l;
    float lam = NUP32((float)((double)u / width));
    float icp = NUP32((float)(-(double)lam * (double)l));
    r.ls = (u > -l) ? 1.0f : 0.0f; r.li = 0.0f; r.us = lam; r.ui = icp;
    return r;
}

/* layers/common/crown_dense.rs:41-286 with compose.rs:84-185 (default exact-zero-slope gate off) */
static lbounds relu_backward_crown(const lbounds *in, const float *pl, const float *pu) {
    int rows = in->rows, n = in->n;
    lbounds out = lb_alloc(rows, n, 1);
    relax_t *rx = (relax_t *)malloc(sizeof(relax_t) * (size_t)n);
    for (int i = 0; i < n; ++i) rx[i] = relu_relaxation(pl[i], pu[i]);
    for (int j = 0; j < rows; ++j) {
        double lb64 = (double)in->lb[j], ub64 = (double)in->ub[j];
        double lberr = 0.0, uberr = 0.0;
        int lnf = 0, unf = 0;
        for (int i = 0; i < n; ++i) {
            size_t o = (size_t)j * n + i;
            float la = in->la[o], ua = in->ua[o];
            const relax_t *r = &rx[i];
            /* compose_lower */
            float lc = 0.0f; double lslope = 0.0;
            if (la > 0.0f) {
                float p = la * r->ls; lslope = (double)r->ls;
                lc = isfinite(p) ? NDN32(p) : 0.0f; lnf |= !isfinite(p);
                lb64 += (double)la * (double)r->li;
            } else if (la < 0.0f) {
                float p = la * r->us; lslope = (double)r->us;
                lc = isfinite(p) ? NDN32(p) : 0.0f; lnf |= !isfinite(p);
                lb64 += (double)la * (double)r->ui;
            }
            out.la[o] = lc;
            /* compose_upper */
            float uc = 0.0f; double uslope = 0.0;
            if (ua > 0.0f) {
                float p = ua * r->us; uslope = (double)r->us;
                uc = isfinite(p) ? NUP32(p) : 0.0f; unf |= !isfinite(p);
                ub64 += (double)ua * (double)r->ui;
            } else if (ua < 0.0f) {
                float p = ua * r->ls; uslope = (double)r->ls;
                uc = isfinite(p) ? NUP32(p) : 0.0f; unf |= !isfinite(p);
                ub64 += (double)ua * (double)r->li;
            }
            out.ua[o] = uc;
            double slope_sum = (double)(fabsf(r->ls) + fabsf(r->us));
            double int_sum = (double)(fabsf(r->li) + fabsf(r->ui));
            {
                double gap = (la != 0.0f) ? fabs((double)la * lslope - (double)lc) : 0.0;
                double ea = in->le ? (double)in->le[o] : 0.0;
                if (gap != 0.0 || ea != 0.0) {
                    double sc, ic;
                    if (fabs((double)la) > ea) { sc = fabs(lslope); ic = (la > 0.0f) ? (double)fabsf(r->li) : (double)fabsf(r->ui); }
                    else { sc = slope_sum; ic = int_sum; }
                    out.le[o] = NUP32((float)(ea * sc + gap));
                    if (ea != 0.0) lberr += ea * ic;
                }
            }
            {
                double gap = (ua != 0.0f) ? fabs((double)ua * uslope - (double)uc) : 0.0;
                double ea = in->ue ? (double)in->ue[o] : 0.0;
                if (gap != 0.0 || ea != 0.0) {
                    double sc, ic;
                    if (fabs((double)ua) > ea) { sc = fabs(uslope); ic = (ua > 0.0f) ? (double)fabsf(r->ui) : (double)fabsf(r->li); }
                    else { sc = slope_sum; ic = int_sum; }
                    out.ue[o] = NUP32((float)(ea * sc + gap));
                    if (ea != 0.0) uberr += ea * ic;
                }
            }
        }
        if (g_error_channel) { lb64 -= lberr; ub64 += uberr; }
        out.lb[j] = (lb64 == 0.0) ? 0.0f : NDN32((float)lb64);
        out.ub[j] = (ub64 == 0.0) ? 0.0f : NUP32((float)ub64);
        if (lnf) { for (int i = 0; i < n; ++i) { out.la[(size_t)j * n + i] = 0; out.le[(size_t)j * n + i] = 0; } out.lb[j] = -INFINITY; }
        if (unf) { for (int i = 0; i < n; ++i) { out.ua[(size_t)j * n + i] = 0; out.ue[(size_t)j * n + i] = 0; } out.ub[j] = INFINITY; }
    }
    free(rx);
    return out;
}

/* beta_crown/engine/backward/relu_backward.rs:33-185.  split[i]: 0 none, +1 active, -1 inactive;
 * sbeta[i]: signed beta (beta * sign) or 0; has_sb[i] marks neurons that carry a beta entry.
 * The result carries no error matrices (LinearBounds::new_or_conservative). */
#define RELU_RELAX_MIN_WIDTH 1e-8f
static lbounds relu_backward_beta(const lbounds *in, const float *pl, const float *pu,
                                  const signed char *split, const float *sbeta, const unsigned char *has_sb,
                                  const float *alpha, const float *alpha_up) {
    /* alpha_up: separate lower slope for the upper bound's negative coefficients (the dual alpha of
     * activations/relu/mod.rs:570-1128); NULL = the same slope as the lower path. */
    int rows = in->rows, n = in->n;
    lbounds out = lb_alloc(rows, n, 0);
    double *lb64 = (double *)malloc(sizeof(double) * (size_t)rows);
    double *ub64 = (double *)malloc(sizeof(double) * (size_t)rows);
    for (int i = 0; i < rows; ++i) { lb64[i] = (double)in->lb[i]; ub64[i] = (double)in->ub[i]; }
    int nonfinite = 0;
    for (int j = 0; j < n; ++j) {
        float l = pl[j], u = pu[j];
        float ls, li, us, ui;
        int free_slope = 0;
        if (split && split[j] != 0) {
            if (split[j] > 0) { ls = 1; li = 0; us = 1; ui = 0; } else { ls = 0; li = 0; us = 0; ui = 0; }
        } else if (isnan(l) || isnan(u)) { ls = 0; li = -INFINITY; us = 0; ui = INFINITY; }
        else if (l >= 0.0f) { ls = 1; li = 0; us = 1; ui = 0; }
        else if (u <= 0.0f) { ls = 0; li = 0; us = 0; ui = 0; }
        else if (isinf(l) && isinf(u)) { ls = 0; li = 0; us = 0; ui = INFINITY; }
        else if (isinf(u)) { ls = 1; li = 0; us = 1; ui = -l; }
        else if (isinf(l)) { ls = 0; li = 0; us = 0; ui = u; }
        else {
            float width = fmaxf(u - l, RELU_RELAX_MIN_WIDTH);
            us = u / width; ui = -l * u / width;
            ls = alpha ? alpha[j] : ((u > -l) ? 1.0f : 0.0f); li = 0.0f;
            free_slope = 1;
        }
        float ls_up = (free_slope && alpha_up) ? alpha_up[j] : ls;
        for (int i = 0; i < rows; ++i) {
            size_t o = (size_t)i * n + j;
            float la = in->la[o], ua = in->ua[o];
            if (la > 0.0f) {
                float p = la * ls;
                if (isfinite(p)) out.la[o] = NDN32(p); else { nonfinite = 1; out.la[o] = 0; }
                lb64[i] += (double)la * (double)li;
            } else if (la < 0.0f) {
                float p = la * us;
                if (isfinite(p)) out.la[o] = NDN32(p); else { nonfinite = 1; out.la[o] = 0; }
                lb64[i] += (double)la * (double)ui;
            } else out.la[o] = 0.0f;
            if (ua > 0.0f) {
                float p = ua * us;
                if (isfinite(p)) out.ua[o] = NUP32(p); else { nonfinite = 1; out.ua[o] = 0; }
                ub64[i] += (double)ua * (double)ui;
            } else if (ua < 0.0f) {
                float p = ua * ls_up;
                if (isfinite(p)) out.ua[o] = NUP32(p); else { nonfinite = 1; out.ua[o] = 0; }
                ub64[i] += (double)ua * (double)li;
            } else out.ua[o] = 0.0f;
        }
        if (has_sb && has_sb[j] && isfinite(sbeta[j])) {
            for (int i = 0; i < rows; ++i) { out.la[(size_t)i * n + j] -= sbeta[j]; out.ua[(size_t)i * n + j] += sbeta[j]; }
        }
    }
    if (nonfinite) { /* LinearBounds::conservative: zero coefficients, bias -inf/+inf */
        memset(out.la, 0, 4 * (size_t)rows * n); memset(out.ua, 0, 4 * (size_t)rows * n);
        for (int i = 0; i < rows; ++i) { out.lb[i] = -INFINITY; out.ub[i] = INFINITY; }
    } else {
        for (int i = 0; i < rows; ++i) { out.lb[i] = NDN32((float)lb64[i]); out.ub[i] = NUP32((float)ub64[i]); }
    }
    free(lb64); free(ub64);
    return out;
}

/* ------------------------------------------------------------------ plain CROWN pipeline */
/* Backward from `seed` (rows x dims[top+1]) through Linear_top, ReLU_{top-1}, ..., Linear_0,
 * then concretize on the input box.  pre_* hold the pre-activation bounds used by the ReLUs. */
static void crown_backward_concretize(const nyo_net *net, int top, lbounds seed, const float *pre_lo,
                                      const float *pre_hi, const float *in_lo, const float *in_hi,
                                      float *out_l, float *out_u) {
    lbounds cur = seed;
    for (int k = top; k >= 0; --k) {
        lin_layer Lk = net_layer(net, k);
        lbounds nxt = linear_backward(&Lk, &cur);
        lb_free(&cur); cur = nxt;
        if (k > 0 && relu_after(net, k - 1)) {
            size_t o = pre_offset(net, k - 1);
            lbounds r = relu_backward_crown(&cur, pre_lo + o, pre_hi + o);
            lb_free(&cur); cur = r;
        }
    }
    concretize(&cur, in_lo, in_hi, out_l, out_u);
    lb_free(&cur);
}

/* ny-tensor bounded_tensor/core/numeric.rs:316-360: intersection with union fallback; returns 0
 * (and leaves a untouched) if any endpoint is NaN. */
static int intersect_per_element(float *al, float *au, const float *bl, const float *bu, int n) {
    for (int i = 0; i < n; ++i) if (isnan(al[i]) || isnan(au[i]) || isnan(bl[i]) || isnan(bu[i])) return 0;
    for (int i = 0; i < n; ++i) {
        float tl = fmaxf(al[i], bl[i]), tu = fminf(au[i], bu[i]);
        if (tl <= tu) { al[i] = tl; au[i] = tu; }
        else { al[i] = fminf(al[i], bl[i]); au[i] = fmaxf(au[i], bu[i]); }
    }
    return 1;
}

/* Pre-activation clamps of a ReLU-split domain on layer k's tightened bounds (constraints/lookups.rs:138-185):
 * active l = max(l, 0), inactive u = min(u, 0).  Returns 1 when a clamp empties an interval (the domain is infeasible). */
static int clamp_splits(const nyo_split *splits, int n_splits, int k, float *l, float *u) {
    int empty = 0;
    for (int s = 0; s < n_splits; ++s) if (splits[s].relu == k) {
        int j = splits[s].neuron;
        if (splits[s].sign > 0) { if (!isnan(l[j])) l[j] = fmaxf(l[j], 0.0f); }
        else { if (!isnan(u[j])) u[j] = fminf(u[j], 0.0f); }
        if (l[j] > u[j]) empty = 1;
    }
    return empty;
}

static int crown_impl(const nyo_net *net, const float *in_lo, const float *in_hi, const nyo_split *splits, int n_splits,
                      float *out_lo, float *out_hi, float *inter_lo, float *inter_hi);

int nyo_crown(const nyo_net *net, const float *in_lo, const float *in_hi, float *out_lo, float *out_hi,
              float *inter_lo, float *inter_hi) {
    return crown_impl(net, in_lo, in_hi, NULL, 0, out_lo, out_hi, inter_lo, inter_hi);
}

/* The same pipeline for a ReLU-split domain (the CROWN-IBP collection of network/ibp/crown_ibp.rs:32-420 run under the
 * domain's clamps): the interval pass is the constrained forward pass without inherited bounds, every layer's tightened
 * bound is clamped before its relaxation is taken, split multipliers stay at zero.  Returns 1 for an infeasible
 * domain (outputs untouched), 0 otherwise. */
int nyo_crown_split(const nyo_net *net, const float *in_lo, const float *in_hi, const nyo_split *splits, int n_splits,
                    float *out_lo, float *out_hi, float *inter_lo, float *inter_hi) {
    return crown_impl(net, in_lo, in_hi, splits, n_splits, out_lo, out_hi, inter_lo, inter_hi);
}

static int crown_impl(const nyo_net *net, const float *in_lo, const float *in_hi, const nyo_split *splits, int n_splits,
                      float *out_lo, float *out_hi, float *inter_lo, float *inter_hi) {
    if (net_has_skip(net)) return -2;
    int L = net->n_linear;
    size_t total = pre_offset(net, L);
    float *ibp_l = (float *)malloc(4 * total), *ibp_u = (float *)malloc(4 * total);
    float *t_l = (float *)malloc(4 * total), *t_u = (float *)malloc(4 * total);
    if (n_splits > 0) {
        float *no_l = (float *)calloc(total, 4), *no_u = (float *)calloc(total, 4);   /* no inherited bounds */
        for (size_t i = 0; i < total; ++i) { no_l[i] = -INFINITY; no_u[i] = INFINITY; }
        int bad = nyo_domain_bounds(net, in_lo, in_hi, no_l, no_u, splits, n_splits, 1, ibp_l, ibp_u);
        free(no_l); free(no_u);
        if (bad) { free(ibp_l); free(ibp_u); free(t_l); free(t_u); return 1; }
    } else nyo_ibp_forward(net, in_lo, in_hi, ibp_l, ibp_u);
    int infeasible = 0;
    int maxn = 0;
    for (int k = 0; k <= L; ++k) if (net->dims[k] > maxn) maxn = net->dims[k];
    float *zl = (float *)malloc(4 * (size_t)maxn), *zu = (float *)malloc(4 * (size_t)maxn);
    float *fl = (float *)malloc(4 * (size_t)maxn), *fu = (float *)malloc(4 * (size_t)maxn);
    float *cl = (float *)malloc(4 * (size_t)maxn), *cu = (float *)malloc(4 * (size_t)maxn);
    /* CROWN-IBP collection (network/ibp/crown_ibp.rs:32-420).  In the reference's layer list
     * [Linear, ReLU, Linear, ...] every Linear output needs a partial CROWN pass (its successor is a
     * ReLU, or it is the last layer); ReLU outputs take the forward shortcut and are recomputed from
     * the tightened pre-activation when the next Linear needs them. */
    for (int k = 0; k < L; ++k) {
        lin_layer Lk = net_layer(net, k);
        size_t o = pre_offset(net, k);
        int n = Lk.n_out;
        const float *il = ibp_l + o, *iu = ibp_u + o;
        int all_stable = 1;
        for (int j = 0; j < n; ++j) if (!(il[j] >= 0.0f || iu[j] <= 0.0f)) { all_stable = 0; break; }
        if (k < L - 1 && relu_after(net, k) && all_stable) { /* ReLU-stable skip (:113-140) */
            memcpy(t_l + o, il, 4 * (size_t)n); memcpy(t_u + o, iu, 4 * (size_t)n);
            infeasible |= clamp_splits(splits, n_splits, k, t_l + o, t_u + o);
            continue;
        }
        /* crown_partial.rs:166-182: forward bound of this layer from the tightened prior bounds */
        if (k == 0) { memcpy(zl, in_lo, 4 * (size_t)Lk.n_in); memcpy(zu, in_hi, 4 * (size_t)Lk.n_in); }
        else {
            /* the ReLU output bound stored by the collection: relu IBP of the tightened
             * pre-activation intersected with the plain IBP ReLU output (crown_ibp_forward.rs:25-100) */
            size_t po = pre_offset(net, k - 1);
            int act = relu_after(net, k - 1);
            for (int j = 0; j < Lk.n_in; ++j) {
                zl[j] = act ? nanmax(t_l[po + j], 0.0f) : t_l[po + j]; zu[j] = act ? nanmax(t_u[po + j], 0.0f) : t_u[po + j];
                fl[j] = act ? nanmax(ibp_l[po + j], 0.0f) : ibp_l[po + j]; fu[j] = act ? nanmax(ibp_u[po + j], 0.0f) : ibp_u[po + j];
            }
            float *tmpl = (float *)malloc(4 * (size_t)Lk.n_in), *tmpu = (float *)malloc(4 * (size_t)Lk.n_in);
            memcpy(tmpl, fl, 4 * (size_t)Lk.n_in); memcpy(tmpu, fu, 4 * (size_t)Lk.n_in);
            if (intersect_per_element(tmpl, tmpu, zl, zu, Lk.n_in)) { memcpy(zl, tmpl, 4 * (size_t)Lk.n_in); memcpy(zu, tmpu, 4 * (size_t)Lk.n_in); }
            else { memcpy(zl, fl, 4 * (size_t)Lk.n_in); memcpy(zu, fu, 4 * (size_t)Lk.n_in); }
            free(tmpl); free(tmpu);
        }
        linear_ibp(&Lk, zl, zu, fl, fu);
        if (k < L - 1 && !relu_after(net, k)) {
            /* Linear feeding a Linear: the successor's backward step is exact and does not read the
             * interval, so the collection takes the forward shortcut (ibp/helpers.rs:99-107,
             * crown_ibp_forward.rs:25-100): forward bound from the tightened input, intersected with IBP. */
            memcpy(t_l + o, il, 4 * (size_t)n); memcpy(t_u + o, iu, 4 * (size_t)n);
            intersect_per_element(t_l + o, t_u + o, fl, fu, n);
            continue;
        }
        /* sparse_merge.rs:118-146: when >= 90% of the neurons are stable only the unstable rows
         * are propagated; stable rows keep the forward bound. */
        int n_unst = 0;
        for (int j = 0; j < n; ++j) if (fl[j] < 0.0f && fu[j] > 0.0f) ++n_unst;
        int sparse = 0;
        if (n_unst > 0) {
            float stable_frac = 1.0f - ((float)n_unst / (float)n);
            if (!(stable_frac < 0.9f)) sparse = 1;
        }
        lbounds seed;
        int *rowmap = NULL;
        if (sparse) {
            seed = lb_alloc(n_unst, n, 0);
            rowmap = (int *)malloc(sizeof(int) * (size_t)n_unst);
            int r = 0;
            for (int j = 0; j < n; ++j) if (fl[j] < 0.0f && fu[j] > 0.0f) {
                seed.la[(size_t)r * n + j] = 1.0f; seed.ua[(size_t)r * n + j] = 1.0f; rowmap[r++] = j;
            }
        } else seed = lb_identity(n);
        int rows = seed.rows;
        float *rl = (float *)malloc(4 * (size_t)rows), *ru = (float *)malloc(4 * (size_t)rows);
        crown_backward_concretize(net, k, seed, t_l, t_u, in_lo, in_hi, rl, ru);
        if (sparse) {
            memcpy(cl, fl, 4 * (size_t)n); memcpy(cu, fu, 4 * (size_t)n);
            for (int r = 0; r < rows; ++r) { cl[rowmap[r]] = rl[r]; cu[rowmap[r]] = ru[r]; }
            free(rowmap);
        } else { memcpy(cl, rl, 4 * (size_t)n); memcpy(cu, ru, 4 * (size_t)n); }
        free(rl); free(ru);
        /* crown_ibp.rs:186-215: intersect the plain IBP bound with the CROWN bound */
        memcpy(t_l + o, il, 4 * (size_t)n); memcpy(t_u + o, iu, 4 * (size_t)n);
        intersect_per_element(t_l + o, t_u + o, cl, cu, n);
        if (k < L - 1) infeasible |= clamp_splits(splits, n_splits, k, t_l + o, t_u + o);
    }
    if (infeasible) {
        free(ibp_l); free(ibp_u); free(t_l); free(t_u); free(zl); free(zu); free(fl); free(fu); free(cl); free(cu);
        return 1;
    }
    /* final backward (crown.rs:262-...) + tighten (crown/tighten.rs:126-190) */
    {
        int n = net->dims[L];
        lbounds seed = lb_identity(n);
        crown_backward_concretize(net, L - 1, seed, t_l, t_u, in_lo, in_hi, out_lo, out_hi);
        size_t o = pre_offset(net, L - 1);
        int has_nan = 0;
        for (int j = 0; j < n; ++j) if (isnan(out_lo[j]) || isnan(out_hi[j])) has_nan = 1;
        if (has_nan) { memcpy(out_lo, t_l + o, 4 * (size_t)n); memcpy(out_hi, t_u + o, 4 * (size_t)n); }
        else intersect_per_element(out_lo, out_hi, t_l + o, t_u + o, n);
    }
    if (inter_lo) memcpy(inter_lo, t_l, 4 * total);
    if (inter_hi) memcpy(inter_hi, t_u, 4 * total);
    free(ibp_l); free(ibp_u); free(t_l); free(t_u); free(zl); free(zu); free(fl); free(fu); free(cl); free(cu);
    return 0;
}

/* ------------------------------------------------------------------ beta-CROWN */
/* beta_crown/engine/optimization/bound_compute.rs:90-167: identity at the output, backward through
 * every layer with the alpha/beta ReLU rule, concretize_sound on the input box. */
int nyo_beta_crown_bound(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                         const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                         float *out_lo, float *out_hi) {
    return nyo_beta_crown_bound_dual(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, NULL, out_lo, out_hi);
}

int nyo_beta_crown_bound_dual(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                              const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                              const float *alpha_up, float *out_lo, float *out_hi) {
    int L = net->n_linear;
    lbounds cur = lb_identity(net->dims[L]);
    /* open identity branches, innermost last: blocks may nest, and several blocks may start at the same variable */
    enum { MAX_OPEN = 16 };
    lbounds stashes[MAX_OPEN]; memset(stashes, 0, sizeof(stashes));
    int stash_src[MAX_OPEN], n_open = 0;
    for (int k = L - 1; k >= 0; --k) {
        lin_layer Lk = net_layer(net, k);
        if (skip_of(net, k) >= 0) {
            /* residual block: the coefficients at pre_k also multiply relu(pre_j) directly; keep a copy until the pass
             * reaches that variable (A_in = backward_F(A) + A, ny-core/src/gemm.rs:1640-1669) */
            if (n_open == MAX_OPEN) { lb_free(&cur); for (int i = 0; i < n_open; ++i) lb_free(&stashes[i]); return -2; }
            lbounds st = lb_alloc(cur.rows, cur.n, cur.le != NULL);
            memcpy(st.la, cur.la, 4 * (size_t)cur.rows * cur.n); memcpy(st.ua, cur.ua, 4 * (size_t)cur.rows * cur.n);
            if (cur.le) { memcpy(st.le, cur.le, 4 * (size_t)cur.rows * cur.n); memcpy(st.ue, cur.ue, 4 * (size_t)cur.rows * cur.n); }
            stashes[n_open] = st; stash_src[n_open] = skip_of(net, k); ++n_open;
        }
        lbounds nxt = linear_backward(&Lk, &cur);
        lb_free(&cur); cur = nxt;
        for (int oi = 0; oi < n_open; ) {
            if (stash_src[oi] != k - 1) { ++oi; continue; }
            lbounds stash = stashes[oi];
            /* cur holds the coefficients of relu(pre_{k-1}): the identity branch joins.  The rounded sums carry their
             * exact residual and both branches' certified errors in the error matrices (RESIDENT_SEG_MERGE). */
            size_t cnt = (size_t)cur.rows * cur.n;
            for (int side = 0; side < 2; ++side) {
                float *A = side ? cur.ua : cur.la, *E = side ? cur.ue : cur.le;
                const float *SA = side ? stash.ua : stash.la, *SE = side ? stash.ue : stash.le;
                for (size_t i = 0; i < cnt; ++i) {
                    double ex = (double)A[i] + (double)SA[i];
                    float v = (float)ex;
                    double e = fabs(ex - (double)v) + (E ? nonneg_err_or_inf(E[i]) : 0.0) + (SE ? nonneg_err_or_inf(SE[i]) : 0.0);
                    A[i] = v;
                    if (E) E[i] = (e == 0.0) ? 0.0f : publish_error_up_normal(e);
                }
            }
            lb_free(&stash);
            for (int m = oi + 1; m < n_open; ++m) { stashes[m - 1] = stashes[m]; stash_src[m - 1] = stash_src[m]; }
            --n_open;
        }
        if (k > 0 && relu_after(net, k - 1)) {
            int r = k - 1, n = net->dims[k];
            size_t o = pre_offset(net, r);
            signed char *sp = (signed char *)calloc((size_t)n, 1);
            unsigned char *hs = (unsigned char *)calloc((size_t)n, 1);
            float *sb = (float *)calloc((size_t)n, 4);
            for (int s = 0; s < n_splits; ++s) if (splits[s].relu == r) {
                int j = splits[s].neuron;
                sp[j] = (signed char)(splits[s].sign > 0 ? 1 : -1);
                hs[j] = 1; sb[j] = splits[s].beta * (splits[s].sign > 0 ? 1.0f : -1.0f);
            }
            lbounds rb = relu_backward_beta(&cur, pre_lo + o, pre_hi + o, sp, sb, hs, alpha ? alpha + o : NULL,
                                            alpha_up ? alpha_up + o : NULL);
            lb_free(&cur); cur = rb;
            free(sp); free(hs); free(sb);
        }
    }
    concretize(&cur, in_lo, in_hi, out_lo, out_hi);
    lb_free(&cur);
    return 0;
}

/* Intermediate bounds of a domain.
 * mode 0: engine/domain/child.rs:51-118 (clamp the split neuron only).
 * mode 1: engine/graph/propagation/constraints/mod.rs:400-760: walk the layers, re-propagate interval
 *         bounds, intersect with the inherited bound, then apply the pre-activation clamps
 *         (lookups.rs:138-185); ReLU outputs honour the split (active [max(l,0),u], inactive [0,0]). */
int nyo_domain_bounds(const nyo_net *net, const float *in_lo, const float *in_hi, const float *inh_lo,
                      const float *inh_hi, const nyo_split *splits, int n_splits, int mode,
                      float *pre_lo, float *pre_hi) {
    int L = net->n_linear;
    size_t total = pre_offset(net, L);
    memcpy(pre_lo, inh_lo, 4 * total); memcpy(pre_hi, inh_hi, 4 * total);
    if (mode == 0) {
        for (int s = 0; s < n_splits; ++s) {
            size_t o = pre_offset(net, splits[s].relu) + (size_t)splits[s].neuron;
            if (splits[s].sign > 0) pre_lo[o] = nanmax(pre_lo[o], 0.0f); else pre_hi[o] = nanmin(pre_hi[o], 0.0f);
            if (pre_lo[o] > pre_hi[o]) return 1;
        }
        return 0;
    }
    int maxn = 0;
    for (int k = 0; k <= L; ++k) if (net->dims[k] > maxn) maxn = net->dims[k];
    float *zl = (float *)malloc(4 * (size_t)maxn), *zu = (float *)malloc(4 * (size_t)maxn);
    float *nl = (float *)malloc(4 * (size_t)maxn), *nu = (float *)malloc(4 * (size_t)maxn);
    /* post-activation intervals of every layer, kept for the identity branches of residual blocks */
    float *post_l = net_has_skip(net) ? (float *)malloc(4 * total) : NULL, *post_u = post_l ? (float *)malloc(4 * total) : NULL;
    memcpy(zl, in_lo, 4 * (size_t)net->dims[0]); memcpy(zu, in_hi, 4 * (size_t)net->dims[0]);
    int infeasible = 0;
    for (int k = 0; k < L && !infeasible; ++k) {
        lin_layer Lk = net_layer(net, k);
        size_t o = pre_offset(net, k);
        int n = Lk.n_out;
        linear_ibp(&Lk, zl, zu, nl, nu);
        if (skip_of(net, k) >= 0) {  /* pre_k = W z + b + relu(pre_j): interval sum, rounded outward */
            size_t so = pre_offset(net, skip_of(net, k));
            for (int j = 0; j < n; ++j) {
                nl[j] = f64_to_f32_down_ns((double)nl[j] + (double)post_l[so + j]);
                nu[j] = f64_to_f32_up_ns((double)nu[j] + (double)post_u[so + j]);
            }
        }
        /* repropagated.intersection_per_element(current) (:738-741): self = re-propagated */
        if (intersect_per_element(nl, nu, pre_lo + o, pre_hi + o, n)) { memcpy(pre_lo + o, nl, 4 * (size_t)n); memcpy(pre_hi + o, nu, 4 * (size_t)n); }
        else { memcpy(pre_lo + o, nl, 4 * (size_t)n); memcpy(pre_hi + o, nu, 4 * (size_t)n); }
        if (k == L - 1) break;
        if (!relu_after(net, k)) {
            for (int j = 0; j < n; ++j) { zl[j] = pre_lo[o + j]; zu[j] = pre_hi[o + j]; }
            continue;
        }
        for (int s = 0; s < n_splits; ++s) if (splits[s].relu == k) {
            size_t q = o + (size_t)splits[s].neuron;
            if (splits[s].sign > 0) pre_lo[q] = nanmax(pre_lo[q], 0.0f); else pre_hi[q] = nanmin(pre_hi[q], 0.0f);
            if (pre_lo[q] > pre_hi[q]) infeasible = 1;
        }
        /* ReLU node (:428-548).  The inherited post-activation bound is relu(inherited pre-activation);
         * it never conflicts with the fresh bound because the pre-activation was already intersected. */
        for (int j = 0; j < n; ++j) { zl[j] = nanmax(pre_lo[o + j], 0.0f); zu[j] = nanmax(pre_hi[o + j], 0.0f); }
        for (int s = 0; s < n_splits; ++s) if (splits[s].relu == k) {
            int j = splits[s].neuron;
            if (splits[s].sign > 0) { if (pre_hi[o + j] < 0.0f) infeasible = 1; zl[j] = nanmax(pre_lo[o + j], 0.0f); zu[j] = pre_hi[o + j]; }
            else { if (pre_lo[o + j] > 0.0f) infeasible = 1; zl[j] = 0.0f; zu[j] = 0.0f; }
        }
        if (post_l) { memcpy(post_l + o, zl, 4 * (size_t)n); memcpy(post_u + o, zu, 4 * (size_t)n); }
    }
    free(zl); free(zu); free(nl); free(nu); free(post_l); free(post_u);
    return infeasible;
}

typedef struct {
    const nyo_net *net; const float *in_lo, *in_hi, *inh_lo, *inh_hi;
    const nyo_split *splits; const int32_t *n_splits; int max_splits, D, mode;
    float *out_lo, *out_hi; int32_t *infeasible;
    int next; pthread_mutex_t mu;
} batch_job;

static void *batch_worker(void *arg) {
    batch_job *J = (batch_job *)arg;
    int L = J->net->n_linear;
    size_t total = pre_offset(J->net, L);
    int S = J->net->dims[L];
    float *pl = (float *)malloc(4 * total), *pu = (float *)malloc(4 * total);
    for (;;) {
        pthread_mutex_lock(&J->mu);
        int d = J->next++;
        pthread_mutex_unlock(&J->mu);
        if (d >= J->D) break;
        const nyo_split *sp = J->splits + (size_t)d * J->max_splits;
        int inf = nyo_domain_bounds(J->net, J->in_lo, J->in_hi, J->inh_lo, J->inh_hi, sp, J->n_splits[d], J->mode, pl, pu);
        if (J->infeasible) J->infeasible[d] = inf;
        if (inf) {
            for (int s = 0; s < S; ++s) { J->out_lo[(size_t)d * S + s] = INFINITY; J->out_hi[(size_t)d * S + s] = -INFINITY; }
        } else {
            nyo_beta_crown_bound(J->net, J->in_lo, J->in_hi, pl, pu, sp, J->n_splits[d], NULL,
                                 J->out_lo + (size_t)d * S, J->out_hi + (size_t)d * S);
        }
    }
    free(pl); free(pu);
    return NULL;
}

/* The reference parallelises BaB children with rayon over domains
 * (beta_crown/engine/core.rs:651-684); this driver uses a pthread pool the same way. */
int nyo_bab_bound_batch(const nyo_net *net, const float *in_lo, const float *in_hi, const float *inh_lo,
                        const float *inh_hi, const nyo_split *splits, const int32_t *n_splits, int max_splits,
                        int D, int mode, float *out_lo, float *out_hi, int32_t *infeasible, int n_threads) {
    if (n_threads <= 0) { long c = sysconf(_SC_NPROCESSORS_ONLN); n_threads = c > 0 ? (int)c : 1; }
    if (n_threads > D) n_threads = D > 0 ? D : 1;
    batch_job J = { net, in_lo, in_hi, inh_lo, inh_hi, splits, n_splits, max_splits, D, mode, out_lo, out_hi, infeasible, 0, PTHREAD_MUTEX_INITIALIZER };
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)n_threads);
    for (int t = 1; t < n_threads; ++t) pthread_create(&th[t], NULL, batch_worker, &J);
    batch_worker(&J);
    for (int t = 1; t < n_threads; ++t) pthread_join(th[t], NULL);
    free(th);
    return n_threads;
}

/* beta_crown/engine/branching/sequential.rs:49-104 */
int nyo_select_largest_width(const nyo_net *net, const float *pre_lo, const float *pre_hi, const nyo_split *splits,
                             int n_splits, int32_t *relu, int32_t *neuron, float *width) {
    int L = net->n_linear, found = 0;
    float best = 0.0f;
    for (int r = 0; r < L - 1; ++r) {
        if (!relu_after(net, r)) continue;
        size_t o = pre_offset(net, r);
        for (int j = 0; j < net->dims[r + 1]; ++j) {
            float l = pre_lo[o + j], u = pre_hi[o + j];
            if (l >= 0.0f || u <= 0.0f) continue;
            int constrained = 0;
            for (int s = 0; s < n_splits; ++s) if (splits[s].relu == r && splits[s].neuron == j) { constrained = 1; break; }
            if (constrained) continue;
            float w = u - l;
            if (isnan(w)) continue;
            if (!found || w > best) { found = 1; best = w; *relu = r; *neuron = j; }
        }
    }
    if (found && width) *width = best;
    return found;
}

/* Intercept-score branching of the batched graph engine (batched_domain/domain_list/picked.rs:153-233):
 * score (-l*u)/(u-l) in fp32 over unstable unsplit neurons with u-l > 0, strict '>' so the first maximum in
 * (relu, neuron) order wins, NaN bounds skipped. */
int nyo_select_intercept(const nyo_net *net, const float *pre_lo, const float *pre_hi, const nyo_split *splits,
                         int n_splits, int32_t *relu, int32_t *neuron, float *score) {
    int L = net->n_linear, found = 0;
    float best = 0.0f;
    for (int r = 0; r < L - 1; ++r) {
        if (!relu_after(net, r)) continue;
        size_t o = pre_offset(net, r);
        for (int j = 0; j < net->dims[r + 1]; ++j) {
            float l = pre_lo[o + j], u = pre_hi[o + j];
            if (isnan(l) || isnan(u)) continue;
            if (l >= 0.0f || u <= 0.0f) continue;
            int constrained = 0;
            for (int s = 0; s < n_splits; ++s) if (splits[s].relu == r && splits[s].neuron == j) { constrained = 1; break; }
            if (constrained) continue;
            float w = u - l;
            if (!(w > 0.0f)) continue;
            float sc = (-l * u) / w;
            if (!found || sc > best) { found = 1; best = sc; *relu = r; *neuron = j; }
        }
    }
    if (found && score) *score = best;
    return found;
}

/* beta_crown/config/beta_config.rs:1552-1610 (lower mode) */
int nyo_domain_verified(float lower, float upper, float threshold) {
    if (!isfinite(lower) || !isfinite(upper) || !isfinite(threshold) || lower > upper) return 0;
    return lower > threshold;
}
int nyo_domain_violated(float lower, float upper, float threshold) {
    if (!isfinite(lower) || !isfinite(upper) || !isfinite(threshold)) return 0;
    if (lower > upper) return 0;
    return upper < threshold;
}

/* ------------------------------------------------------------------ alpha/beta optimisation */
/* Value of the lower rows and its joint gradient with respect to every lower slope alpha and every split
 * multiplier beta, by the forward fold + reverse adjoint of ny-core/src/joint_alpha_grad.rs:22-50,101-170
 * (coefficient and bias channels, no certified-error channel: the gradient only proposes the next
 * parameters, the bound itself is always re-evaluated by the sound fold).  The ReLU lines are the BaB ones
 * (beta_crown/engine/backward/relu_backward.rs:63-101); beta enters as A' -= beta*sign, so
 * d(bound_s)/d(beta_j) = -sign_j * Zpre[s,j] (beta_crown/engine/optimization/gradients/joint.rs:447-568).
 * The objective is the sum of the lower bounds over the spec rows.  Binary64 throughout. */
int nyo_joint_gradient(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                       const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                       double *lower_out, float *grad_alpha, float *grad_beta) {
    return nyo_joint_gradient_rows(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, lower_out, grad_alpha,
                                   grad_beta, -1);
}

/* only_row >= 0: the objective is that single row's lower bound (the argmin-lower row of
 * beta_crown/engine/optimization/optimize_loop.rs:77-333) instead of the sum over rows. */
int nyo_joint_gradient_rows(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                            const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                            double *lower_out, float *grad_alpha, float *grad_beta, int only_row) {
    if (net_has_conv(net) || net_has_skip(net)) return -2;
    int L = net->n_linear, S = net->dims[L];
    size_t total = pre_offset(net, L);
    /* per-ReLU records */
    double **apre = (double **)calloc((size_t)L, sizeof(double *));
    double **sig = (double **)calloc((size_t)L, sizeof(double *));
    double **tau = (double **)calloc((size_t)L, sizeof(double *));
    int n = S;
    double *A = (double *)calloc((size_t)S * n, 8), *b = (double *)calloc((size_t)S, 8);
    for (int s = 0; s < S; ++s) A[(size_t)s * n + s] = 1.0;
    for (int k = L - 1; k >= 0; --k) {
        lin_layer Lk = net_layer(net, k);
        double *An = (double *)calloc((size_t)S * Lk.n_in, 8);
        for (int s = 0; s < S; ++s)
            for (int o = 0; o < Lk.n_out; ++o) {
                double a = A[(size_t)s * Lk.n_out + o];
                if (a == 0.0) continue;
                const float *w = Lk.W + (size_t)o * Lk.n_in;
                for (int j = 0; j < Lk.n_in; ++j) An[(size_t)s * Lk.n_in + j] += a * (double)w[j];
                if (Lk.b) b[s] += a * (double)Lk.b[o];
            }
        free(A); A = An; n = Lk.n_in;
        if (k > 0 && relu_after(net, k - 1)) {
            int r = k - 1;
            size_t o = pre_offset(net, r);
            apre[r] = (double *)malloc(8 * (size_t)S * n);
            sig[r] = (double *)malloc(8 * (size_t)S * n);
            tau[r] = (double *)malloc(8 * (size_t)S * n);
            for (int j = 0; j < n; ++j) {
                float l = pre_lo[o + j], u = pre_hi[o + j];
                int sp = 0; float sb = 0.0f;
                for (int q = 0; q < n_splits; ++q) if (splits[q].relu == r && splits[q].neuron == j) {
                    sp = splits[q].sign > 0 ? 1 : -1; sb = isfinite(splits[q].beta) ? splits[q].beta * (float)sp : 0.0f;
                }
                double ls, us, ui;
                if (sp > 0) { ls = 1; us = 1; ui = 0; }
                else if (sp < 0) { ls = 0; us = 0; ui = 0; }
                else if (l >= 0.0f) { ls = 1; us = 1; ui = 0; }
                else if (u <= 0.0f) { ls = 0; us = 0; ui = 0; }
                else {
                    float w = fmaxf(u - l, RELU_RELAX_MIN_WIDTH);
                    us = (double)(u / w); ui = (double)(-l * u / w);
                    ls = alpha ? (double)alpha[o + j] : ((u > -l) ? 1.0 : 0.0);
                }
                for (int s = 0; s < S; ++s) {
                    size_t q = (size_t)s * n + j;
                    double a = A[q];
                    apre[r][q] = a;
                    double sg = (a >= 0.0) ? ls : us, ta = (a >= 0.0) ? 0.0 : ui;
                    sig[r][q] = sg; tau[r][q] = ta;
                    b[s] += a * ta;
                    A[q] = a * sg - (double)sb;
                }
            }
        }
    }
    /* concretise and seed the adjoint */
    int n0 = net->dims[0];
    double *Z = (double *)malloc(8 * (size_t)S * n0);
    for (int s = 0; s < S; ++s) {
        double v = b[s];
        for (int j = 0; j < n0; ++j) {
            double a = A[(size_t)s * n0 + j];
            double x = (a >= 0.0) ? (double)in_lo[j] : (double)in_hi[j];
            Z[(size_t)s * n0 + j] = x;
            v += a * x;
        }
        if (lower_out) lower_out[s] = v;
    }
    if (grad_alpha) memset(grad_alpha, 0, 4 * total);
    if (grad_beta) memset(grad_beta, 0, 4 * (size_t)(n_splits > 0 ? n_splits : 0));
    n = n0;
    for (int k = 0; k < L; ++k) {
        lin_layer Lk = net_layer(net, k);
        double *Zn = (double *)calloc((size_t)S * Lk.n_out, 8);
        for (int s = 0; s < S; ++s)
            for (int o = 0; o < Lk.n_out; ++o) {
                const float *w = Lk.W + (size_t)o * Lk.n_in;
                double acc = Lk.b ? (double)Lk.b[o] : 0.0;
                for (int j = 0; j < Lk.n_in; ++j) acc += Z[(size_t)s * Lk.n_in + j] * (double)w[j];
                Zn[(size_t)s * Lk.n_out + o] = acc;
            }
        free(Z); Z = Zn; n = Lk.n_out;
        if (k < L - 1 && relu_after(net, k)) {
            size_t o = pre_offset(net, k);
            for (int j = 0; j < n; ++j) {
                float l = pre_lo[o + j], u = pre_hi[o + j];
                int split_idx = -1;
                for (int q = 0; q < n_splits; ++q) if (splits[q].relu == k && splits[q].neuron == j) split_idx = q;
                double ga = 0.0, gz = 0.0;
                for (int s = 0; s < S; ++s) {
                    size_t q = (size_t)s * n + j;
                    double ap = apre[k][q];
                    if (only_row < 0 || s == only_row) {
                        ga += Z[q] * (ap > 0.0 ? ap : 0.0);
                        gz += Z[q];
                    }
                    Z[q] = Z[q] * sig[k][q] + tau[k][q];
                }
                if (split_idx >= 0) { if (grad_beta) grad_beta[split_idx] = (float)(-(double)(splits[split_idx].sign > 0 ? 1 : -1) * gz); }
                else if (l < 0.0f && u > 0.0f && grad_alpha) grad_alpha[o + j] = (float)ga;
            }
        }
    }
    for (int r = 0; r < L; ++r) { free(apre[r]); free(sig[r]); free(tau[r]); }
    free(apre); free(sig); free(tau); free(A); free(b); free(Z);
    return 0;
}

/* Upper-bound counterpart of the joint gradient for the dual alpha: value of the upper rows and the gradient of
 * their sum with respect to alpha_up, the slope the upper path applies to negative coefficients on unstable
 * unsplit neurons (activations/relu/mod.rs:570-1128: "upper-path alpha for ua < 0").  Fold: a >= 0 takes the chord
 * (us, ui), a < 0 takes (alpha_up, 0), then + beta*sign; corner x_u for a >= 0 else x_l;
 * d(upper_s)/d(alpha_up_i) = Zpre[s,i] * min(Apre[s,i], 0).  Binary64 throughout. */
int nyo_upper_gradient(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                       const float *pre_hi, const nyo_split *splits, int n_splits, const float *alpha,
                       const float *alpha_up, double *upper_out, float *grad_alpha_up) {
    if (net_has_conv(net) || net_has_skip(net)) return -2;
    int L = net->n_linear, S = net->dims[L];
    size_t total = pre_offset(net, L);
    double **apre = (double **)calloc((size_t)L, sizeof(double *));
    double **sig = (double **)calloc((size_t)L, sizeof(double *));
    double **tau = (double **)calloc((size_t)L, sizeof(double *));
    int n = S;
    double *A = (double *)calloc((size_t)S * n, 8), *b = (double *)calloc((size_t)S, 8);
    for (int s = 0; s < S; ++s) A[(size_t)s * n + s] = 1.0;
    for (int k = L - 1; k >= 0; --k) {
        lin_layer Lk = net_layer(net, k);
        double *An = (double *)calloc((size_t)S * Lk.n_in, 8);
        for (int s = 0; s < S; ++s)
            for (int o = 0; o < Lk.n_out; ++o) {
                double a = A[(size_t)s * Lk.n_out + o];
                if (a == 0.0) continue;
                const float *w = Lk.W + (size_t)o * Lk.n_in;
                for (int j = 0; j < Lk.n_in; ++j) An[(size_t)s * Lk.n_in + j] += a * (double)w[j];
                if (Lk.b) b[s] += a * (double)Lk.b[o];
            }
        free(A); A = An; n = Lk.n_in;
        if (k > 0 && relu_after(net, k - 1)) {
            int r = k - 1;
            size_t o = pre_offset(net, r);
            apre[r] = (double *)malloc(8 * (size_t)S * n);
            sig[r] = (double *)malloc(8 * (size_t)S * n);
            tau[r] = (double *)malloc(8 * (size_t)S * n);
            for (int j = 0; j < n; ++j) {
                float l = pre_lo[o + j], u = pre_hi[o + j];
                int sp = 0; float sb = 0.0f;
                for (int q = 0; q < n_splits; ++q) if (splits[q].relu == r && splits[q].neuron == j) {
                    sp = splits[q].sign > 0 ? 1 : -1; sb = isfinite(splits[q].beta) ? splits[q].beta * (float)sp : 0.0f;
                }
                double lsu, us, ui;
                if (sp > 0) { lsu = 1; us = 1; ui = 0; }
                else if (sp < 0) { lsu = 0; us = 0; ui = 0; }
                else if (l >= 0.0f) { lsu = 1; us = 1; ui = 0; }
                else if (u <= 0.0f) { lsu = 0; us = 0; ui = 0; }
                else {
                    float w = fmaxf(u - l, RELU_RELAX_MIN_WIDTH);
                    us = (double)(u / w); ui = (double)(-l * u / w);
                    lsu = alpha_up ? (double)alpha_up[o + j] : (alpha ? (double)alpha[o + j] : ((u > -l) ? 1.0 : 0.0));
                }
                for (int s = 0; s < S; ++s) {
                    size_t q = (size_t)s * n + j;
                    double a = A[q];
                    apre[r][q] = a;
                    double sg = (a >= 0.0) ? us : lsu, ta = (a >= 0.0) ? ui : 0.0;
                    sig[r][q] = sg; tau[r][q] = ta;
                    b[s] += a * ta;
                    A[q] = a * sg + (double)sb;
                }
            }
        }
    }
    int n0 = net->dims[0];
    double *Z = (double *)malloc(8 * (size_t)S * n0);
    for (int s = 0; s < S; ++s) {
        double v = b[s];
        for (int j = 0; j < n0; ++j) {
            double a = A[(size_t)s * n0 + j];
            double x = (a >= 0.0) ? (double)in_hi[j] : (double)in_lo[j];
            Z[(size_t)s * n0 + j] = x;
            v += a * x;
        }
        if (upper_out) upper_out[s] = v;
    }
    if (grad_alpha_up) memset(grad_alpha_up, 0, 4 * total);
    n = n0;
    for (int k = 0; k < L; ++k) {
        lin_layer Lk = net_layer(net, k);
        double *Zn = (double *)calloc((size_t)S * Lk.n_out, 8);
        for (int s = 0; s < S; ++s)
            for (int o = 0; o < Lk.n_out; ++o) {
                const float *w = Lk.W + (size_t)o * Lk.n_in;
                double acc = Lk.b ? (double)Lk.b[o] : 0.0;
                for (int j = 0; j < Lk.n_in; ++j) acc += Z[(size_t)s * Lk.n_in + j] * (double)w[j];
                Zn[(size_t)s * Lk.n_out + o] = acc;
            }
        free(Z); Z = Zn; n = Lk.n_out;
        if (k < L - 1 && relu_after(net, k)) {
            size_t o = pre_offset(net, k);
            for (int j = 0; j < n; ++j) {
                float l = pre_lo[o + j], u = pre_hi[o + j];
                int is_split = 0;
                for (int q = 0; q < n_splits; ++q) if (splits[q].relu == k && splits[q].neuron == j) is_split = 1;
                double ga = 0.0;
                for (int s = 0; s < S; ++s) {
                    size_t q = (size_t)s * n + j;
                    double ap = apre[k][q];
                    ga += Z[q] * (ap < 0.0 ? ap : 0.0);
                    Z[q] = Z[q] * sig[k][q] + tau[k][q];
                }
                if (!is_split && l < 0.0f && u > 0.0f && grad_alpha_up) grad_alpha_up[o + j] = (float)ga;
            }
        }
    }
    for (int r = 0; r < L; ++r) { free(apre[r]); free(sig[r]); free(tau[r]); }
    free(apre); free(sig); free(tau); free(A); free(b); free(Z);
    return 0;
}

/* Projected-Adam ascent on alpha (clamped to [0,1], unstable unsplit neurons only:
 * bounds/alpha/shared.rs:106-146) and beta (clamped to >= 0, gradient clipped to +-clip:
 * beta_crown/state/beta.rs:314-441), learning rate lr * decay^(t-1), intermediate bounds fixed.  Each iteration
 * evaluates the sound bound with the current parameters first and keeps the element-wise best
 * (network/alpha_crown_loop.rs:928-936), then steps along the joint gradient.  alpha (n_pre layout) and the
 * beta fields of `splits` are updated in place. */
int nyo_optimize(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo, const float *pre_hi,
                 nyo_split *splits, int n_splits, float *alpha, int iterations, float lr_alpha, float lr_beta,
                 float lr_decay, float clip_beta, float *best_lo, float *best_hi) {
    return nyo_optimize_objective(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, iterations, lr_alpha, lr_beta,
                                  lr_decay, clip_beta, 0, best_lo, best_hi);
}

/* objective 0: sum of the rows' lower bounds; 1: the row whose current lower bound is smallest; 2: dual alpha -
 * as 0 for alpha and beta, and in addition a separate upper-path slope alpha_up (started at alpha) descends the sum
 * of the upper bounds.  alpha_up_out (n_pre floats, may be NULL) receives the final upper-path slopes. */
int nyo_optimize_objective(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                           const float *pre_hi, nyo_split *splits, int n_splits, float *alpha, int iterations,
                           float lr_alpha, float lr_beta, float lr_decay, float clip_beta, int objective, float *best_lo,
                           float *best_hi) {
    return nyo_optimize_dual(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, iterations, lr_alpha, lr_beta,
                             lr_decay, clip_beta, objective, best_lo, best_hi, NULL);
}

int nyo_optimize_dual(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                      const float *pre_hi, nyo_split *splits, int n_splits, float *alpha, int iterations,
                      float lr_alpha, float lr_beta, float lr_decay, float clip_beta, int objective, float *best_lo,
                      float *best_hi, float *alpha_up_out) {
    nyo_opt_cfg c;
    memset(&c, 0, sizeof(c));
    c.iterations = iterations; c.lr_alpha = lr_alpha; c.lr_beta = lr_beta; c.lr_decay = lr_decay; c.clip_beta = clip_beta;
    c.objective = objective;
    return nyo_optimize_ex(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, &c, best_lo, best_hi, alpha_up_out, NULL);
}

/* The loop with the reference's update rules and stopping rules selectable:
 *   rule 0  projected Adam (above);
 *   rule 1  the plain projected step that is the reference's default (use_adaptive = false):
 *           beta <- max(0, beta + lr g) (BetaState::gradient_step, beta_crown/state/beta.rs:272-305),
 *           alpha <- clamp(alpha + lr g, 0, 1); no moments; the gradient clip does not apply;
 *   rule 2  Adam with AMSGrad's running maximum of the second moment (beta.rs:369-376).
 *   tolerance > 0: stop once max |gradient| over the domain's parameters (clipped beta gradients, raw alpha gradients)
 *           is below it (optimize_loop.rs:272-279; NaN never compares below);
 *   patience > 0: stop once the objective's best value has not improved for more than `patience` iterations
 *           (patience_exhausted_after_iteration, optimize_loop.rs:45-57);
 *   start_save_best in (0, 1): the element-wise best bounds are only updated at the first iteration, after
 *           iterations * start_save_best iterations, at the last one and when stopping
 *           (should_save_best, bounds/alpha_config.rs:1085-1091; alpha_crown_loop.rs:928-936).
 * A stop takes effect after the update of its iteration; the parameters it leaves are evaluated once more and that
 * evaluation is folded into the best bounds (the reference returns without it: this can only be tighter).
 * iterations_run (may be NULL) receives the number of bound evaluations made. */
int nyo_optimize_ex(const nyo_net *net, const float *in_lo, const float *in_hi, const float *pre_lo,
                    const float *pre_hi, nyo_split *splits, int n_splits, float *alpha, const nyo_opt_cfg *cfg,
                    float *best_lo, float *best_hi, float *alpha_up_out, int *iterations_run) {
    const int iterations = cfg->iterations, objective = cfg->objective, rule = cfg->rule;
    const float lr_alpha = cfg->lr_alpha, lr_beta = cfg->lr_beta, lr_decay = cfg->lr_decay, clip_beta = cfg->clip_beta;
    int L = net->n_linear, S = net->dims[L];
    size_t total = pre_offset(net, L);
    float *ga = (float *)calloc(total, 4), *ma = (float *)calloc(total, 4), *va = (float *)calloc(total, 4);
    float *gb = (float *)calloc((size_t)(n_splits + 1), 4), *mb = (float *)calloc((size_t)(n_splits + 1), 4), *vb = (float *)calloc((size_t)(n_splits + 1), 4);
    float *xa = (float *)calloc(total, 4), *xu = (float *)calloc(total, 4), *xb = (float *)calloc((size_t)(n_splits + 1), 4); /* AMSGrad maxima */
    float *lo = (float *)malloc(4 * (size_t)S), *hi = (float *)malloc(4 * (size_t)S);
    const float b1 = 0.9f, b2 = 0.999f, eps = 1e-8f;
    const int dual = objective == 2 && alpha != NULL;
    float *aup = NULL, *gu = NULL, *mu = NULL, *vu = NULL;
    if (dual) {
        aup = (float *)malloc(4 * total); memcpy(aup, alpha, 4 * total);
        gu = (float *)calloc(total, 4); mu = (float *)calloc(total, 4); vu = (float *)calloc(total, 4);
    }
    for (int s = 0; s < S; ++s) { best_lo[s] = -INFINITY; best_hi[s] = INFINITY; }
    const int save_from = (int)((float)iterations * cfg->start_save_best);  /* zero-based iteration threshold */
    float best_obj = -INFINITY;
    int no_improve = 0, stopping = 0, runs = 0;
    for (int t = 1; t <= iterations; ++t) {
        nyo_beta_crown_bound_dual(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, aup, lo, hi);
        ++runs;
        if (t == 1 || (t - 1) > save_from || t == iterations || stopping || !(cfg->start_save_best > 0.0f))
            for (int s = 0; s < S; ++s) { if (lo[s] > best_lo[s]) best_lo[s] = lo[s]; if (hi[s] < best_hi[s]) best_hi[s] = hi[s]; }
        if (t == iterations || stopping) break;
        float obj = 0.0f;
        if (objective == 1) { obj = lo[0]; for (int s = 1; s < S; ++s) if (lo[s] < obj) obj = lo[s]; }
        else for (int s = 0; s < S; ++s) if (isfinite(lo[s])) obj += lo[s];
        if (dual) nyo_upper_gradient(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, aup, NULL, gu);
        int row = -1;
        if (objective == 1) { row = 0; for (int s = 1; s < S; ++s) if (lo[s] < lo[row]) row = s; }
        nyo_joint_gradient_rows(net, in_lo, in_hi, pre_lo, pre_hi, splits, n_splits, alpha, NULL, ga, gb, row);
        float bc1 = fmaxf(1.0f - powf(b1, (float)t), 1.1920929e-7f), bc2 = fmaxf(1.0f - powf(b2, (float)t), 1.1920929e-7f);
        float lra = lr_alpha * powf(lr_decay, (float)(t - 1)), lrb = lr_beta * powf(lr_decay, (float)(t - 1));
        size_t hidden = pre_offset(net, L - 1);
        float max_grad = 0.0f;
#define NYO_MAXG(g) do { float _a = fabsf(g); if (isnan(_a) || isnan(max_grad)) max_grad = NAN; else if (_a > max_grad) max_grad = _a; } while (0)
        if (alpha && lr_alpha > 0.0f) for (size_t i = 0; i < hidden; ++i) {
            if (!(pre_lo[i] < 0.0f && pre_hi[i] > 0.0f)) continue;
            int is_split = 0;
            for (int q = 0; q < n_splits; ++q) if (pre_offset(net, splits[q].relu) + (size_t)splits[q].neuron == i) is_split = 1;
            if (is_split) continue;
            float g = ga[i];
            NYO_MAXG(g);
            float a;
            if (rule == 1) a = alpha[i] + lra * g;
            else {
                ma[i] = b1 * ma[i] + (1.0f - b1) * g;
                va[i] = b2 * va[i] + (1.0f - b2) * g * g;
                float v = va[i];
                if (rule == 2) { xa[i] = (isnan(xa[i]) || isnan(v)) ? NAN : fmaxf(xa[i], v); v = xa[i]; }
                a = alpha[i] + lra * (ma[i] / bc1) / (sqrtf(v / bc2) + eps);
            }
            a = fminf(fmaxf(a, 0.0f), 1.0f);
            if (isnan(a)) { a = 0.5f; ma[i] = 0.0f; va[i] = 0.0f; xa[i] = 0.0f; }
            alpha[i] = a;
        }
        if (dual && lr_alpha > 0.0f) for (size_t i = 0; i < hidden; ++i) {
            if (!(pre_lo[i] < 0.0f && pre_hi[i] > 0.0f)) continue;
            int is_split = 0;
            for (int q = 0; q < n_splits; ++q) if (pre_offset(net, splits[q].relu) + (size_t)splits[q].neuron == i) is_split = 1;
            if (is_split) continue;
            float g = gu[i];
            float a;
            if (rule == 1) a = aup[i] - lra * g;
            else {
                mu[i] = b1 * mu[i] + (1.0f - b1) * g;
                vu[i] = b2 * vu[i] + (1.0f - b2) * g * g;
                float v = vu[i];
                if (rule == 2) { xu[i] = (isnan(xu[i]) || isnan(v)) ? NAN : fmaxf(xu[i], v); v = xu[i]; }
                a = aup[i] - lra * (mu[i] / bc1) / (sqrtf(v / bc2) + eps);   /* descent: the upper bound shrinks */
            }
            a = fminf(fmaxf(a, 0.0f), 1.0f);
            if (isnan(a)) { a = 0.5f; mu[i] = 0.0f; vu[i] = 0.0f; xu[i] = 0.0f; }
            aup[i] = a;
        }
        if (lr_beta > 0.0f) for (int q = 0; q < n_splits; ++q) {
            float g = gb[q];
            if (rule != 1 && clip_beta > 0.0f) g = fminf(fmaxf(g, -clip_beta), clip_beta);
            NYO_MAXG(g);
            float bnew;
            if (rule == 1) bnew = splits[q].beta + lrb * g;
            else {
                mb[q] = b1 * mb[q] + (1.0f - b1) * g;
                vb[q] = b2 * vb[q] + (1.0f - b2) * g * g;
                float v = vb[q];
                if (rule == 2) { xb[q] = (isnan(xb[q]) || isnan(v)) ? NAN : fmaxf(xb[q], v); v = xb[q]; }
                bnew = splits[q].beta + lrb * (mb[q] / bc1) / (sqrtf(v / bc2) + eps);
            }
            if (isnan(bnew) || isinf(bnew)) { bnew = 0.0f; mb[q] = 0.0f; vb[q] = 0.0f; xb[q] = 0.0f; }
            splits[q].beta = fmaxf(bnew, 0.0f);
        }
#undef NYO_MAXG
        if (cfg->tolerance > 0.0f && max_grad < cfg->tolerance) stopping = 1;
        if (obj > best_obj) { best_obj = obj; no_improve = 0; } else ++no_improve;
        if (cfg->patience > 0 && no_improve > cfg->patience) stopping = 1;
    }
    if (iterations_run) *iterations_run = runs;
    if (dual && alpha_up_out) memcpy(alpha_up_out, aup, 4 * total);
    free(aup); free(gu); free(mu); free(vu); free(xa); free(xu); free(xb);
    free(ga); free(ma); free(va); free(gb); free(mb); free(vb); free(lo); free(hi);
    return 0;
}
