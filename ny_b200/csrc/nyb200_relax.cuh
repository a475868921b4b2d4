// The per-coefficient step of the beta-CROWN ReLU relaxation pass, shared by the stand-alone relaxation kernels and
// by the fused backward chain so that both produce the same coefficient bits.
#pragma once

namespace nyb {

// One coefficient `a` of a row (`upper`: the row bounds from above) through ReLU's relaxation
// t = (lower slope, upper slope, upper intercept, signed beta), then the charges of the contraction that follows.
// au: the upper path's own lower slope (dual alpha, activations/relu/mod.rs:570-1128); equals t.x otherwise.
// za = max|pre-activation|, qv = |W| max|z| of the next contraction, bk its bias entry, eps its rounding rate.
// Accumulates the row's bias (sb, binary64), bias magnitude (sa) and rounding penalty (sp), both rounded upwards.
// `upper` may be a compile-time constant (the selects fold) or a per-thread value (no divergence either way).
template <bool RELAX, bool BIAS>
__device__ __forceinline__ float relax_coeff(const bool upper, float a, float4 t, float au, float za, float qv, float bk,
                                             float eps, double &sb, float &sa, float &sp) {
    float nw = a;
    if (RELAX) {
        const bool pos = a > 0.f;
        // lower rows: a > 0 takes the lower line (slope ls, no intercept), a < 0 the upper line (us, ui);
        // upper rows mirror it (relu_backward.rs:105-153)
        const float slope = (pos != upper) ? (upper ? au : t.x) : t.y;
        const float icp = ((pos == upper) && a != 0.f) ? t.z : 0.f;
        // the reference's rounding: round to nearest, then one ulp outward (relu_backward.rs:105-153); an exact
        // zero product (a == 0 or slope == 0) needs no step.  A directed product would be up to one ulp tighter,
        // which is visible on bounds that cancel to almost nothing; staying on the reference's values is worth
        // more here than that ulp.
        const float prod = __fmul_rn(a, slope);
        const unsigned pb = __float_as_uint(prod);
        const int neg = (int)pb >> 31;  // 0 or -1: one ulp outward is +-1 on the bit pattern, mirrored for negatives
        const unsigned step = 1u + 2u * (unsigned)neg;
        const float stepped = __uint_as_float(upper ? pb + step : pb - step);
        // a product that underflowed to zero takes the directed product instead (the bit step would wrap); an
        // overflowed one steps into a NaN pattern, which the concretisation turns into [-inf, +inf] for the row
        nw = stepped;
        if (prod == 0.f) nw = upper ? __fmul_ru(a, slope) : __fmul_rd(a, slope);
        nw = (a == 0.f || slope == 0.f) ? 0.f : nw;
        // The step above is outward in the coefficient.  That alone is sound where the variable it multiplies cannot
        // be negative: a neuron that is active on the whole domain (table (1, 1, 0): pre-activation lower bound >= 0,
        // by its interval or by a split).  Everywhere else the pre-activation may be negative and the gap between the
        // exact product and the stepped one is charged against its magnitude.
        const bool nonneg = (t.y == 1.f) && (t.z == 0.f);
        sp = __fmaf_ru(nonneg ? 0.f : fabsf(fmaf(a, slope, -nw)), za, sp);
        sb = fma((double)a, (double)icp, sb);
        sa = __fmaf_ru(fabsf(a), fabsf(icp), sa);
        nw = upper ? nw + t.w : nw - t.w;  // signed beta (zero for unsplit neurons), relu_backward.rs:156-175
    }
    if (BIAS) {
        sb = fma((double)nw, (double)bk, sb);
        sa = __fmaf_ru(fabsf(nw), fabsf(bk), sa);
    }
    sp = __fmaf_ru(__fmul_ru(eps, fabsf(nw)), qv, sp);
    return nw;
}

// The same coefficient step for the fused backward chain, with the row sums arranged for issue rate: the coefficient
// bits are those of relax_coeff (same product, same outward step, same beta addition); what differs is the
// bookkeeping around them.
//   * One charge per coefficient, |nw| * cj, with cj prepared once per (domain, column) by the caller:
//         cj = eps * q + (1.6 * 2^-23 + kappa) * max|z| + kappa * |bias|.
//     1.6 * 2^-23 |nw| bounds the gap between the exact product and the stepped one (within 1.5 ulp); it is charged
//     for neurons that cannot be negative as well (at most 3% more than the contraction's own charge).  kappa covers
//     the fp32 accumulation of the two dot products below: a run of n fused multiply-adds errs by at most
//     n * 2^-24 times the run's magnitude sum, and that sum is bounded term by term: |nw bias| directly, and
//     |a * intercept| <= |nw| * max|z| * (1 + 2^-21), because an intercept only applies on the upper line, where the
//     outward step moves nw away from zero (|nw| >= |a| * slope) and intercept / slope = -l up to rounding.
//     A product that underflows to zero stays zero; the floor of the charge encloses it.
//   * The intercept and bias dot products are accumulated in fp32 (gi, gb: one fused multiply-add per term) over a
//     short run of columns; the caller adds each run to the row's binary64 bias.
// dir = +1 for an upper row, -1 for a lower row; dirf the same as a float.
__device__ __forceinline__ float relax_coeff_fast(const bool upper, const int dir, const float dirf, float a, float4 t, float au,
                                                  float cj, float bk, float &gi, float &gb, float &sp) {
    const bool pos = a > 0.f;
    const float slope = (pos != upper) ? (upper ? au : t.x) : t.y;
    const float icp = (pos == upper) ? t.z : 0.f;   // times a == 0 it adds nothing
    const float prod = __fmul_rn(a, slope);
    const int pb = __float_as_int(prod);
    // one ulp outward on the bit pattern: +dir for a positive product, -dir for a negative one; a zero product (zero
    // slope or zero coefficient: common, every stably inactive neuron has one) stays zero without a branch
    // A zero product stays zero: exactly zero when the coefficient or the slope is zero (no step: every stably inactive
    // neuron has one); a product that underflowed (|a * slope| <= 2^-150) is enclosed by the floor of the charge below.
    float nw = __int_as_float((pb << 1) ? pb + dir + 2 * dir * (pb >> 31) : 0);
    gi = fmaf(a, icp, gi);
    nw = fmaf(t.w, dirf, nw);   // signed beta: nw + t.w on upper rows, nw - t.w on lower rows (t.w * +-1 is exact)
    gb = fmaf(nw, bk, gb);
    // the floor covers the underflow case, where the coefficient is taken as zero and the exact product is at most
    // 2^-150: 2^-148 max|z| <= 1.6e-38 cj because cj >= 1.9e-7 max|z| (and cj >= kappa |bias| for the bias product)
    sp = __fmaf_ru(fmaxf(fabsf(nw), 1.6e-38f), cj, sp);
    return nw;
}

}  // namespace nyb
