// BaBSR branching scores for the resident batch (select_babsr_neuron / compute_babsr_scores,
// crates/ny-propagate/src/beta_crown/engine/branching/sequential.rs:106-198, 784-882; the score kernel is
// compute_babsr_score_parts, branching/score.rs:28-97).
//
// Per domain a coefficient matrix C starts as the specification rows and walks the network backwards:
// C <- C W_k at a Linear layer; at ReLU r every neuron j gets
//   ratio_0 = max(u,0) / (max(u,0) - min(l,0)),  ratio_1 = -min(l,0) * ratio_0
//   score_j = mean_s | min(b_j c_sj (ratio_0 - 1), b_j c_sj ratio_0) + min(c_sj, 0) ratio_1 |
// (b_j the bias of the producing Linear layer), then column j of C is scaled by the upper slope (1 for l >= 0,
// 0 for u <= 0, u / max(u - l, 1e-8) otherwise).  The split goes to the unstable, unsplit neuron with the largest
// score; the first one in (relu, neuron) order wins ties; neurons whose score cannot be formed score 0.
// All domains walk in lock-step, the products run on the engine's contraction path.  A heuristic: nothing here
// enters a bound.
#include <math.h>

#include "nyb200_internal.cuh"

namespace nyb {

namespace {

__global__ void k_babsr_seed(long rows, int S, int nL, const float *__restrict__ spec, float *__restrict__ C, int ldc) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= rows * nL) return;
    long r = t / nL;
    int j = (int)(t - r * nL);
    C[r * ldc + j] = spec[(long)(r % S) * nL + j];
}

__global__ void k_babsr_fill(long n, float v, float *__restrict__ p) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) p[t] = v;
}

// One thread per (domain, neuron of this ReLU): score from its column of C, then the column is scaled.
__global__ void __launch_bounds__(256)
k_babsr_relu(int n, int off, int D, int S, long nps, float *__restrict__ C, int ldc, const float *__restrict__ pre_lo,
             const float *__restrict__ pre_hi, const signed char *__restrict__ code, const float *__restrict__ bias,
             float *__restrict__ score, float *__restrict__ backup) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * n) return;
    const int d = (int)(t / n), j = (int)(t - (long)d * n);
    const long o = (long)d * nps + off + j;
    const float l = pre_lo[o], u = pre_hi[o];
    const float b = bias ? bias[j] : 0.f;
    // babsr_ratio_terms
    bool have = isfinite(l) && isfinite(u);
    float r0 = 0.f, r1 = 0.f;
    if (have) {
        const float lt = fminf(l, 0.f), ut = fmaxf(u, 0.f), w = __fsub_rn(ut, lt);
        if (fabsf(w) <= 1e-6f) have = false;
        else {
            r0 = __fdiv_rn(ut, w);
            r1 = __fmul_rn(-lt, r0);
            have = isfinite(r0) && isfinite(r1);
        }
    }
    // relu_upper_slope
    float slope;
    if (!isfinite(l) || !isfinite(u)) slope = 1.f;
    else if (l >= 0.f) slope = 1.f;
    else if (u <= 0.f) slope = 0.f;
    else slope = __fdiv_rn(u, fmaxf(__fsub_rn(u, l), 1e-8f));
    double sum = 0.0, bsum = 0.0;
    bool ok = have;
    float *col = C + (long)d * S * ldc + j;
    for (int s = 0; s < S; ++s) {
        const float c = col[(long)s * ldc];
        if (ok) {
            if (!isfinite(c)) ok = false;
            else {
                const float ic = __fmul_rn(fminf(c, 0.f), r1);
                const float bs = __fmul_rn(b, c);
                const float bc = fminf(__fmul_rn(bs, __fsub_rn(r0, 1.f)), __fmul_rn(bs, r0));
                const float mc = fabsf(__fadd_rn(bc, ic));
                if (!isfinite(ic) || !isfinite(mc)) ok = false;
                else { sum += (double)mc; bsum += (double)ic; }
            }
        }
        col[(long)s * ldc] = __fmul_rn(c, slope);
    }
    const bool candidate = l < 0.f && u > 0.f && code[o] == 0;
    score[o] = candidate ? (ok ? (float)(sum / (double)S) : 0.f) : -1.f;
    // the "backup" score of the filtered heuristics: mean intercept term, <= 0, more negative = looser relaxation
    backup[o] = candidate ? (ok ? (float)(bsum / (double)S) : 0.f) : 1.f;
}

// First maximum of the scores (non-candidates hold -1, NaN never wins), one warp per domain.
__global__ void __launch_bounds__(256)
k_babsr_pick(NetView nv, int D, const float *__restrict__ score, int *__restrict__ relu, int *__restrict__ neuron,
             float *__restrict__ out) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= D) return;
    const int n_hidden = nv.pre_off[nv.L - 1];
    float best = -1.f;
    int bidx = 0x7fffffff;
    for (int i = lane; i < n_hidden; i += 32) {
        float s = score[(long)warp * nv.nps + i];
        if (s > best) { best = s; bidx = i; }  // false for NaN; ascending i per lane keeps the first maximum
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; }
    }
    if (lane == 0) {
        if (bidx == 0x7fffffff) { relu[warp] = -1; neuron[warp] = -1; out[warp] = 0.f; }
        else {
            int r = 0;
            while (r + 1 < nv.L - 1 && bidx >= nv.pre_off[r + 1]) ++r;
            relu[warp] = r; neuron[warp] = bidx - nv.pre_off[r]; out[warp] = best;
        }
    }
}

}  // namespace

// Scores every hidden neuron of every domain of the resident batch (after a run) and picks the split.
// score_out (device, [D x nps]) may be read back by the caller for diagnostics.
int babsr_select(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int *relu, int *neuron, float *best,
                 float **score_dev) {
    const NetView &nv = net.v;
    const int L = nv.L, D = b.D, S = b.S;
    for (int k = 0; k < L; ++k)
        if (net.is_conv(k)) return set_err(e, NYB200_ERR_UNSUPPORTED, "BaBSR scores are built for Linear layers only");
    if (net.has_skip()) return set_err(e, NYB200_ERR_UNSUPPORTED, "BaBSR scores are not built for residual networks");
    const long rows = (long)D * S, np = nv.nps;
    const int ldc = p.lda;
    const bool tensor = e->path == NYB200_PATH_TF32X3;
    NYB_WS(c0, float *, e, "babsr_c0", (size_t)rows * ldc * 4);
    NYB_WS(c1, float *, e, "babsr_c1", (size_t)rows * ldc * 4);
    NYB_WS(score, float *, e, "babsr_score", (size_t)2 * D * np * 4);  // main scores, then the backup scores
    float *backup = score + (size_t)D * np;
    int *derr = nullptr;
    if (tensor) {
        NYB_TRY(prepare_backward_operands(e, net));
        derr = (int *)ws_get(e, "umma_err", 256);
        if (!derr) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(derr, 0, 4, e->stream));
    }
    const int nL = nv.dims[L];
    k_babsr_fill<<<(unsigned)(((long)D * np + 255) / 256), 256, 0, e->stream>>>((long)D * np, -1.f, score);  // output block, padding
    k_babsr_fill<<<(unsigned)(((long)D * np + 255) / 256), 256, 0, e->stream>>>((long)D * np, 1.f, backup);
    e->launches += 2;
    k_babsr_seed<<<(unsigned)((rows * nL + 255) / 256), 256, 0, e->stream>>>(rows, S, nL, p.spec, c0, ldc);
    e->launches++;
    float *cur = c0, *nxt = c1;
    for (int k = L - 1; k >= 1; --k) {
        NYB_DEADLINE(e, "branching scores");
        const int K = nv.dims[k + 1], N = nv.dims[k];
        if (tensor) NYB_TRY(launch_umma(e, net.umma[k], (int)rows, cur, ldc, nxt, ldc, derr));
        else launch_gemm_f64(e, (int)rows, N, K, cur, ldc, nv.W[k], N, nxt, ldc, 1, nullptr, nullptr, 0, nullptr);
        const long tot = (long)D * N;
        k_babsr_relu<<<(unsigned)((tot + 255) / 256), 256, 0, e->stream>>>(N, nv.pre_off[k - 1], D, S, np, nxt, ldc, p.pre_lo,
                                                                          p.pre_hi, p.code, nv.b[k - 1], score, backup);
        e->launches++;
        float *t = cur; cur = nxt; nxt = t;
    }
    k_babsr_pick<<<(unsigned)(((long)D * 32 + 255) / 256), 256, 0, e->stream>>>(nv, D, score, relu, neuron, best);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    if (derr) {
        int herr = 0;
        NYB_CUDA(e, cudaMemcpyAsync(&herr, derr, 4, cudaMemcpyDeviceToHost, e->stream));
        NYB_CUDA(e, cudaStreamSynchronize(e->stream));
        if (herr) return set_err(e, NYB200_ERR_INTERNAL, "tcgen05 pipeline wait expired (code " + std::to_string(herr) + ")");
    }
    if (score_dev) *score_dev = score;
    return NYB200_OK;
}

}  // namespace nyb
