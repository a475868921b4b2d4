// Plain CROWN bounds with CROWN-IBP intermediate bounds for D input boxes in lock-step: the reference's
// `crown` pipeline (crates/ny-propagate/src/network/core/sequential/crown.rs:168-330 with the collection of
// network/ibp/crown_ibp.rs:32-420 and crown_partial.rs:166-182) on the device.
//
// For every Linear layer k whose output feeds a ReLU:
//   f   = interval image of Linear_k on the tightened input  z = relu(t_{k-1}) n relu(ibp_{k-1})
//   c   = partial CROWN pass from Linear_k's output (identity rows) down to the input box, with the ReLU
//         relaxations of the tightened bounds t_0..t_{k-1} (plain-CROWN chord: activations/relu/mod.rs:105-132,
//         activations/mod.rs:99-121)
//   t_k = ibp_k                                   if every neuron is IBP-stable (crown_ibp.rs:113-140)
//       = ibp_k n (f on f-stable neurons, c elsewhere)   if >= 90% of the neurons are f-stable
//                                                 (sparse merge: only unstable rows are propagated,
//                                                 ibp/sparse_merge.rs:118-146)
//       = ibp_k n c                               otherwise (crown_ibp.rs:186-215)
// where n is the per-element intersection with union fallback, skipped for the whole vector when it holds a NaN
// (ny-tensor bounded_tensor/core/numeric.rs:316-360).  The network's last Linear feeds the specification rows
// (another Linear): it takes the forward shortcut t = ibp n f (ibp/helpers.rs:99-107).  The specification rows
// are then bounded by the full backward pass, merged by the same rule, and intersected once more
// (crown/tighten.rs:126-190).  The stable rows of a sparse pass are computed here too (one dense pass is cheaper
// on the device than a gather) and simply not used, so the values are those of the reference's rule.
#include "nyb200_internal.cuh"

namespace nyb {

namespace {

constexpr int kAllStable = 1, kSparse = 2, kNan = 4;

__device__ __forceinline__ float next_up32(float x) {
    unsigned b = __float_as_uint(x), mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) return x;
    if (mag == 0) return __uint_as_float(1u);
    return (b & 0x80000000u) ? __uint_as_float(b - 1) : __uint_as_float(b + 1);
}

// Per (domain, layer): all-stable / sparse / NaN flags of the merge rule.  One warp per domain.
// ibp, f: [D x stride] blocks at `off`; c: [D x n] dense.
__global__ void __launch_bounds__(256)
k_crown_flags(int D, int n, const float *__restrict__ ibp_lo, const float *__restrict__ ibp_hi,
              const float *__restrict__ f_lo, const float *__restrict__ f_hi, long stride, int off,
              const float *__restrict__ c_lo, const float *__restrict__ c_hi, int *__restrict__ flags) {
    int d = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (d >= D) return;
    long o = (long)d * stride + off;
    int unstable_ibp = 0, n_unst = 0;
    for (int j = lane; j < n; j += 32) {
        float il = ibp_lo[o + j], iu = ibp_hi[o + j];
        if (!(il >= 0.f || iu <= 0.f)) unstable_ibp = 1;
        float l = f_lo[o + j], u = f_hi[o + j];
        if (l < 0.f && u > 0.f) ++n_unst;
    }
    unstable_ibp = __any_sync(0xffffffffu, unstable_ibp);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) n_unst += __shfl_xor_sync(0xffffffffu, n_unst, s);
    int sparse = 0;
    if (n_unst > 0) {
        float stable_frac = 1.0f - ((float)n_unst / (float)n);
        if (!(stable_frac < 0.9f)) sparse = 1;
    }
    int nan = 0;
    for (int j = lane; j < n; j += 32) {
        float il = ibp_lo[o + j], iu = ibp_hi[o + j];
        float l = f_lo[o + j], u = f_hi[o + j];
        bool use_f = c_lo == nullptr || (sparse && !(l < 0.f && u > 0.f));
        float cl = use_f ? l : c_lo[(long)d * n + j], cu = use_f ? u : c_hi[(long)d * n + j];
        if (isnan(il) || isnan(iu) || isnan(cl) || isnan(cu)) nan = 1;
    }
    nan = __any_sync(0xffffffffu, nan);
    if (lane == 0) flags[d] = (unstable_ibp ? 0 : kAllStable) | (sparse ? kSparse : 0) | (nan ? kNan : 0);
}

__device__ __forceinline__ void intersect(float &l, float &u, float bl, float bu) {
    float tl = fmaxf(l, bl), tu = fminf(u, bu);
    if (tl <= tu) { l = tl; u = tu; }
    else { l = fminf(l, bl); u = fmaxf(u, bu); }
}

// Merge of layer k's bounds and, for a layer that feeds a ReLU, its plain-CROWN relaxation table and the
// post-activation interval the next layer reads.  relu = 0: a Linear feeding a Linear (forward shortcut,
// c_lo == nullptr).
__global__ void k_crown_merge(int D, int n, int off, long stride, int relu, const float *__restrict__ ibp_lo,
                              const float *__restrict__ ibp_hi, const float *__restrict__ f_lo,
                              const float *__restrict__ f_hi, const float *__restrict__ c_lo,
                              const float *__restrict__ c_hi, const int *__restrict__ lflags, float *__restrict__ t_lo,
                              float *__restrict__ t_hi, float *__restrict__ zl, float *__restrict__ zu,
                              float4 *__restrict__ tab, float *__restrict__ zabs, int *__restrict__ dflags,
                              const signed char *__restrict__ code) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * n) return;
    int d = (int)(t / n), j = (int)(t % n);
    long o = (long)d * stride + off + j;
    const int sc = (relu && code) ? (int)code[o] : 0;   // +1 / -1: the domain fixes this neuron active / inactive
    int fl = lflags[d];
    float il = ibp_lo[o], iu = ibp_hi[o];
    float l = il, u = iu;
    const bool skip = relu && (fl & kAllStable);
    if (!skip && !(fl & kNan)) {
        float a = f_lo[o], b = f_hi[o];
        bool use_f = c_lo == nullptr || ((fl & kSparse) && !(a < 0.f && b > 0.f));
        float cl = use_f ? a : c_lo[(long)d * n + j], cu = use_f ? b : c_hi[(long)d * n + j];
        intersect(l, u, cl, cu);
    }
    // pre-activation clamp of a ReLU split (constraints/lookups.rs:138-185); an emptied interval marks the domain
    if (sc > 0 && !isnan(l)) l = fmaxf(l, 0.f);
    if (sc < 0 && !isnan(u)) u = fminf(u, 0.f);
    if (sc != 0 && l > u) atomicOr(&dflags[d], kFlagInfeasible);
    t_lo[o] = l; t_hi[o] = u;
    if (!relu) { zl[o] = l; zu[o] = u; return; }
    // plain-CROWN relaxation (chord computed in binary64, slope and intercept stepped up)
    float ls, us, ui;
    if (isnan(l) || isnan(u) || ((isinf(l) || isinf(u)) && l < 0.f && u > 0.f)) {
        // the reference's closed forms for these arms all imply or enclose [-inf, +inf] for the domain
        atomicOr(&dflags[d], kFlagDegraded);
        ls = 0.f; us = 0.f; ui = 0.f;
    } else if (l >= 0.f) { ls = 1.f; us = 1.f; ui = 0.f; }
    else if (u <= 0.f) { ls = 0.f; us = 0.f; ui = 0.f; }
    else {
        double width = (double)u - (double)l;
        us = next_up32((float)((double)u / width));
        ui = next_up32((float)(-(double)us * (double)l));
        ls = (u > -l) ? 1.f : 0.f;
    }
    tab[o] = make_float4(ls, us, ui, 0.f);
    zabs[o] = fmaxf(fabsf(l), fabsf(u));
    // the next layer's input: relu of the tightened bound intersected with relu of the IBP bound
    // (crown_ibp_forward.rs:25-100); with a NaN anywhere in the vector the IBP one is kept
    float pl = fmaxf(il, 0.f), pu = fmaxf(iu, 0.f);
    if (isnan(il)) pl = il;
    if (isnan(iu)) pu = iu;
    if (!(fl & kNan)) {
        float ql = fmaxf(l, 0.f), qu = fmaxf(u, 0.f);
        intersect(pl, pu, ql, qu);
    }
    if (sc < 0) { pl = 0.f; pu = 0.f; }   // an inactive split: the output is zero whatever the interval arithmetic says
    zl[o] = pl; zu[o] = pu;
}

// Interval image of the specification rows: lo = C+ l + C- u (binary64 accumulation, outward slack and cast).
__global__ void k_spec_interval(int D, int S, int nL, const float *__restrict__ spec, const float *__restrict__ lo,
                                const float *__restrict__ hi, long stride, int off, float *__restrict__ out_lo,
                                float *__restrict__ out_hi) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= D * S) return;
    int d = t / S, s = t % S;
    const float *l = lo + (long)d * stride + off, *u = hi + (long)d * stride + off;
    double a = 0.0, b = 0.0, q = 0.0;
    for (int j = 0; j < nL; ++j) {
        double w = spec[s * nL + j];
        bool pos = w > 0.0;
        a = fma(w, pos ? (double)l[j] : (double)u[j], a);
        b = fma(w, pos ? (double)u[j] : (double)l[j], b);
        q = fma(fabs(w), fmax(fabs((double)l[j]), fabs((double)u[j])), q);
    }
    double slack = (double)(nL + 2) * 1.1102230246251565e-16 * 1.000001 * q;
    float lf = __double2float_rd(a - slack), hf = __double2float_ru(b + slack);
    if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
    out_lo[t] = lf; out_hi[t] = hf;
}

// Final merge of the specification rows: t = ibp n (f or c), result = c n t (t alone when c holds a NaN).
__global__ void k_crown_final(int D, int S, const float *__restrict__ ibp_lo, const float *__restrict__ ibp_hi,
                              const float *__restrict__ f_lo, const float *__restrict__ f_hi, float *__restrict__ c_lo,
                              float *__restrict__ c_hi, const int *__restrict__ dflags) {
    int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    if (dflags[d] & (kFlagDegraded | kFlagInvalid | kFlagInfeasible)) return;  // already widened by the concretisation
    int n_unst = 0;
    bool nan = false, cnan = false;
    for (int s = 0; s < S; ++s) {
        int o = d * S + s;
        if (f_lo[o] < 0.f && f_hi[o] > 0.f) ++n_unst;
    }
    bool sparse = false;
    if (n_unst > 0) {
        float stable_frac = 1.0f - ((float)n_unst / (float)S);
        if (!(stable_frac < 0.9f)) sparse = true;
    }
    for (int s = 0; s < S; ++s) {
        int o = d * S + s;
        bool use_f = sparse && !(f_lo[o] < 0.f && f_hi[o] > 0.f);
        float cl = use_f ? f_lo[o] : c_lo[o], cu = use_f ? f_hi[o] : c_hi[o];
        if (isnan(ibp_lo[o]) || isnan(ibp_hi[o]) || isnan(cl) || isnan(cu)) nan = true;
        if (isnan(c_lo[o]) || isnan(c_hi[o])) cnan = true;
    }
    for (int s = 0; s < S; ++s) {
        int o = d * S + s;
        float l = ibp_lo[o], u = ibp_hi[o];
        if (!nan) {
            bool use_f = sparse && !(f_lo[o] < 0.f && f_hi[o] > 0.f);
            intersect(l, u, use_f ? f_lo[o] : c_lo[o], use_f ? f_hi[o] : c_hi[o]);
        }
        float rl = c_lo[o], ru = c_hi[o];
        bool tnan = isnan(l) || isnan(u);
        if (cnan) { rl = l; ru = u; }
        else if (!tnan) intersect(rl, ru, l, u);
        c_lo[o] = rl; c_hi[o] = ru;
    }
}

// acc += the loose-domain counter the last concretisation left (word 4 of the min-lower block)
__global__ void k_accumulate_loose(const float *__restrict__ min_lower_block, int *__restrict__ acc) {
    if (threadIdx.x == 0 && blockIdx.x == 0) *acc += ((const int *)min_lower_block)[4];
}

}  // namespace

// Host-side split lists of a ReLU-split batch (multipliers are ignored: plain CROWN keeps them at zero).
struct CrownSplits {
    const nyb200_split *splits = nullptr;
    const int32_t *n_splits = nullptr;
    int max_splits = 0;
    int32_t *infeasible = nullptr;   // [D] out
};

static int crown_bounds_once(nyb200_engine *e, int net_id, const float *spec, int S, const float *in_lo,
                             const float *in_hi, int box_stride, int D, float *out_lo, float *out_hi, float *inter_lo,
                             float *inter_hi, int *loose_out, const CrownSplits *cs = nullptr) {
    Net *net;
    NYB_TRY(find_net(e, net_id, &net));
    const NetView &nv = net->v;
    if (D <= 0 || S <= 0) return set_err(e, NYB200_ERR_SHAPE, "D and S must be positive");
    if (box_stride != 0 && box_stride != nv.dims[0]) return set_err(e, NYB200_ERR_SHAPE, "box_stride must be 0 or dims[0]");
    const bool split = cs && cs->max_splits > 0;
    if (box_stride == 0 && D != 1 && !split) return set_err(e, NYB200_ERR_SHAPE, "a shared box is one domain: D must be 1");
    int max_rows = S;
    for (int k = 1; k < nv.L; ++k) max_rows = nv.dims[k] > max_rows ? nv.dims[k] : max_rows;
    if ((long)D * 2 * max_rows > 0x7fffffffL / 64) return set_err(e, NYB200_ERR_UNSUPPORTED, "batch too large for one call");
    const int L = nv.L;
    const long np = nv.nps;
    cudaStream_t st = e->stream;
    // the widest pass decides the workspace: allocate for it once
    Batch b;
    b.net_id = net_id; b.D = D; b.mode = 1; b.box_stride = box_stride; b.max_splits = split ? cs->max_splits : 0;
    b.S = max_rows; b.R = 2 * max_rows;
    BatchPtrs p;
    NYB_TRY(batch_ptrs(e, *net, b, p));
    e->batch = Batch();  // the resident batch's buffers are being reused
    NYB_WS(ibp_lo, float *, e, "ibp_lo", (size_t)D * np * 4);
    NYB_WS(ibp_hi, float *, e, "ibp_hi", (size_t)D * np * 4);
    NYB_WS(lflags, int *, e, "crown_flags", (size_t)D * 4);
    NYB_WS(loose_acc, int *, e, "crown_loose", 256);
    NYB_CUDA(e, cudaMemsetAsync(loose_acc, 0, 4, e->stream));
    NYB_WS(sp_ibp_lo, float *, e, "spec_ibp_lo", (size_t)D * S * 4);
    NYB_WS(sp_ibp_hi, float *, e, "spec_ibp_hi", (size_t)D * S * 4);
    NYB_WS(sp_f_lo, float *, e, "spec_f_lo", (size_t)D * S * 4);
    NYB_WS(sp_f_hi, float *, e, "spec_f_hi", (size_t)D * S * 4);
    size_t box = (size_t)nv.dims[0] * (box_stride ? (size_t)D : 1);
    NYB_CUDA(e, cudaMemcpyAsync(p.spec, spec, (size_t)S * nv.dims[L] * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.in_lo, in_lo, box * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.in_hi, in_hi, box * 4, cudaMemcpyHostToDevice, st));
    if (e->path == NYB200_PATH_TF32X3) {
        int *derr = (int *)ws_get(e, "umma_err", 256);
        if (!derr) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(derr, 0, 4, st));
    }
    if (split) {
        // the domains' split lists with their multipliers zeroed (plain CROWN carries none)
        std::vector<nyb200_split> sp((size_t)D * cs->max_splits);
        memcpy(sp.data(), cs->splits, sp.size() * sizeof(nyb200_split));
        for (auto &x : sp) x.beta = 0.f;
        NYB_CUDA(e, cudaMemcpyAsync(p.splits, sp.data(), sp.size() * sizeof(nyb200_split), cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(p.nsplits, cs->n_splits, (size_t)D * 4, cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaStreamSynchronize(st));   // sp is a local
    }
    // plain IBP of the whole network (also clears the per-domain flags and the split tables); with split lists, the
    // interval pass under the domains' clamps and no inherited bounds (mode 3)
    NYB_TRY(run_forward(e, *net, b, p, split ? 3 : 2));
    NYB_CUDA(e, cudaMemcpyAsync(ibp_lo, p.pre_lo, (size_t)D * np * 4, cudaMemcpyDeviceToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(ibp_hi, p.pre_hi, (size_t)D * np * 4, cudaMemcpyDeviceToDevice, st));

    for (int k = 0; k < L; ++k) {
        const int n = nv.dims[k + 1], off = nv.pre_off[k];
        const bool relu = k < L - 1;
        // f: forward image of the tightened input (layer 0 reads the box: f = ibp there)
        const float *zl = k == 0 ? p.in_lo : p.zl + nv.pre_off[k - 1], *zu = k == 0 ? p.in_hi : p.zu + nv.pre_off[k - 1];
        if (net->is_conv(k)) launch_ibp_conv(e, nv, net->geom[k], k, D, zl, zu, k == 0 ? (long)box_stride : np, p.raw_lo, p.raw_hi, p.q, np);
        else launch_ibp_linear(e, nv, k, D, zl, zu, k == 0 ? (long)box_stride : np, p.raw_lo, p.raw_hi, p.q, np);
        if (net->skip_of(k) >= 0)  // pre_k = W z + b + relu(pre_j): the identity branch joins with its tightened interval
            launch_skip_interval(e, D, n, np, p.raw_lo, p.raw_hi, off, p.zl, p.zu, nv.pre_off[net->skip_of(k)]);
        const float *c_lo = nullptr, *c_hi = nullptr;
        if (relu) {
            Batch bk = b;
            bk.S = n; bk.R = 2 * n;
            BatchPtrs pk;
            NYB_TRY(batch_ptrs(e, *net, bk, pk));
            if (e->error_channel == NYB200_ERRCH_REFERENCE) NYB_TRY(run_backward_ref(e, *net, bk, pk, k));
            else NYB_TRY(run_backward(e, *net, bk, pk, nullptr, 0, k));
            k_accumulate_loose<<<1, 32, 0, st>>>(pk.min_lower, loose_acc);
            e->launches++;
            c_lo = pk.out_lo; c_hi = pk.out_hi;
        }
        k_crown_flags<<<(unsigned)(((long)D * 32 + 255) / 256), 256, 0, st>>>(D, n, ibp_lo, ibp_hi, p.raw_lo, p.raw_hi, np, off,
                                                                             c_lo, c_hi, lflags);
        long tot = (long)D * n;
        k_crown_merge<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(D, n, off, np, relu ? 1 : 0, ibp_lo, ibp_hi, p.raw_lo,
                                                                   p.raw_hi, c_lo, c_hi, lflags, p.pre_lo, p.pre_hi, p.zl, p.zu,
                                                                   p.tab, p.zabs, p.flags, split ? p.code : nullptr);
        e->launches += 2;
    }
    // specification rows: IBP image, forward image of the tightened output, full backward pass, merge
    const int offL = nv.pre_off[L - 1];
    const unsigned gs = (unsigned)((D * S + 255) / 256);
    k_spec_interval<<<gs, 256, 0, st>>>(D, S, nv.dims[L], p.spec, ibp_lo, ibp_hi, np, offL, sp_ibp_lo, sp_ibp_hi);
    k_spec_interval<<<gs, 256, 0, st>>>(D, S, nv.dims[L], p.spec, p.pre_lo, p.pre_hi, np, offL, sp_f_lo, sp_f_hi);
    e->launches += 2;
    Batch bs = b;
    bs.S = S; bs.R = 2 * S;
    BatchPtrs ps;
    NYB_TRY(batch_ptrs(e, *net, bs, ps));
    if (e->error_channel == NYB200_ERRCH_REFERENCE) NYB_TRY(run_backward_ref(e, *net, bs, ps, -1));
    else {
        ps.keep_final = true;   // nyb200_crown_input_coeffs reads the final pass's input-level rows
        NYB_TRY(run_backward(e, *net, bs, ps, nullptr, 0, -1));
    }
    k_accumulate_loose<<<1, 32, 0, st>>>(ps.min_lower, loose_acc);
    e->launches++;
    k_crown_final<<<(unsigned)((D + 255) / 256), 256, 0, st>>>(D, S, sp_ibp_lo, sp_ibp_hi, sp_f_lo, sp_f_hi, ps.out_lo, ps.out_hi,
                                                              ps.flags);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaMemcpyAsync(out_lo, ps.out_lo, (size_t)D * S * 4, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaMemcpyAsync(out_hi, ps.out_hi, (size_t)D * S * 4, cudaMemcpyDeviceToHost, st));
    size_t w = (size_t)nv.n_pre * 4;
    if (inter_lo) NYB_CUDA(e, cudaMemcpy2DAsync(inter_lo, w, p.pre_lo, (size_t)np * 4, w, (size_t)D, cudaMemcpyDeviceToHost, st));
    if (inter_hi) NYB_CUDA(e, cudaMemcpy2DAsync(inter_hi, w, p.pre_hi, (size_t)np * 4, w, (size_t)D, cudaMemcpyDeviceToHost, st));
    int herr = 0;
    if (e->path == NYB200_PATH_TF32X3) {
        int *derr = (int *)ws_get(e, "umma_err", 256);
        if (derr) NYB_CUDA(e, cudaMemcpyAsync(&herr, derr, 4, cudaMemcpyDeviceToHost, st));
    }
    NYB_CUDA(e, cudaMemcpyAsync(loose_out, loose_acc, 4, cudaMemcpyDeviceToHost, st));
    if (split && cs->infeasible) NYB_CUDA(e, cudaMemcpyAsync(cs->infeasible, p.flags, (size_t)D * 4, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaStreamSynchronize(st));
    if (herr) return set_err(e, NYB200_ERR_INTERNAL, "tcgen05 pipeline wait expired (code " + std::to_string(herr) + ")");
    if (split && cs->infeasible) {
        for (int d = 0; d < D; ++d) {
            if (cs->infeasible[d] & kFlagInvalid) return set_err(e, NYB200_ERR_INVALID, "split entry out of range");
            cs->infeasible[d] = (cs->infeasible[d] & kFlagInfeasible) ? 1 : 0;
        }
    }
    e->batch.crown_a = ps.a_final;
    e->batch.crown_lda = ps.lda; e->batch.crown_D = D; e->batch.crown_S = S; e->batch.crown_n0 = nv.dims[0];
    return NYB200_OK;
}

// Input-level coefficient rows of the last plain-CROWN call: lower_a / upper_a [D x S x dims[0]] (either may be null).
int crown_input_coeffs(nyb200_engine *e, float *lower_a, float *upper_a) {
    const Batch &b = e->batch;
    if (!b.crown_a) return set_err(e, NYB200_ERR_INVALID, "no plain-CROWN result is held (another call has reused the workspace)");
    const size_t w = (size_t)b.crown_n0 * 4, pitch = (size_t)b.crown_lda * 4;
    for (int d = 0; d < b.crown_D; ++d) {
        const float *base = b.crown_a + (size_t)d * 2 * b.crown_S * b.crown_lda;
        if (lower_a)
            NYB_CUDA(e, cudaMemcpy2DAsync(lower_a + (size_t)d * b.crown_S * b.crown_n0, w, base, pitch, w, (size_t)b.crown_S,
                                          cudaMemcpyDeviceToHost, e->stream));
        if (upper_a)
            NYB_CUDA(e, cudaMemcpy2DAsync(upper_a + (size_t)d * b.crown_S * b.crown_n0, w, base + (size_t)b.crown_S * b.crown_lda,
                                          pitch, w, (size_t)b.crown_S, cudaMemcpyDeviceToHost, e->stream));
    }
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    return NYB200_OK;
}

// On the fast path, a pass whose rounding charge is visible at the refine tolerance (narrow boxes: bounds much
// smaller than the terms they are made of) sends the whole pipeline through the binary64 contractions once more,
// like the batch entry points do.
static int crown_bounds_cs(nyb200_engine *e, int net_id, const float *spec, int S, const float *in_lo, const float *in_hi,
                           int box_stride, int D, float *out_lo, float *out_hi, float *inter_lo, float *inter_hi,
                           const CrownSplits *cs) {
    if (e->error_channel == NYB200_ERRCH_REFERENCE) {
        // the reference's convention is a binary64 computation throughout (interval products included)
        const int saved = e->path;
        e->path = NYB200_PATH_F64;
        int loose_unused = 0;
        int st = crown_bounds_once(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi, &loose_unused, cs);
        e->path = saved;
        return st;
    }
    int loose = 0;
    NYB_TRY(crown_bounds_once(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi, &loose, cs));
    if (loose > 0 && e->path == NYB200_PATH_TF32X3 && e->refine_tol > 0.f) {
        e->path = NYB200_PATH_F64;
        int st = crown_bounds_once(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi, &loose, cs);
        e->path = NYB200_PATH_TF32X3;
        return st;
    }
    return NYB200_OK;
}

int crown_bounds(nyb200_engine *e, int net_id, const float *spec, int S, const float *in_lo, const float *in_hi,
                 int box_stride, int D, float *out_lo, float *out_hi, float *inter_lo, float *inter_hi) {
    return crown_bounds_cs(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi, nullptr);
}

int crown_bounds_split(nyb200_engine *e, int net_id, const float *spec, int S, const float *in_lo, const float *in_hi,
                       int box_stride, int D, float *out_lo, float *out_hi, float *inter_lo, float *inter_hi,
                       const nyb200_split *splits, const int32_t *n_splits, int max_splits, int32_t *infeasible) {
    CrownSplits cs;
    cs.splits = splits; cs.n_splits = n_splits; cs.max_splits = max_splits; cs.infeasible = infeasible;
    return crown_bounds_cs(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi, &cs);
}

}  // namespace nyb

extern "C" int32_t nyb200_crown_input_coeffs(nyb200_engine *e, float *lower_a, float *upper_a) {
    if (!e || (!lower_a && !upper_a)) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::crown_input_coeffs(e, lower_a, upper_a);
}

extern "C" int32_t nyb200_crown_bounds(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                                       const float *in_hi, int32_t box_stride, int32_t D, float *out_lo, float *out_hi,
                                       float *inter_lo, float *inter_hi) {
    if (!e || !spec || !in_lo || !in_hi || !out_lo || !out_hi) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    return nyb::crown_bounds(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi);
}

extern "C" int32_t nyb200_crown_bounds_split(nyb200_engine *e, int32_t net_id, const float *spec, int32_t S, const float *in_lo,
                                             const float *in_hi, int32_t box_stride, const nyb200_split *splits,
                                             const int32_t *n_splits, int32_t max_splits, int32_t D, float *out_lo,
                                             float *out_hi, float *inter_lo, float *inter_hi, int32_t *infeasible) {
    if (!e || !spec || !in_lo || !in_hi || !out_lo || !out_hi || !n_splits || !infeasible) return NYB200_ERR_INVALID;
    if (max_splits < 0 || (max_splits > 0 && !splits)) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    if (e->error_channel == NYB200_ERRCH_REFERENCE)
        return nyb::set_err(e, NYB200_ERR_UNSUPPORTED, "split domains are bounded in the default error convention");
    for (int d = 0; d < D; ++d)
        if (n_splits[d] < 0 || n_splits[d] > max_splits) return nyb::set_err(e, NYB200_ERR_INVALID, "n_splits out of range");
    if (max_splits == 0) {
        // no split anywhere: the plain pipeline (a shared box is then one domain)
        for (int d = 0; d < D; ++d) infeasible[d] = 0;
        return nyb::crown_bounds(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi);
    }
    return nyb::crown_bounds_split(e, net_id, spec, S, in_lo, in_hi, box_stride, D, out_lo, out_hi, inter_lo, inter_hi, splits,
                                   n_splits, max_splits, infeasible);
}
