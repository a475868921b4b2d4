// Reference-shaped entry points: the calls a binding of ny's GpuCrownBackward / GemmEngine traits makes with the
// operands those traits pass - layer lists in BACKWARD order (output -> input, as
// crates/ny-cuda/src/sound_crown.rs:1159-1260 walks them) whose Activation members carry relaxation slopes the
// CALLER baked, per-domain signed multipliers and abs-max tables - instead of split lists from which this engine
// derives the relaxation itself.  They are host adapters over the kernels of the batch calls:
//   nyb200_crown_backward              crown_backward_gpu_sound / _seeded_sound (crates/ny-core/src/gemm.rs:3357, 3387)
//   nyb200_crown_resnet_beta_batched   crown_backward_gpu_resnet_sound_beta_batched (gemm.rs:3944)
//   nyb200_crown_resnet_beta_batched_adam  ..._beta_batched_adam (gemm.rs:4042, GpuBetaAdamConfig :2960-2993)
//   nyb200_gemm_f64_triplet            GemmEngine::gemm_f64_triplet (gemm.rs:523)
// The layer weights are cached on the device under a key made of their host address, shape and a 64-bit hash of
// their contents (the reference keys its residency cache on Arc pointer identity, gemm.rs:568-578; a C caller
// cannot pin an allocation, so the contents are part of the key); nyb200_clear_working_set drops the cache.
#include <string.h>

#include "nyb200_internal.cuh"

namespace nyb {

namespace {

uint64_t fnv1a(const void *p, size_t bytes, uint64_t h) {
    const unsigned char *c = (const unsigned char *)p;
    // eight bytes per step: the hash only has to tell weight tensors apart, not resist an adversary
    size_t i = 0;
    for (; i + 8 <= bytes; i += 8) {
        uint64_t w;
        memcpy(&w, c + i, 8);
        h = (h ^ w) * 1099511628211ull;
    }
    for (; i < bytes; ++i) h = (h ^ c[i]) * 1099511628211ull;
    return h;
}

struct Parsed {
    std::vector<const nyb200_crown_layer *> lin;  // forward order
    std::vector<const nyb200_crown_layer *> act;  // act[k] follows lin[k] (forward order), size lin.size() - 1
    const nyb200_crown_layer *lead_act = nullptr;  // seeded lists may open with the Activation that follows lin.back()
};

// Backward-order list: Linear (Activation Linear)*; a seeded suffix may open with an Activation (the frontier then
// sits behind that activation).  Anything else is a decline.
int parse_layers(nyb200_engine *e, const nyb200_crown_layer *layers, int n_layers, Parsed &out, bool seeded = false) {
    const bool lead = seeded && n_layers >= 2 && (n_layers & 1) == 0 &&
                      (layers[0].kind == NYB200_CROWN_ACTIVATION || layers[0].kind == NYB200_CROWN_RELU_DUAL_ALPHA);
    if (n_layers < 1 || (!lead && (n_layers & 1) == 0)) return set_err(e, NYB200_ERR_UNSUPPORTED, "layer list must be Linear (Activation Linear)* in backward order");
    std::vector<const nyb200_crown_layer *> lin_b, act_b;
    for (int i = 0; i < n_layers; ++i) {
        const nyb200_crown_layer &l = layers[i];
        if (((i + (lead ? 1 : 0)) & 1) == 0) {
            if (l.kind == NYB200_CROWN_CONV2D) return set_err(e, NYB200_ERR_UNSUPPORTED, "Conv2d members are declined by the reference-shaped entry points; register the network and use the batch calls");
            if (l.kind != NYB200_CROWN_LINEAR) return set_err(e, NYB200_ERR_UNSUPPORTED, "expected a Linear layer");
            if (!l.weight || l.out_features <= 0 || l.in_features <= 0) return set_err(e, NYB200_ERR_SHAPE, "Linear layer without weights or with a non-positive size");
            lin_b.push_back(&l);
        } else {
            if (l.kind != NYB200_CROWN_ACTIVATION && l.kind != NYB200_CROWN_RELU_DUAL_ALPHA) return set_err(e, NYB200_ERR_UNSUPPORTED, "expected an Activation layer");
            if (!l.lower_slope || !l.upper_slope || !l.upper_intercept || l.num_neurons <= 0) return set_err(e, NYB200_ERR_SHAPE, "Activation layer without its slope tables");
            if (l.kind == NYB200_CROWN_RELU_DUAL_ALPHA && !l.upper_neg_slope) return set_err(e, NYB200_ERR_SHAPE, "dual-alpha Activation without upper_neg_slope");
            act_b.push_back(&l);
        }
    }
    if (lead) {
        out.lead_act = act_b.front();
        act_b.erase(act_b.begin());
        if (out.lead_act->num_neurons != lin_b.front()->out_features) return set_err(e, NYB200_ERR_SHAPE, "leading Activation width differs from the layer it follows");
    }
    out.lin.assign(lin_b.rbegin(), lin_b.rend());
    out.act.assign(act_b.rbegin(), act_b.rend());
    for (size_t k = 0; k + 1 < out.lin.size(); ++k) {
        if (out.lin[k]->out_features != out.lin[k + 1]->in_features) return set_err(e, NYB200_ERR_SHAPE, "layer widths do not chain");
        if (out.act[k]->num_neurons != out.lin[k]->out_features) return set_err(e, NYB200_ERR_SHAPE, "Activation width differs from the layer it follows");
    }
    return NYB200_OK;
}

// The registered network for these weights (created and cached on first sight).
int net_for(nyb200_engine *e, const Parsed &P, int *net_id) {
    uint64_t h = 1469598103934665603ull;
    for (const nyb200_crown_layer *l : P.lin) {
        const uintptr_t wp = (uintptr_t)l->weight, bp = (uintptr_t)l->bias;
        h = fnv1a(&wp, sizeof(wp), h); h = fnv1a(&bp, sizeof(bp), h);
        h = fnv1a(&l->out_features, 4, h); h = fnv1a(&l->in_features, 4, h);
        h = fnv1a(l->weight, (size_t)l->out_features * l->in_features * 4, h);
        if (l->bias) h = fnv1a(l->bias, (size_t)l->out_features * 4, h);
    }
    auto it = e->boundary_nets.find(h);
    if (it != e->boundary_nets.end() && e->nets.count(it->second)) { *net_id = it->second; return NYB200_OK; }
    const int L = (int)P.lin.size();
    std::vector<int32_t> dims((size_t)L + 1), hb((size_t)L);
    std::vector<float> w, b;
    dims[0] = P.lin[0]->in_features;
    for (int k = 0; k < L; ++k) {
        const nyb200_crown_layer *l = P.lin[k];
        dims[k + 1] = l->out_features;
        hb[k] = l->bias ? 1 : 0;
        w.insert(w.end(), l->weight, l->weight + (size_t)l->out_features * l->in_features);
        if (l->bias) b.insert(b.end(), l->bias, l->bias + l->out_features);
    }
    std::vector<nyb200_layer_desc> ld((size_t)L);
    for (int k = 0; k < L; ++k) {
        memset(&ld[k], 0, sizeof(ld[k]));
        ld[k].kind = NYB200_LAYER_LINEAR; ld[k].in_features = dims[k]; ld[k].out_features = dims[k + 1]; ld[k].has_bias = hb[k];
    }
    int id = 0;
    NYB_TRY(create_net(e, L, ld.data(), w.data(), b.empty() ? nullptr : b.data(), &id));
    e->boundary_nets[h] = id;
    *net_id = id;
    return NYB200_OK;
}

}  // namespace

}  // namespace nyb

using namespace nyb;

extern "C" {

int32_t nyb200_crown_backward(nyb200_engine *e, const nyb200_crown_layer *layers, int32_t n_layers, const float *spec,
                              int32_t num_specs, const nyb200_crown_seed *seed, const float *in_lo, const float *in_hi,
                              float *out_lo, float *out_hi) {
    if (!e || !layers || !in_lo || !in_hi || !out_lo || !out_hi || (!spec && !seed)) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    Parsed P;
    NYB_TRY(parse_layers(e, layers, n_layers, P, seed != nullptr));
    const int L = (int)P.lin.size();
    const int S = seed ? seed->num_specs : num_specs;
    const int top = P.lin[L - 1]->out_features;
    if (S <= 0) return set_err(e, NYB200_ERR_SHAPE, "num_specs must be positive");
    if (seed && (seed->current_dim != top || !seed->lower_a || !seed->upper_a)) return set_err(e, NYB200_ERR_SHAPE, "seed width differs from the first layer's output");
    int net_id = 0;
    NYB_TRY(net_for(e, P, &net_id));
    Net *net;
    NYB_TRY(find_net(e, net_id, &net));
    const NetView &nv = net->v;
    Batch b;
    b.net_id = net_id; b.S = S; b.R = 2 * S; b.D = 1; b.mode = 1; b.box_stride = 0; b.max_splits = 0;
    BatchPtrs p;
    NYB_TRY(batch_ptrs(e, *net, b, p));
    e->batch = Batch();
    cudaStream_t st = e->stream;
    // relaxation tables as the caller baked them: (lower slope, upper slope, upper intercept, lower intercept)
    std::vector<float4> tab((size_t)nv.nps, make_float4(0.f, 0.f, 0.f, 0.f));
    for (int k = 0; k < L; ++k) {
        const nyb200_crown_layer *a = k + 1 < L ? P.act[k] : P.lead_act;
        if (!a) continue;
        for (int j = 0; j < a->num_neurons; ++j) {
            const float li = a->lower_intercept ? a->lower_intercept[j] : 0.f;
            if (a->kind == NYB200_CROWN_RELU_DUAL_ALPHA && a->upper_neg_slope[j] != a->lower_slope[j])
                return set_err(e, NYB200_ERR_UNSUPPORTED, "distinct upper-path slopes are served by the batch optimisation (objective 2), not by this entry point");
            tab[(size_t)nv.pre_off[k] + j] = make_float4(a->lower_slope[j], a->upper_slope[j], a->upper_intercept[j], li);
        }
    }
    for (const float4 &t : tab)
        if (!(std::isfinite(t.x) && std::isfinite(t.y) && std::isfinite(t.z) && std::isfinite(t.w))) return set_err(e, NYB200_ERR_NUMERICAL, "non-finite relaxation table entry");
    NYB_CUDA(e, cudaMemcpyAsync(p.tab, tab.data(), (size_t)nv.nps * 16, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.in_lo, in_lo, (size_t)nv.dims[0] * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.in_hi, in_hi, (size_t)nv.dims[0] * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemsetAsync(p.flags, 0, 4, st));
    RefSeed rs;
    if (seed) {
        NYB_WS(sla, float *, e, "seed_la", (size_t)S * top * 4);
        NYB_WS(sua, float *, e, "seed_ua", (size_t)S * top * 4);
        NYB_WS(sb, float *, e, "seed_b", (size_t)2 * S * 4);
        NYB_CUDA(e, cudaMemcpyAsync(sla, seed->lower_a, (size_t)S * top * 4, cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(sua, seed->upper_a, (size_t)S * top * 4, cudaMemcpyHostToDevice, st));
        std::vector<float> hb((size_t)2 * S, 0.f);
        if (seed->lower_b) memcpy(hb.data(), seed->lower_b, (size_t)S * 4);
        if (seed->upper_b) memcpy(hb.data() + S, seed->upper_b, (size_t)S * 4);
        NYB_CUDA(e, cudaMemcpyAsync(sb, hb.data(), (size_t)2 * S * 4, cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaStreamSynchronize(st));  // hb is a local
        rs.lower_a = sla; rs.upper_a = sua; rs.bias = sb; rs.relu_first = P.lead_act != nullptr;
    } else {
        NYB_CUDA(e, cudaMemcpyAsync(p.spec, spec, (size_t)S * top * 4, cudaMemcpyHostToDevice, st));
    }
    NYB_TRY(run_backward_ref(e, *net, b, p, -1, seed ? &rs : nullptr));
    NYB_CUDA(e, cudaMemcpyAsync(out_lo, p.out_lo, (size_t)S * 4, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaMemcpyAsync(out_hi, p.out_hi, (size_t)S * 4, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaStreamSynchronize(st));
    return NYB200_OK;
}

static int upload_domains(nyb200_engine *e, const nyb200_domain_ref *domains, int32_t D, const float *spec, int32_t num_specs,
                          Net **net_out, BatchPtrs &p, bool want_splits) {
    if (D <= 0 || num_specs <= 0) return set_err(e, NYB200_ERR_SHAPE, "D and num_specs must be positive");
    Parsed P0;
    NYB_TRY(parse_layers(e, domains[0].layers, domains[0].n_layers, P0));
    const int L = (int)P0.lin.size();
    int net_id = 0;
    NYB_TRY(net_for(e, P0, &net_id));
    Net *net;
    NYB_TRY(find_net(e, net_id, &net));
    const NetView &nv = net->v;
    if (P0.lin[L - 1]->out_features != nv.dims[L]) return set_err(e, NYB200_ERR_INTERNAL, "cached network shape");
    int max_splits = 0;
    for (int d = 0; d < D && want_splits; ++d) max_splits = domains[d].n_splits > max_splits ? domains[d].n_splits : max_splits;
    Batch b;
    b.net_id = net_id; b.S = num_specs; b.R = 2 * num_specs; b.D = D; b.mode = 1; b.box_stride = nv.dims[0]; b.max_splits = max_splits;
    b.has_alpha = false;
    NYB_TRY(batch_ptrs(e, *net, b, p));
    const size_t np = (size_t)nv.nps, n0 = (size_t)nv.dims[0];
    std::vector<float4> tab((size_t)D * np, make_float4(0.f, 0.f, 0.f, 0.f));
    std::vector<float> zabs((size_t)D * np, 0.f), lo((size_t)D * n0), hi((size_t)D * n0), pre_lo((size_t)D * np, 0.f), pre_hi((size_t)D * np, 0.f);
    std::vector<signed char> code((size_t)D * np, 0);
    std::vector<nyb200_split> splits((size_t)D * (size_t)(max_splits > 0 ? max_splits : 1));
    std::vector<int> ns((size_t)D, 0);
    for (int d = 0; d < D; ++d) {
        const nyb200_domain_ref &dr = domains[d];
        if (!dr.layers || !dr.input_lower || !dr.input_upper || !dr.node_abs) return set_err(e, NYB200_ERR_INVALID, "domain without layers, box or node_abs");
        Parsed P;
        if (d == 0) P = P0;
        else {
            NYB_TRY(parse_layers(e, dr.layers, dr.n_layers, P));
            if ((int)P.lin.size() != L) return set_err(e, NYB200_ERR_SHAPE, "domains of one batch must share the network");
            for (int k = 0; k < L; ++k)  // the weights are shared: same tensors (gemm.rs:2925-2931)
                if (P.lin[k]->weight != P0.lin[k]->weight || P.lin[k]->bias != P0.lin[k]->bias || P.lin[k]->out_features != P0.lin[k]->out_features)
                    return set_err(e, NYB200_ERR_INVALID, "heterogeneous batch: every domain must reference the same weight tensors");
        }
        memcpy(&lo[(size_t)d * n0], dr.input_lower, n0 * 4);
        memcpy(&hi[(size_t)d * n0], dr.input_upper, n0 * 4);
        for (int k = 0; k + 1 < L; ++k) {
            // fold order = backward order: Activation r of the fold belongs to forward layer L - 2 - r
            const int fold = L - 2 - k;
            const nyb200_crown_layer *a = P.act[k];
            const float *sb = dr.beta_signed ? dr.beta_signed[fold] : nullptr;
            const float *na = dr.node_abs[fold];
            if (!na) return set_err(e, NYB200_ERR_INVALID, "node_abs entry missing");
            for (int j = 0; j < a->num_neurons; ++j) {
                if (a->lower_intercept && a->lower_intercept[j] != 0.f) return set_err(e, NYB200_ERR_UNSUPPORTED, "non-zero lower intercepts are served by nyb200_crown_backward only");
                const size_t o = (size_t)d * np + (size_t)nv.pre_off[k] + j;
                const float beta = (sb && std::isfinite(sb[j])) ? sb[j] : 0.f;   // non-finite multipliers are skipped (relu_backward.rs:156-173)
                const float4 t = make_float4(a->lower_slope[j], a->upper_slope[j], a->upper_intercept[j], beta);
                if (!(std::isfinite(t.x) && std::isfinite(t.y) && std::isfinite(t.z) && std::isfinite(na[j]) && na[j] >= 0.f))
                    return set_err(e, NYB200_ERR_NUMERICAL, "non-finite relaxation table or abs-max entry: the batch is refused as a whole");
                tab[o] = t;
                zabs[o] = na[j];
                // the optimiser classifies neurons by their interval: any interval consistent with the baked line
                const bool unstable = !(t.y == 1.f && t.z == 0.f) && !(t.y == 0.f && t.z == 0.f);
                pre_lo[o] = unstable ? -na[j] : (t.y == 1.f ? 0.f : -na[j]);
                pre_hi[o] = unstable ? na[j] : (t.y == 1.f ? na[j] : 0.f);
            }
        }
        if (want_splits) {
            ns[d] = dr.n_splits;
            for (int q = 0; q < dr.n_splits; ++q) {
                nyb200_split s = dr.splits[q];
                if (s.relu < 0 || s.relu >= L - 1 || s.neuron < 0 || s.neuron >= nv.dims[s.relu + 1] || (s.sign != 1 && s.sign != -1))
                    return set_err(e, NYB200_ERR_INVALID, "split mapping entry out of range");
                splits[(size_t)d * max_splits + q] = s;
                code[(size_t)d * np + (size_t)nv.pre_off[s.relu] + s.neuron] = (signed char)s.sign;
            }
        }
    }
    cudaStream_t st = e->stream;
    NYB_CUDA(e, cudaMemcpyAsync(p.spec, spec, (size_t)num_specs * nv.dims[L] * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.in_lo, lo.data(), lo.size() * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.in_hi, hi.data(), hi.size() * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.tab, tab.data(), tab.size() * 16, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.zabs, zabs.data(), zabs.size() * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.pre_lo, pre_lo.data(), pre_lo.size() * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.pre_hi, pre_hi.data(), pre_hi.size() * 4, cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.code, code.data(), code.size(), cudaMemcpyHostToDevice, st));
    NYB_CUDA(e, cudaMemsetAsync(p.flags, 0, (size_t)D * 4, st));
    if (max_splits > 0) {
        NYB_CUDA(e, cudaMemcpyAsync(p.splits, splits.data(), splits.size() * sizeof(nyb200_split), cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(p.nsplits, ns.data(), (size_t)D * 4, cudaMemcpyHostToDevice, st));
    }
    // q = |W_k| max|z_{k-1}|, the weights of the rounding charge: from the box for the first layer, from the previous
    // ReLU's abs-max table (its post-activation magnitude is at most that) for the others
    for (int k = 0; k < L; ++k) {
        const float *zl = k == 0 ? p.in_lo : p.zabs + nv.pre_off[k - 1];
        const float *zu = k == 0 ? p.in_hi : p.zabs + nv.pre_off[k - 1];
        launch_ibp_linear(e, nv, k, D, zl, zu, k == 0 ? (long)n0 : (long)np, p.raw_lo, p.raw_hi, p.q, (long)np);
    }
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaStreamSynchronize(st));  // the staging vectors are locals
    b.valid = true;
    b.external_tables = true;
    e->batch = b;
    *net_out = net;
    return NYB200_OK;
}

int32_t nyb200_crown_resnet_beta_batched(nyb200_engine *e, const nyb200_domain_ref *domains, int32_t D, const float *spec,
                                         int32_t num_specs, float *out_lo, float *out_hi) {
    if (!e || !domains || !spec || !out_lo || !out_hi) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    Net *net;
    BatchPtrs p;
    NYB_TRY(upload_domains(e, domains, D, spec, num_specs, &net, p, false));
    int *derr = nullptr;
    if (e->path == NYB200_PATH_TF32X3) {
        derr = (int *)ws_get(e, "umma_err", 256);
        if (!derr) return NYB200_ERR_OOM;
        NYB_CUDA(e, cudaMemsetAsync(derr, 0, 4, e->stream));
    }
    NYB_TRY(run_backward(e, *net, e->batch, p, nullptr, 0));
    e->batch.ran = true; e->batch.finished = false; e->batch.optimized = false; e->batch.refined = 0;
    int herr = 0, loose = 0;
    if (derr) {
        NYB_CUDA(e, cudaMemcpyAsync(&herr, derr, 4, cudaMemcpyDeviceToHost, e->stream));
        NYB_CUDA(e, cudaMemcpyAsync(&loose, (int *)p.min_lower + 4, 4, cudaMemcpyDeviceToHost, e->stream));
    }
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    if (herr) return set_err(e, NYB200_ERR_INTERNAL, "tcgen05 pipeline wait expired (code " + std::to_string(herr) + ")");
    if (loose > 0 && e->refine_tol > 0.f) {
        // a visible rounding charge: the same tables once more with binary64 contractions
        const int saved = e->path;
        e->path = NYB200_PATH_F64;
        int st = run_backward(e, *net, e->batch, p, nullptr, 0);
        e->path = saved;
        NYB_TRY(st);
        e->batch.refined = loose;
    }
    e->batch.finished = true;
    const size_t n = (size_t)D * num_specs;
    NYB_CUDA(e, cudaMemcpyAsync(out_lo, p.out_lo, n * 4, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaMemcpyAsync(out_hi, p.out_hi, n * 4, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    return NYB200_OK;
}

int32_t nyb200_crown_resnet_beta_batched_adam(nyb200_engine *e, const nyb200_domain_ref *domains, int32_t D, const float *spec,
                                              int32_t num_specs, const nyb200_beta_adam_config *cfg, float *out_lo,
                                              float *out_hi, float *out_beta, int32_t max_splits) {
    if (!e || !domains || !spec || !cfg || !out_lo || !out_hi) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    if (cfg->iterations < 1 || !(cfg->beta_lr > 0.f) || !(cfg->tolerance >= 0.f)) return set_err(e, NYB200_ERR_INVALID, "GpuBetaAdamConfig: iterations >= 1, beta_lr > 0, tolerance >= 0");
    Net *net;
    BatchPtrs p;
    NYB_TRY(upload_domains(e, domains, D, spec, num_specs, &net, p, true));
    nyb200_opt_config oc;
    memset(&oc, 0, sizeof(oc));
    oc.iterations = cfg->iterations; oc.lr_alpha = 0.f; oc.lr_beta = cfg->beta_lr; oc.lr_decay = 1.f;
    oc.beta1 = cfg->beta1; oc.beta2 = cfg->beta2; oc.epsilon = cfg->epsilon; oc.clip_beta = 0.f;
    oc.objective = 0; oc.rule = 2 /* AMSGrad second moments, gemm.rs:2955-2958 */; oc.tolerance = cfg->tolerance;
    NYB_TRY(optimize_batch(e, oc));
    NYB_TRY(finish_batch_public(e));
    const size_t n = (size_t)D * num_specs;
    NYB_CUDA(e, cudaMemcpyAsync(out_lo, p.out_lo, n * 4, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaMemcpyAsync(out_hi, p.out_hi, n * 4, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    if (out_beta) {
        if (max_splits < e->batch.max_splits) return set_err(e, NYB200_ERR_SHAPE, "out_beta is narrower than the longest split list");
        std::vector<float> tmp((size_t)D * (size_t)(e->batch.max_splits > 0 ? e->batch.max_splits : 1));
        NYB_TRY(download_params(e, nullptr, e->batch.max_splits > 0 ? tmp.data() : nullptr));
        for (int d = 0; d < D; ++d)
            for (int q = 0; q < max_splits; ++q) out_beta[(size_t)d * max_splits + q] = q < e->batch.max_splits ? tmp[(size_t)d * e->batch.max_splits + q] : 0.f;
    }
    return NYB200_OK;
}

int32_t nyb200_gemm_f64_triplet(nyb200_engine *e, int32_t m, int32_t k, int32_t n, const double *const a[3],
                                const double *const b[3], double *const c_out[3]) {
    if (!e || !a || !b || !c_out) return NYB200_ERR_INVALID;
    for (int i = 0; i < 3; ++i) if (!a[i] || !b[i] || !c_out[i]) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    if (m <= 0 || k <= 0 || n <= 0) return set_err(e, NYB200_ERR_SHAPE, "gemm_f64_triplet: non-positive dimension");
    NYB_CUDA(e, cudaSetDevice(e->device));
    NYB_DEADLINE(e, "binary64 product triplet");
    const size_t na = (size_t)m * k, nb = (size_t)k * n, nc = (size_t)m * n;
    NYB_WS(da, double *, e, "gemm3_a", 3 * na * 8);
    NYB_WS(db, double *, e, "gemm3_b", 3 * nb * 8);
    NYB_WS(dc, double *, e, "gemm3_c", 3 * nc * 8);
    // the three products are queued on one stream and synchronised once; an operand that repeats (the sound CROWN
    // triplet shares |W| between its second and third product) is uploaded once
    for (int i = 0; i < 3; ++i) {
        int same_a = -1, same_b = -1;
        for (int j = 0; j < i; ++j) { if (a[j] == a[i]) same_a = j; if (b[j] == b[i]) same_b = j; }
        const double *pa = same_a >= 0 ? da + same_a * na : da + i * na;
        const double *pb = same_b >= 0 ? db + same_b * nb : db + i * nb;
        if (same_a < 0) NYB_CUDA(e, cudaMemcpyAsync(da + i * na, a[i], na * 8, cudaMemcpyHostToDevice, e->stream));
        if (same_b < 0) NYB_CUDA(e, cudaMemcpyAsync(db + i * nb, b[i], nb * 8, cudaMemcpyHostToDevice, e->stream));
        launch_dgemm(e, m, n, k, pa, pb, dc + i * nc);
        NYB_CUDA(e, cudaMemcpyAsync(c_out[i], dc + i * nc, nc * 8, cudaMemcpyDeviceToHost, e->stream));
    }
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    return NYB200_OK;
}

}  // extern "C"
