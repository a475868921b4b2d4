// Device-resident BaB frontier: the open domain set of a ReLU-split branch-and-bound search lives on the GPU as a
// ring of split histories, and one call per round pops a batch, bounds it, decides every domain, picks the split
// neuron of every open one and appends both children - what BetaCrownVerifier's loop does between engine calls
// (crates/ny-propagate/src/beta_crown/engine/core.rs:492-735: pop batch, bound, prune verified / infeasible, branch,
// push children) without the split lists ever visiting the host.  The order is the host loop's: batches leave from
// the front, the children of the open domains are appended at the back in domain order, active child first, so a
// search run through this file bounds exactly the domains the host loop (ny_b200/bab.py) bounds.
//
// One bound per domain with the multipliers at zero (the reference's throughput default, beta_iterations = 0); the
// optimising search with warm starts stays on the host loop.
#include <cstring>
#include <vector>

#include "nyb200_internal.cuh"

namespace nyb {

constexpr int kMaxRowsF = 64;

struct ResidentFrontier {
    int net_id = -1, S = 0, maxd = 0, n_clauses = 0;
    long cap = 0, head = 0, count = 0;
    nyb200_split *buf = nullptr;   // [cap x maxd]
    int *ns = nullptr;             // [cap]
    int *stats = nullptr;          // device: open, verified, infeasible, stuck, (float) min lower
    float *thr = nullptr;          // device [S]
    int *owner = nullptr;          // device [S]
    float *consts = nullptr;       // device copies of spec, box and inherited bounds, back to back
    size_t n_spec = 0, n_box = 0, n_inh = 0;
    long bounded = 0;
    // warm starts of the optimising search: one row of slopes per ring slot [cap x nps], allocated by the first
    // optimising round.  The first no_alpha_front records (counted from the front) have no slopes of their own (the
    // root, records that arrived from outside, children of a round that did not optimise); every record behind has.
    float *alpha = nullptr;
    long no_alpha_front = 0;
    size_t buf_bytes = 0, ns_bytes = 0, thr_bytes = 0, consts_bytes = 0, alpha_bytes = 0;   // what the arrays can hold
    bool optimistic = true;   // queue the decisions behind the bound without waiting (until a round is flagged)
    bool verdict_refinement = false;   // nyb200_frontier_set_refinement
};

void frontier_free(ResidentFrontier *f) {
    if (!f) return;
    cudaFree(f->buf); cudaFree(f->ns); cudaFree(f->stats); cudaFree(f->thr); cudaFree(f->owner); cudaFree(f->consts);
    cudaFree(f->alpha);
    delete f;
}

namespace {

// done[d] = 1 when the domain needs no children: infeasible, or every clause of the violation has a row whose lower
// bound is above its threshold (strictly: the verdict predicate of beta_crown/config/tests.rs).  NaN never verifies.
__global__ void k_frontier_decide(int D, int S, int n_clauses, const float *__restrict__ out_lo, const int *__restrict__ flags,
                                  const float *__restrict__ thr, const int *__restrict__ owner, int *__restrict__ done,
                                  int *__restrict__ stats) {
    int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const int fl = flags[d];
    if (fl & kFlagInfeasible) { done[d] = 1; atomicAdd(&stats[2], 1); return; }
    unsigned refuted = 0;
    float m = INFINITY;
    for (int s = 0; s < S; ++s) {
        const float l = out_lo[(long)d * S + s];
        if (l > thr[s]) refuted |= 1u << owner[s];
        m = fminf(m, l);
    }
    const bool verified = refuted == (n_clauses >= 32 ? 0xffffffffu : ((1u << n_clauses) - 1u));
    done[d] = verified ? 1 : 0;
    if (verified) atomicAdd(&stats[1], 1);
    // global lower bound over feasible domains (float bits as ordered integers: the values are compared as floats
    // by the host from the per-round minimum the concretisation already keeps; this one is per search round)
    if (!isnan(m)) {
        int *p = &stats[4];
        int old = *p;
        while (__int_as_float(old) > m) {
            int prev = atomicCAS(p, old, __float_as_int(m));
            if (prev == old) break;
            old = prev;
        }
    }
}

// Exclusive scan of the open flags (single block, D <= 1 << 16), the number of open domains and of stuck ones
// (undecided, but no neuron left to split).
__global__ void k_frontier_scan(int D, const int *__restrict__ done, const int *__restrict__ relu, const int *__restrict__ pns,
                                int *__restrict__ pos, int *__restrict__ stats) {
    __shared__ int part[1024];
    const int t = threadIdx.x, per = (D + 1023) / 1024;
    const int b0 = t * per, b1 = min(D, b0 + per);
    int c = 0, stuck = 0, deep = 0;
    for (int d = b0; d < b1; ++d) {
        const bool open = !done[d];
        if (open && relu[d] >= 0) ++c;
        if (open && relu[d] < 0) ++stuck;
        deep = max(deep, pns[d]);
    }
    if (deep) atomicMax(&stats[5], deep);   // longest split history in the batch
    part[t] = c;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {   // Hillis-Steele inclusive scan
        int v = t >= o ? part[t - o] : 0;
        __syncthreads();
        part[t] += v;
        __syncthreads();
    }
    int run = part[t] - c;
    for (int d = b0; d < b1; ++d) {
        const bool open = !done[d] && relu[d] >= 0;
        pos[d] = open ? run : -1;
        if (open) ++run;
    }
    if (stuck) atomicAdd(&stats[3], stuck);
    if (t == 1023) stats[0] = part[1023];
}

// Both children of every open domain: the parent's history with the new split appended (multiplier 0), the active
// child at ring slot tail + 2 pos, the inactive one behind it.
__global__ void k_frontier_children(int D, int maxd, long cap, long tail, const nyb200_split *__restrict__ psplits,
                                    const int *__restrict__ pns, const int *__restrict__ pos, const int *__restrict__ relu,
                                    const int *__restrict__ neuron, nyb200_split *__restrict__ buf, int *__restrict__ ns) {
    const int d = blockIdx.x;
    if (d >= D || pos[d] < 0) return;
    const int n = pns[d];
    const long s0 = (tail + 2L * pos[d]) % cap, s1 = (tail + 2L * pos[d] + 1) % cap;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        nyb200_split r = psplits[(long)d * maxd + i];
        r.beta = 0.f;
        buf[s0 * maxd + i] = r;
        buf[s1 * maxd + i] = r;
    }
    if (threadIdx.x == 0) {
        nyb200_split r;
        r.relu = relu[d]; r.neuron = neuron[d]; r.sign = 1; r.beta = 0.f;
        buf[s0 * maxd + n] = r;
        r.sign = -1;
        buf[s1 * maxd + n] = r;
        ns[s0] = n + 1; ns[s1] = n + 1;
    }
}

// The same for the optimising search: the parent's records carry its optimised multipliers (|signed beta| of the
// relaxation table, beta_crown/state/beta.rs warm start), the new split starts at 0, and both children inherit the
// parent's optimised slopes (the table's lower slopes) in their slots of the slope ring.
__global__ void k_frontier_children_warm(NetView nv, int D, int maxd, long cap, long tail, const nyb200_split *__restrict__ psplits,
                                         const int *__restrict__ pns, const int *__restrict__ pos, const int *__restrict__ relu,
                                         const int *__restrict__ neuron, const float4 *__restrict__ tab,
                                         nyb200_split *__restrict__ buf, int *__restrict__ ns, float *__restrict__ alpha) {
    const int d = blockIdx.x;
    if (d >= D || pos[d] < 0) return;
    const int n = pns[d];
    const long s0 = (tail + 2L * pos[d]) % cap, s1 = (tail + 2L * pos[d] + 1) % cap;
    const float4 *t = tab + (long)d * nv.nps;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        nyb200_split r = psplits[(long)d * maxd + i];
        float b = 0.f;
        if (r.relu >= 0 && r.relu < nv.L - 1 && r.neuron >= 0 && r.neuron < nv.dims[r.relu + 1]) b = fabsf(t[nv.pre_off[r.relu] + r.neuron].w);
        r.beta = b;
        buf[s0 * maxd + i] = r;
        buf[s1 * maxd + i] = r;
    }
    for (long j = threadIdx.x; j < nv.nps; j += blockDim.x) {
        const float a = j < nv.n_pre ? t[j].x : 0.f;
        alpha[s0 * nv.nps + j] = a;
        alpha[s1 * nv.nps + j] = a;
    }
    if (threadIdx.x == 0) {
        nyb200_split r;
        r.relu = relu[d]; r.neuron = neuron[d]; r.sign = 1; r.beta = 0.f;
        buf[s0 * maxd + n] = r;
        r.sign = -1;
        buf[s1 * maxd + n] = r;
        ns[s0] = n + 1; ns[s1] = n + 1;
    }
}

}  // namespace

}  // namespace nyb

using namespace nyb;

extern "C" {

int32_t nyb200_frontier_create(nyb200_engine *e, int32_t net_id, const float *spec, const float *thresholds, const int32_t *owner,
                               int32_t S, int32_t n_clauses, const float *in_lo, const float *in_hi, const float *inh_lo,
                               const float *inh_hi, int32_t max_depth, int64_t capacity) {
    if (!e || !spec || !thresholds || !owner || !in_lo || !in_hi || !inh_lo || !inh_hi) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    Net *net;
    NYB_TRY(find_net(e, net_id, &net));
    const NetView &nv = net->v;
    if (S <= 0 || S > kMaxRowsF || n_clauses <= 0 || n_clauses > 32) return set_err(e, NYB200_ERR_SHAPE, "1..64 rows in 1..32 clauses");
    if (max_depth <= 0 || capacity < 2) return set_err(e, NYB200_ERR_SHAPE, "max_depth and capacity must be positive");
    for (int s = 0; s < S; ++s)
        if (owner[s] < 0 || owner[s] >= n_clauses) return set_err(e, NYB200_ERR_INVALID, "row owner out of range");
    // A search per property creates and destroys its frontier; the arrays of the last one are kept and serve again when
    // they are large enough (an allocation or a release of this size synchronises the device and costs milliseconds).
    if (e->frontier) { frontier_free(e->frontier); e->frontier = nullptr; }
    ResidentFrontier *f = e->frontier_spare ? e->frontier_spare : new ResidentFrontier();
    e->frontier_spare = nullptr;
    f->net_id = net_id; f->S = S; f->maxd = max_depth; f->n_clauses = n_clauses; f->cap = capacity;
    f->bounded = 0; f->optimistic = true; f->verdict_refinement = false;
    f->n_spec = (size_t)S * nv.dims[nv.L]; f->n_box = (size_t)nv.dims[0]; f->n_inh = (size_t)nv.n_pre;
    auto fit = [&](void **ptr, size_t *have, size_t need) -> bool {
        if (*ptr && *have >= need) return true;
        if (*ptr) { cudaFree(*ptr); *ptr = nullptr; *have = 0; }
        if (cudaMalloc(ptr, need) != cudaSuccess) return false;
        *have = need;
        return true;
    };
    const size_t thr_need = (size_t)kMaxRowsF * 4;
    if (f->alpha && f->alpha_bytes < (size_t)capacity * nv.nps * 4) { cudaFree(f->alpha); f->alpha = nullptr; f->alpha_bytes = 0; }
    if (!fit((void **)&f->buf, &f->buf_bytes, (size_t)capacity * max_depth * sizeof(nyb200_split)) ||
        !fit((void **)&f->ns, &f->ns_bytes, (size_t)capacity * 4) ||
        (!f->stats && cudaMalloc(&f->stats, 64) != cudaSuccess) ||
        !fit((void **)&f->thr, &f->thr_bytes, thr_need) ||
        (!f->owner && cudaMalloc(&f->owner, thr_need) != cudaSuccess) ||
        !fit((void **)&f->consts, &f->consts_bytes, (f->n_spec + 2 * f->n_box + 2 * f->n_inh) * 4)) {
        frontier_free(f);
        return set_err(e, NYB200_ERR_OOM, "device allocation failed for the frontier");
    }
    NYB_CUDA(e, cudaMemcpy(f->thr, thresholds, (size_t)S * 4, cudaMemcpyHostToDevice));
    NYB_CUDA(e, cudaMemcpy(f->owner, owner, (size_t)S * 4, cudaMemcpyHostToDevice));
    {
        float *c = f->consts;
        NYB_CUDA(e, cudaMemcpy(c, spec, f->n_spec * 4, cudaMemcpyHostToDevice)); c += f->n_spec;
        NYB_CUDA(e, cudaMemcpy(c, in_lo, f->n_box * 4, cudaMemcpyHostToDevice)); c += f->n_box;
        NYB_CUDA(e, cudaMemcpy(c, in_hi, f->n_box * 4, cudaMemcpyHostToDevice)); c += f->n_box;
        NYB_CUDA(e, cudaMemcpy(c, inh_lo, f->n_inh * 4, cudaMemcpyHostToDevice)); c += f->n_inh;
        NYB_CUDA(e, cudaMemcpy(c, inh_hi, f->n_inh * 4, cudaMemcpyHostToDevice));
    }
    // the root: one domain without splits
    NYB_CUDA(e, cudaMemset(f->ns, 0, 4));
    f->head = 0; f->count = 1; f->no_alpha_front = 1;
    e->frontier = f;
    return NYB200_OK;
}

void nyb200_frontier_destroy(nyb200_engine *e) {
    if (!e) return;
    std::lock_guard<std::mutex> g(e->mu);
    if (e->frontier) {
        cudaSetDevice(e->device);
        cudaStreamSynchronize(e->stream);
        if (e->frontier_spare) frontier_free(e->frontier_spare);
        e->frontier_spare = e->frontier;   // its arrays serve the next frontier of this engine
        e->frontier = nullptr;
    }
}

// stats out: [0] domains bounded this round, [1] verified, [2] infeasible, [3] stuck (undecided, nothing left to
// split: they stay at the front of the frontier), [4] open domains in the frontier after the round, [5] deepest history
// bounded; min_lower: smallest lower bound of the round's feasible domains.
static int32_t frontier_round_impl(nyb200_engine *e, int32_t batch, int32_t branching, const nyb200_opt_config *cfg,
                                   int64_t *stats_out, float *min_lower) {
    if (!e || !stats_out || !min_lower || batch <= 0) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    const bool optimise = cfg && cfg->iterations > 1;
    ResidentFrontier *f = e->frontier;
    if (!f) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    if (branching != NYB200_BRANCH_WIDTH && branching != NYB200_BRANCH_INTERCEPT && branching != NYB200_BRANCH_BABSR)
        return set_err(e, NYB200_ERR_INVALID, "unknown branching score");
    if (batch > (1 << 16)) return set_err(e, NYB200_ERR_UNSUPPORTED, "at most 65536 domains per round");
    for (int i = 0; i < 6; ++i) stats_out[i] = 0;
    *min_lower = INFINITY;
    if (f->count == 0) return NYB200_OK;
    Net *net;
    NYB_TRY(find_net(e, f->net_id, &net));
    const NetView &nv = net->v;
    const int D = (int)(f->count < batch ? f->count : batch);
    cudaStream_t st = e->stream;
    if (optimise && !f->alpha) {
        if (cudaMalloc(&f->alpha, (size_t)f->cap * nv.nps * 4) != cudaSuccess)
            return set_err(e, NYB200_ERR_OOM, "device allocation failed for the frontier's slopes (capacity x neurons)");
        f->alpha_bytes = (size_t)f->cap * nv.nps * 4;
    }
    // warm start only when every domain of the batch has slopes of its own (the host loop's rule)
    const bool warm = optimise && f->no_alpha_front == 0;
    Batch b;
    b.net_id = f->net_id; b.S = f->S; b.R = 2 * f->S; b.D = D; b.mode = 1; b.box_stride = 0; b.max_splits = f->maxd;
    b.has_alpha = warm;
    BatchPtrs p;
    NYB_TRY(batch_ptrs(e, *net, b, p));
    {   // the search's constants, device to device (the workspace arrays may have served another call in between)
        const float *c = f->consts;
        NYB_CUDA(e, cudaMemcpyAsync(p.spec, c, f->n_spec * 4, cudaMemcpyDeviceToDevice, st)); c += f->n_spec;
        NYB_CUDA(e, cudaMemcpyAsync(p.in_lo, c, f->n_box * 4, cudaMemcpyDeviceToDevice, st)); c += f->n_box;
        NYB_CUDA(e, cudaMemcpyAsync(p.in_hi, c, f->n_box * 4, cudaMemcpyDeviceToDevice, st)); c += f->n_box;
        NYB_CUDA(e, cudaMemcpyAsync(p.inh_lo, c, f->n_inh * 4, cudaMemcpyDeviceToDevice, st)); c += f->n_inh;
        NYB_CUDA(e, cudaMemcpyAsync(p.inh_hi, c, f->n_inh * 4, cudaMemcpyDeviceToDevice, st));
    }
    // the batch: the first D ring slots (two pieces when the ring wraps)
    const long first = (f->cap - f->head) < D ? (f->cap - f->head) : D;
    const size_t row = (size_t)f->maxd * sizeof(nyb200_split);
    NYB_CUDA(e, cudaMemcpyAsync(p.splits, f->buf + f->head * f->maxd, (size_t)first * row, cudaMemcpyDeviceToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(p.nsplits, f->ns + f->head, (size_t)first * 4, cudaMemcpyDeviceToDevice, st));
    if (first < D) {
        NYB_CUDA(e, cudaMemcpyAsync(p.splits + first * f->maxd, f->buf, (size_t)(D - first) * row, cudaMemcpyDeviceToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(p.nsplits + first, f->ns, (size_t)(D - first) * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (warm) {
        NYB_CUDA(e, cudaMemcpyAsync(p.alpha, f->alpha + f->head * nv.nps, (size_t)first * nv.nps * 4, cudaMemcpyDeviceToDevice, st));
        if (first < D)
            NYB_CUDA(e, cudaMemcpyAsync(p.alpha + first * nv.nps, f->alpha, (size_t)(D - first) * nv.nps * 4, cudaMemcpyDeviceToDevice, st));
    }
    b.valid = true;
    b.decision_thr = f->verdict_refinement ? f->thr : nullptr;   // which domains the binary64 re-evaluation is worth
    e->batch = b;
    NYB_WS(done, int *, e, "fr_done", (size_t)D * 4);
    NYB_WS(pos, int *, e, "fr_pos", (size_t)D * 4);
    NYB_WS(dr, int *, e, "br_relu", (size_t)D * 4);
    NYB_WS(dn, int *, e, "br_neuron", (size_t)D * 4);
    NYB_WS(dw, float *, e, "br_width", (size_t)D * 4);
    int hs[6];
    // decisions, split neurons, the open domains' positions and the round's counters, read with one synchronisation
    auto evaluate = [&]() -> int {
        static const int init_stats[6] = {0, 0, 0, 0, 0x7f800000, 0};   // +inf as float bits
        NYB_CUDA(e, cudaMemcpyAsync(f->stats, init_stats, sizeof(init_stats), cudaMemcpyHostToDevice, st));
        k_frontier_decide<<<(D + 255) / 256, 256, 0, st>>>(D, f->S, f->n_clauses, p.out_lo, p.flags, f->thr, f->owner, done, f->stats);
        e->launches++;
        if (branching == NYB200_BRANCH_BABSR) NYB_TRY(babsr_select(e, *net, e->batch, p, dr, dn, dw, nullptr));
        else launch_select_branch(e, nv, D, p.pre_lo, p.pre_hi, p.code, dr, dn, dw, branching);
        k_frontier_scan<<<1, 1024, 0, st>>>(D, done, dr, p.nsplits, pos, f->stats);
        e->launches++;
        NYB_CUDA(e, cudaMemcpyAsync(hs, f->stats, sizeof(hs), cudaMemcpyDeviceToHost, st));
        NYB_CUDA(e, cudaStreamSynchronize(st));
        return NYB200_OK;
    };
    if (optimise) {
        NYB_TRY(optimize_batch(e, *cfg));
        NYB_TRY(finish_batch_public(e));   // synchronises; folds a binary64 re-evaluation into the best bounds if flagged
        NYB_TRY(evaluate());
    } else if (f->optimistic) {
        // The decisions are queued behind the bound without waiting for it.  The run's last kernel has published the
        // pipeline error word and the number of domains flagged for the binary64 re-evaluation to mapped host memory
        // by the time the counters have arrived; a flagged round pays for a second pass, and the next round waits for
        // its bound before it decides (searches on narrow boxes flag most rounds).
        NYB_TRY(run_batch_public(e));
        NYB_TRY(evaluate());
        const volatile int *sw = e->status_host;
        if (sw && (sw[1] != 0 || sw[2] > 0)) {
            NYB_TRY(finish_batch_public(e));
            NYB_TRY(evaluate());
            f->optimistic = false;
        }
    } else {
        NYB_TRY(run_batch_public(e));
        NYB_TRY(finish_batch_public(e));   // synchronises; re-evaluates flagged domains in binary64
        NYB_TRY(evaluate());
        f->optimistic = e->batch.refined == 0;
    }
    const int n_open = hs[0], n_stuck = hs[3], deepest = hs[5];
    stats_out[1] = hs[1]; stats_out[2] = hs[2]; stats_out[3] = n_stuck; stats_out[5] = deepest;
    memcpy(min_lower, &hs[4], 4);
    if (n_stuck > 0) {
        // a domain that can be neither decided nor split: the batch goes back untouched and the search ends "unknown"
        stats_out[0] = 0; stats_out[4] = f->count;
        return NYB200_OK;
    }
    if (n_open > 0 && deepest + 1 > f->maxd) return set_err(e, NYB200_ERR_UNSUPPORTED, "split history deeper than the frontier's max_depth");
    if (f->count - D + 2L * n_open > f->cap) return set_err(e, NYB200_ERR_OOM, "frontier capacity exceeded");
    const long tail = (f->head + f->count) % f->cap;
    if (n_open > 0) {
        if (optimise) k_frontier_children_warm<<<D, 128, 0, st>>>(nv, D, f->maxd, f->cap, tail, p.splits, p.nsplits, pos, dr, dn, p.tab, f->buf, f->ns, f->alpha);
        else k_frontier_children<<<D, 64, 0, st>>>(D, f->maxd, f->cap, tail, p.splits, p.nsplits, pos, dr, dn, f->buf, f->ns);
        e->launches++;
    }
    NYB_CUDA(e, cudaGetLastError());
    f->head = (f->head + D) % f->cap;
    f->count += 2L * n_open - D;
    f->no_alpha_front = f->no_alpha_front > D ? f->no_alpha_front - D : 0;
    if (!optimise && n_open > 0) f->no_alpha_front = f->count;   // children without slopes behind whatever was there
    f->bounded += D;
    stats_out[0] = D; stats_out[4] = f->count;
    return NYB200_OK;
}

int32_t nyb200_frontier_round(nyb200_engine *e, int32_t batch, int32_t branching, int64_t *stats_out, float *min_lower) {
    return frontier_round_impl(e, batch, branching, nullptr, stats_out, min_lower);
}

int32_t nyb200_frontier_round_optimized(nyb200_engine *e, int32_t batch, int32_t branching, const nyb200_opt_config *cfg,
                                        int64_t *stats_out, float *min_lower) {
    if (!cfg) return NYB200_ERR_INVALID;
    return frontier_round_impl(e, batch, branching, cfg, stats_out, min_lower);
}

int32_t nyb200_frontier_set_refinement(nyb200_engine *e, int32_t verdict_only) {
    if (!e) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    if (!e->frontier) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    e->frontier->verdict_refinement = verdict_only != 0;
    return NYB200_OK;
}

int32_t nyb200_frontier_count(nyb200_engine *e, int64_t *open) {
    if (!e || !open) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    if (!e->frontier) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    *open = e->frontier->count;
    return NYB200_OK;
}

// Up to n records leave from the back of the ring (the domains that would be bounded last) into the caller's device
// arrays: dev_splits [n x max_depth] records, dev_nsplits [n].  The copies are complete when the call returns, so
// the caller may hand the arrays to any stream or to a collective.
int32_t nyb200_frontier_take(nyb200_engine *e, int64_t n, void *dev_splits, int32_t *dev_nsplits, int64_t *taken) {
    if (!e || !taken || n < 0 || (n > 0 && (!dev_splits || !dev_nsplits))) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    ResidentFrontier *f = e->frontier;
    if (!f) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    const long m = n < f->count ? (long)n : f->count;
    *taken = m;
    if (m == 0) return NYB200_OK;
    cudaStream_t st = e->stream;
    const size_t row = (size_t)f->maxd * sizeof(nyb200_split);
    const long start = (f->head + f->count - m) % f->cap;           // first of the m last slots
    const long first = (f->cap - start) < m ? (f->cap - start) : m;  // slots before the ring wraps
    NYB_CUDA(e, cudaMemcpyAsync(dev_splits, f->buf + start * f->maxd, (size_t)first * row, cudaMemcpyDeviceToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(dev_nsplits, f->ns + start, (size_t)first * 4, cudaMemcpyDeviceToDevice, st));
    if (first < m) {
        NYB_CUDA(e, cudaMemcpyAsync((char *)dev_splits + (size_t)first * row, f->buf, (size_t)(m - first) * row, cudaMemcpyDeviceToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(dev_nsplits + first, f->ns, (size_t)(m - first) * 4, cudaMemcpyDeviceToDevice, st));
    }
    NYB_CUDA(e, cudaStreamSynchronize(st));
    f->count -= m;
    if (f->no_alpha_front > f->count) f->no_alpha_front = f->count;
    return NYB200_OK;
}

// n records (same layout, device arrays whose contents are complete: the caller has synchronised the stream or the
// collective that filled them) are appended at the back of the ring.
int32_t nyb200_frontier_give(nyb200_engine *e, int64_t n, const void *dev_splits, const int32_t *dev_nsplits) {
    if (!e || n < 0 || (n > 0 && (!dev_splits || !dev_nsplits))) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    ResidentFrontier *f = e->frontier;
    if (!f) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    if (n == 0) return NYB200_OK;
    if (f->count + n > f->cap) return set_err(e, NYB200_ERR_OOM, "frontier capacity exceeded");
    cudaStream_t st = e->stream;
    const size_t row = (size_t)f->maxd * sizeof(nyb200_split);
    const long tail = (f->head + f->count) % f->cap;
    const long first = (f->cap - tail) < n ? (f->cap - tail) : (long)n;
    NYB_CUDA(e, cudaMemcpyAsync(f->buf + tail * f->maxd, dev_splits, (size_t)first * row, cudaMemcpyDeviceToDevice, st));
    NYB_CUDA(e, cudaMemcpyAsync(f->ns + tail, dev_nsplits, (size_t)first * 4, cudaMemcpyDeviceToDevice, st));
    if (first < n) {
        NYB_CUDA(e, cudaMemcpyAsync(f->buf, (const char *)dev_splits + (size_t)first * row, (size_t)(n - first) * row, cudaMemcpyDeviceToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(f->ns, dev_nsplits + first, (size_t)(n - first) * 4, cudaMemcpyDeviceToDevice, st));
    }
    NYB_CUDA(e, cudaStreamSynchronize(st));   // the caller may reuse its arrays
    f->count += n;
    f->no_alpha_front = f->count;   // records from outside carry no slopes
    return NYB200_OK;
}

// The open records in ring order (front first) to host arrays [count x max_depth] / [count]; the frontier keeps them.
int32_t nyb200_frontier_download(nyb200_engine *e, int64_t capacity, nyb200_split *splits, int32_t *nsplits, int64_t *n_out) {
    if (!e || !n_out || capacity < 0) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    ResidentFrontier *f = e->frontier;
    if (!f) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    *n_out = f->count;
    if (f->count == 0) return NYB200_OK;
    if (capacity < f->count || !splits || !nsplits) return set_err(e, NYB200_ERR_SHAPE, "host arrays smaller than the frontier");
    cudaStream_t st = e->stream;
    const size_t row = (size_t)f->maxd * sizeof(nyb200_split);
    const long m = f->count;
    const long first = (f->cap - f->head) < m ? (f->cap - f->head) : m;
    NYB_CUDA(e, cudaMemcpyAsync(splits, f->buf + f->head * f->maxd, (size_t)first * row, cudaMemcpyDeviceToHost, st));
    NYB_CUDA(e, cudaMemcpyAsync(nsplits, f->ns + f->head, (size_t)first * 4, cudaMemcpyDeviceToHost, st));
    if (first < m) {
        NYB_CUDA(e, cudaMemcpyAsync((char *)splits + (size_t)first * row, f->buf, (size_t)(m - first) * row, cudaMemcpyDeviceToHost, st));
        NYB_CUDA(e, cudaMemcpyAsync(nsplits + first, f->ns, (size_t)(m - first) * 4, cudaMemcpyDeviceToHost, st));
    }
    NYB_CUDA(e, cudaStreamSynchronize(st));
    return NYB200_OK;
}

// Replaces the frontier's contents by n host records ([n x depth] with depth <= max_depth, [n]): the resume of a dump.
int32_t nyb200_frontier_upload(nyb200_engine *e, int64_t n, int32_t depth, const nyb200_split *splits, const int32_t *nsplits) {
    if (!e || n < 0 || depth <= 0 || (n > 0 && (!splits || !nsplits))) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    NYB_CUDA(e, cudaSetDevice(e->device));
    ResidentFrontier *f = e->frontier;
    if (!f) return set_err(e, NYB200_ERR_INVALID, "no frontier");
    if (n > f->cap) return set_err(e, NYB200_ERR_OOM, "frontier capacity exceeded");
    if (depth > f->maxd) return set_err(e, NYB200_ERR_SHAPE, "histories deeper than the frontier's max_depth");
    for (int64_t i = 0; i < n; ++i)
        if (nsplits[i] < 0 || nsplits[i] > depth) return set_err(e, NYB200_ERR_INVALID, "history length out of range");
    cudaStream_t st = e->stream;
    f->head = 0; f->count = 0;
    if (n > 0) {
        NYB_CUDA(e, cudaMemcpy2DAsync(f->buf, (size_t)f->maxd * sizeof(nyb200_split), splits, (size_t)depth * sizeof(nyb200_split),
                                      (size_t)depth * sizeof(nyb200_split), (size_t)n, cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaMemcpyAsync(f->ns, nsplits, (size_t)n * 4, cudaMemcpyHostToDevice, st));
        NYB_CUDA(e, cudaStreamSynchronize(st));
    }
    f->count = n;
    f->no_alpha_front = n;
    return NYB200_OK;
}

}  // extern "C"
