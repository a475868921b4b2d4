// Fused backward chain: the CROWN coefficient rows of a 128-row tile go through ALL hidden layers inside one
// persistent CTA - contraction A * W_k on tcgen05 (3xTF32), ReLU relaxation with alpha slopes and beta
// multipliers, bias and rounding-penalty row sums, TF32 split of the result - without leaving the SM between
// layers.  Rows (domain, spec row) never mix across layers, so a CTA owns its rows for the whole chain
// (the role of relu_backward_with_alpha_beta, beta_crown/engine/backward/relu_backward.rs:33-185, applied right
// after propagate_linear, layers/linear/crown_single.rs:1931-2226, for every hidden layer in turn).
//
// Roles of one CTA (4 control warps + NSUB*4 epilogue warps):
//   warp 0      streams the pre-split weight tiles Wl^T, Wh^T of every layer by TMA into a ring of three 32 KB
//               slots (K-major, 128-byte swizzle), running ahead of the tensor core across layers and tiles;
//   warp 1      issues tcgen05.mma (M128 x N<=256 x K8, kind::tf32): per 32-wide K chunk four steps Ah*Wl and four
//               Al*Wh into the CROSS accumulator and four Ah*Wh into the MAIN accumulator (tensor memory columns
//               [256, 512) and [0, 256)); every chunk's commit hands its operand slots back;
//   warp 2      allocates / frees the 512 tensor-memory columns;
//   warp 3      stages the relaxation tables (slopes, intercept, signed multiplier; the prepared charge weights; the
//               bias slice) of the tile's domains into a four-slot ring by 1-D bulk copies, 64 columns at a time,
//               so that the epilogue reads them from shared memory instead of waiting on L2 (the CTA's shared
//               memory leaves almost no L1);
//   epilogue    thread = (row of the tile, one slice of every 32-column chunk).  When a layer's products are
//               complete it drains its slices of both accumulators into registers (main + cross, one fp32 add),
//               releases the accumulators, then walks its chunks: relaxation step per coefficient (the same
//               function the stand-alone relaxation kernel uses, so the coefficient bits are the same for the same
//               input), row sums in registers, TF32 high/low split written straight into the next layer's operand
//               ring in the swizzled layout the tensor core reads.  The next layer's products start as soon as the
//               first chunk is there.  The last fused layer's rows go to global memory for the final (wide)
//               contraction and the concretisation.
//
// Keeping the cross terms in their own accumulator is what makes a full-K accumulation chain affordable in the
// rounding model: the main accumulator sees K/8 steps at the scale of S = |A||W|, the cross accumulator 2K/8 steps
// at 2^-10 S, and their sum one fp32 rounding (see chain_eps).  Every mbarrier wait is bounded; on expiry the
// kernel records a code, every role stops at its next check, tensor memory is freed and the kernel returns.
#include "nyb200_internal.cuh"
#include "nyb200_relax.cuh"
#include "nyb200_tcgen05.cuh"

namespace nyb {

namespace chain {

using namespace umma;

constexpr int BM = 128, BN = 256, BK = 32;
constexpr int A_HALF = BM * BK * 4;   // 16 KB: the high or the low part of one operand chunk
constexpr int A_SLOT = 2 * A_HALF;    // 32 KB
constexpr int W_SLOT = BN * BK * 4;   // 32 KB: one of Wh / Wl for one K chunk
constexpr int NA = 2, NW = 3;
// Table ring: the relaxation tables of the domains a tile's rows belong to, staged by bulk copies one chunk PAIR (64
// columns) at a time.  Slot layout: 64 bias values, then per domain 64 table entries (float4), 64 charge weights and
// 16 bytes of padding (so that the rows of different domains read different banks).
constexpr int NT = 4;
constexpr int MAXD = 10;                                   // domains a 128-row tile may span in the staged variant
constexpr int T_COLS = 2 * BK;
constexpr int T_DOM = T_COLS * 16 + T_COLS * 4 + 16;       // 1296
constexpr int T_HEAD = T_COLS * 4;                         // 256: the bias slice
constexpr int T_SLOT = (T_HEAD + MAXD * T_DOM + 127) & ~127;
constexpr int BAR_BYTES = 512;
constexpr int SMEM_BYTES = NA * A_SLOT + NW * W_SLOT + NT * T_SLOT + 1024 /*alignment*/ + BAR_BYTES;
static_assert(SMEM_BYTES <= 232448, "more than the 227 KB a CTA can opt into");
constexpr int kMaxChain = 16;         // fused contractions per launch
constexpr int MAX_CHUNKS = BN / BK;   // 8

struct Layer {
    alignas(64) CUtensorMap tm_hi;
    alignas(64) CUtensorMap tm_lo;
    int K, N;            // contraction length (rows' current width) and output width, both <= 256
    int relu_off;        // offset of the ReLU's block inside a per-domain table row
    long q_ds;           // per-domain stride of q for the contraction that follows the relaxation
    const float *bias;   // bias of that contraction's layer (indexed by output column here), or null
    float eps;           // rounding rate of that contraction
    int to_global;       // 1: the relaxed rows leave through A_out (last fused layer)
};

struct Params {
    int n_layers;
    int M, R, S;
    int seed_identity;   // 0: rows are the spec rows; 1: identity rows (partial pass)
    int K_top;           // width of the seed rows
    const float *spec;   // [S x K_top]
    // identity pass in front of the first contraction (its bias and rounding charge)
    const float *top_bias;
    int top_off;
    long top_q_ds;
    float top_eps;
    const float4 *tab;
    const float *zabs, *q, *aup;
    const float *cj;     // [D x nps] per-(domain, column) charge weights prepared by k_chain_prep
    long nps;
    float *A_out;
    int lda;
    double *rb, *rpen;
    int *err;
    Layer layer[kMaxChain];
};

template <int CPT>
__device__ __forceinline__ void tmem_ld_cols(unsigned taddr, unsigned (&r)[CPT]);
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<8>(unsigned taddr, unsigned (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// NSUB epilogue warps share a tensor-memory lane quarter; each takes 32 / NSUB columns of every chunk.
template <int NSUB>
struct Cfg {
    static constexpr int EPI_WARPS = 4 * NSUB;
    static constexpr int THREADS = 128 + 32 * EPI_WARPS;
    static constexpr int CPT = BK / NSUB;                 // columns of a chunk per thread
    static constexpr int VALS = MAX_CHUNKS * CPT;         // accumulator values a thread holds
    // register split: launch with REGS_LAUNCH per thread, control warps drop to 40, epilogue warps take the rest
    static constexpr int REGS_LAUNCH = (65536 / THREADS) & ~7;
    static constexpr int REGS_CONTROL = NSUB == 2 ? 40 : 32;
    static constexpr int REGS_EPI = ((THREADS * REGS_LAUNCH - 128 * REGS_CONTROL) / (32 * EPI_WARPS)) & ~7;
    static_assert(128 * REGS_CONTROL + 32 * EPI_WARPS * REGS_EPI <= THREADS * REGS_LAUNCH, "setmaxnreg targets exceed the allocation");
    static_assert(REGS_EPI <= 255, "register target out of range");
};

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier (addresses and size multiples of 16)
__device__ __forceinline__ void bulk_load(unsigned dst, const void *src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// STAGED: warp 3 brings the tables into shared memory ahead of the epilogue (tiles that span at most MAXD domains);
// otherwise every epilogue thread loads its entries from global memory itself.
template <int NSUB, bool STAGED>
__global__ void __launch_bounds__(Cfg<NSUB>::THREADS, 1) k_chain(const __grid_constant__ Params P) {
    using C = Cfg<NSUB>;
    constexpr int CPT = C::CPT;
    extern __shared__ unsigned char smem_raw[];
    // aligned to 1024 bytes by an offset, not by a cast through an integer: the pointer stays a shared-memory pointer
    // for the compiler, which then emits shared-space loads and stores instead of generic ones
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *a_ring = smem;
    unsigned char *w_ring = smem + NA * A_SLOT;
    unsigned char *t_ring = w_ring + NW * W_SLOT;
    unsigned long long *bars = (unsigned long long *)(t_ring + NT * T_SLOT);
    const int A_FULL = 0, A_EMPTY = NA, W_FULL = 2 * NA, W_EMPTY = 2 * NA + NW, ACC_FULL = 2 * NA + 2 * NW, ACC_EMPTY = ACC_FULL + 1;
    const int T_FULL = ACC_EMPTY + 1, T_EMPTY = T_FULL + NT;
    unsigned *tmem_slot = (unsigned *)(bars + T_EMPTY + NT);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    static_assert((2 * NA + 2 * NW + 2 + 2 * NT) * 8 + 8 <= BAR_BYTES, "barrier block overflows its slots");

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (P.M + BM - 1) / BM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NA; ++s) { mbar_init(smem_u32(&bars[A_FULL + s]), C::EPI_WARPS); mbar_init(smem_u32(&bars[A_EMPTY + s]), 1); }
        for (int s = 0; s < NW; ++s) { mbar_init(smem_u32(&bars[W_FULL + s]), 1); mbar_init(smem_u32(&bars[W_EMPTY + s]), 1); }
        mbar_init(smem_u32(&bars[ACC_FULL]), 1);
        mbar_init(smem_u32(&bars[ACC_EMPTY]), C::EPI_WARPS);
        for (int s = 0; s < NT; ++s) { mbar_init(smem_u32(&bars[T_FULL + s]), 1); mbar_init(smem_u32(&bars[T_EMPTY + s]), C::EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();   // barriers and tensor memory are set up; from here on the kernel reads what earlier kernels wrote

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::REGS_CONTROL));
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ weight producer (TMA)
            unsigned it = 0;
            for (int t = blockIdx.x; t < n_tiles && !*abort_flag; t += gridDim.x) {
                for (int l = 0; l < P.n_layers && !*abort_flag; ++l) {
                    const Layer &Ly = P.layer[l];
                    const int kc = (Ly.K + BK - 1) / BK;
                    for (int c = 0; c < kc; ++c) {
#pragma unroll
                        for (int part = 0; part < 2; ++part, ++it) {  // the low half first: its steps are issued first
                            const int s = it % NW;
                            const unsigned ph = (it / NW) & 1;
                            if (!mbar_wait(smem_u32(&bars[W_EMPTY + s]), ph ^ 1, 400)) { atomicExch(P.err, 11); *abort_flag = 1; break; }
                            const unsigned bar = smem_u32(&bars[W_FULL + s]);
                            mbar_expect_tx(bar, W_SLOT);
                            tma_load_2d(smem_u32(w_ring + s * W_SLOT), part == 0 ? &Ly.tm_lo : &Ly.tm_hi, c * BK, 0, bar);
                        }
                        if (*abort_flag) break;
                    }
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            unsigned wit = 0, ait = 0, lit = 0;
            bool failed = false;
            for (int t = blockIdx.x; t < n_tiles && !failed && !*abort_flag; t += gridDim.x) {
                for (int l = 0; l < P.n_layers && !failed; ++l, ++lit) {
                    const Layer &Ly = P.layer[l];
                    const int kc = (Ly.K + BK - 1) / BK;
                    const int n_eff = min(BN, (Ly.N + 15) & ~15);
                    const unsigned idesc = make_idesc(BM, n_eff);
                    // both accumulators must have been drained by the epilogue of the previous layer
                    if (!mbar_wait(smem_u32(&bars[ACC_EMPTY]), (lit & 1) ^ 1, 100)) { atomicExch(P.err, 12); *abort_flag = 1; failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned d_main = tmem_base, d_cross = tmem_base + BN;
                    for (int c = 0; c < kc && !failed; ++c, ++ait) {
                        const int sa = ait % NA;
                        if (!mbar_wait(smem_u32(&bars[A_FULL + sa]), (ait / NA) & 1, 100)) { atomicExch(P.err, 13); *abort_flag = 1; failed = true; break; }
                        const unsigned long long a_hi = make_desc(smem_u32(a_ring + sa * A_SLOT));
                        const unsigned long long a_lo = make_desc(smem_u32(a_ring + sa * A_SLOT + A_HALF));
                        // Ah * Wl
                        int sw = wit % NW;
                        if (!mbar_wait(smem_u32(&bars[W_FULL + sw]), (wit / NW) & 1, 100)) { atomicExch(P.err, 14); *abort_flag = 1; failed = true; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        unsigned long long b = make_desc(smem_u32(w_ring + sw * W_SLOT));
#pragma unroll
                        for (int k4 = 0; k4 < BK / 8; ++k4) {
                            const unsigned long long adv = (unsigned long long)(k4 * 2);  // 8 TF32 = 32 bytes = 2 x 16 B
                            mma_tf32(d_cross, a_hi + adv, b + adv, idesc, (c == 0 && k4 == 0) ? 0u : 1u);
                        }
                        mma_commit(smem_u32(&bars[W_EMPTY + sw]));
                        ++wit;
                        // Al * Wh (cross), Ah * Wh (main)
                        sw = wit % NW;
                        if (!mbar_wait(smem_u32(&bars[W_FULL + sw]), (wit / NW) & 1, 100)) { atomicExch(P.err, 15); *abort_flag = 1; failed = true; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        b = make_desc(smem_u32(w_ring + sw * W_SLOT));
#pragma unroll
                        for (int k4 = 0; k4 < BK / 8; ++k4) {
                            const unsigned long long adv = (unsigned long long)(k4 * 2);
                            mma_tf32(d_cross, a_lo + adv, b + adv, idesc, 1u);
                        }
#pragma unroll
                        for (int k4 = 0; k4 < BK / 8; ++k4) {
                            const unsigned long long adv = (unsigned long long)(k4 * 2);
                            mma_tf32(d_main, a_hi + adv, b + adv, idesc, (c == 0 && k4 == 0) ? 0u : 1u);
                        }
                        mma_commit(smem_u32(&bars[W_EMPTY + sw]));
                        mma_commit(smem_u32(&bars[A_EMPTY + sa]));
                        ++wit;
                    }
                    if (!failed) mma_commit(smem_u32(&bars[ACC_FULL]));
                }
            }
        } else if (STAGED && warp == 3 && lane == 0) {
            // ------------------------------------------------------------ table producer (bulk copies)
            unsigned tit = 0;
            bool failed = false;
            for (int t = blockIdx.x; t < n_tiles && !failed && !*abort_flag; t += gridDim.x) {
                const long m0 = (long)t * BM;
                const long m1 = (m0 + BM < (long)P.M ? m0 + BM : (long)P.M) - 1;
                const int d0 = (int)(m0 / P.R), nd = (int)(m1 / P.R) - d0 + 1;
                for (int l = 0; l < P.n_layers && !failed; ++l) {
                    const Layer &Ly = P.layer[l];
                    const int nch = (Ly.N + BK - 1) / BK;
                    for (int c2 = 0; c2 < nch; c2 += 2, ++tit) {
                        const int s = tit % NT;
                        if (!mbar_wait(smem_u32(&bars[T_EMPTY + s]), ((tit / NT) & 1) ^ 1, 400)) { atomicExch(P.err, 16); *abort_flag = 1; failed = true; break; }
                        const int w = Ly.N - c2 * BK < T_COLS ? Ly.N - c2 * BK : T_COLS;   // a multiple of 4
                        const unsigned bar = smem_u32(&bars[T_FULL + s]);
                        mbar_expect_tx(bar, (unsigned)((Ly.bias ? w * 4 : 0) + nd * w * 20));
                        const unsigned dst = smem_u32(t_ring + s * T_SLOT);
                        if (Ly.bias) bulk_load(dst, Ly.bias + c2 * BK, (unsigned)(w * 4), bar);
                        for (int dd = 0; dd < nd; ++dd) {
                            const long idx = (long)(d0 + dd) * P.nps + Ly.relu_off + c2 * BK;
                            bulk_load(dst + T_HEAD + dd * T_DOM, P.tab + idx, (unsigned)(w * 16), bar);
                            bulk_load(dst + T_HEAD + dd * T_DOM + T_COLS * 16, P.cj + idx, (unsigned)(w * 4), bar);
                        }
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::REGS_EPI));
        const int qd = warp & 3, sub = (warp - 4) >> 2;
        const int r = qd * 32 + lane;  // row of the tile = tensor-memory lane
        unsigned ait = 0, lit = 0, tit = 0;
        bool dead = false;
        // Writes the thread's CPT columns of chunk `c` (values v, already relaxed) as TF32 high / low parts into ring
        // slot `sa`: row r, 16-byte unit u at position u ^ (r & 7) of the row's 128 bytes.
        auto put_chunk = [&](int sa, const float (&v)[CPT]) {
            float *ah = (float *)(a_ring + sa * A_SLOT), *al = (float *)(a_ring + sa * A_SLOT + A_HALF);
#pragma unroll
            for (int g = 0; g < CPT / 4; ++g) {
                const float4 x = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                const float4 h = make_float4(rn_tf32(x.x), rn_tf32(x.y), rn_tf32(x.z), rn_tf32(x.w));
                const float4 lo = make_float4(rn_tf32(x.x - h.x), rn_tf32(x.y - h.y), rn_tf32(x.z - h.z), rn_tf32(x.w - h.w));
                const int u = sub * (CPT / 4) + g;
                const int off = r * 32 + ((u ^ (r & 7)) << 2);
                *(float4 *)(ah + off) = h;
                *(float4 *)(al + off) = lo;
            }
        };
        // hands a finished chunk to the tensor core: every thread orders its generic-proxy stores before the async
        // proxy's reads, the warp meets, one lane arrives
        auto publish = [&](int sa) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[A_FULL + sa]));
        };
        auto wait_slot = [&](int code) -> bool {
            const int sa = ait % NA;
            bool ok = mbar_wait(smem_u32(&bars[A_EMPTY + sa]), ((ait / NA) & 1) ^ 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) { atomicExch(P.err, code); *abort_flag = 1; } dead = true; }
            return ok;
        };
        for (int t = blockIdx.x; t < n_tiles && !dead && !*abort_flag; t += gridDim.x) {
            const long m = (long)t * BM + r;
            const bool live = m < P.M;
            const int d = live ? (int)(m / P.R) : 0;
            const int dd = live ? d - (int)(((long)t * BM) / P.R) : 0;   // the row's domain among the tile's domains
            const int rr = live ? (int)(m - (long)d * P.R) : 0;
            const bool upper = rr >= P.S;
            double sb = 0.0;      // bias of the row (this thread's columns)
            float spt = 0.f;      // rounding penalty and bias magnitude share, rounded upwards
            const int dir = upper ? 1 : -1;
            const float dirf = upper ? 1.f : -1.f;
            // ---- seed rows and the identity pass in front of the first contraction
            {
                const int kc = (P.K_top + BK - 1) / BK;
                const float *srow = P.spec + (long)(rr % P.S) * P.K_top;
                const float *crow = P.cj + (long)d * P.nps + P.top_off;
                for (int c = 0; c < kc && !dead; ++c, ++ait) {
                    if (!wait_slot(21)) break;
                    float v[CPT];
                    float sp_ = 0.f, gb = 0.f;
#pragma unroll
                    for (int j = 0; j < CPT; ++j) {
                        const int col = c * BK + sub * CPT + j;
                        float a = 0.f;
                        if (live && col < P.K_top) {
                            a = P.seed_identity ? ((rr % P.S) == col ? 1.f : 0.f) : srow[col];
                            if (P.top_bias) gb = fmaf(a, P.top_bias[col], gb);
                            sp_ = __fmaf_ru(fabsf(a), crow[col], sp_);
                        }
                        v[j] = a;
                    }
                    sb += (double)gb;
                    spt = __fadd_ru(spt, sp_);
                    put_chunk(ait % NA, v);
                    publish(ait % NA);
                }
            }
            // ---- the fused layers
            for (int l = 0; l < P.n_layers && !dead; ++l, ++lit) {
                const Layer &Ly = P.layer[l];
                const int N = Ly.N;
                const int nch = (N + BK - 1) / BK;
                bool ok = mbar_wait(smem_u32(&bars[ACC_FULL]), lit & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) { atomicExch(P.err, 22); *abort_flag = 1; } dead = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float acc[C::VALS];
#pragma unroll
                for (int c = 0; c < MAX_CHUNKS; ++c) {
                    if (c < nch) {
                        unsigned rm[CPT], rc[CPT];
                        const unsigned taddr = tmem_base + ((unsigned)(qd * 32) << 16) + (unsigned)(c * BK + sub * CPT);
                        tmem_ld_cols<CPT>(taddr, rm);
                        tmem_ld_cols<CPT>(taddr + BN, rc);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < CPT; ++j) acc[c * CPT + j] = __fadd_rn(__uint_as_float(rm[j]), __uint_as_float(rc[j]));
                    } else {
#pragma unroll
                        for (int j = 0; j < CPT; ++j) acc[c * CPT + j] = 0.f;
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars[ACC_EMPTY]));
                // ---- relaxation, row sums, split, hand-over, one pair of chunks (one slot of the table ring) at a time.
                // The loop is unrolled over the pairs so that every accumulator value is read from a fixed register
                // (a rolled loop has to shift the register array down after every pair, which cost 14 instructions per
                // coefficient, a quarter of the epilogue).
                const long tb = (long)d * P.nps + Ly.relu_off;
                const bool has_bias = Ly.bias != nullptr;
#pragma unroll
                for (int c2 = 0; c2 < MAX_CHUNKS; c2 += 2) {
                    if (c2 >= nch || dead) break;
                    const unsigned char *ts = nullptr;
                    int tslot = 0;
                    if constexpr (STAGED) {
                        tslot = tit % NT;
                        bool tok = mbar_wait(smem_u32(&bars[T_FULL + tslot]), (tit / NT) & 1);
                        tok = __all_sync(0xffffffffu, tok);
                        if (!tok) { if (lane == 0) { atomicExch(P.err, 24); *abort_flag = 1; } dead = true; break; }
                        ts = t_ring + tslot * T_SLOT + T_HEAD + dd * T_DOM;
                    }
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int c = c2 + h2;
                        if (c < nch && !dead) {
                            float v[CPT];
                            float sp_ = 0.f, gi = 0.f, gb = 0.f;
#pragma unroll
                            for (int g = 0; g < CPT / 4; ++g) {
                                const int col = c * BK + sub * CPT + 4 * g;
                                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (live && col < N) {
                                    float4 t0, t1, t2, t3, cj, bk = make_float4(0.f, 0.f, 0.f, 0.f);
                                    if constexpr (STAGED) {
                                        const int cl = h2 * BK + sub * CPT + 4 * g;   // column inside the staged pair
                                        const float4 *tp = (const float4 *)ts + cl;
                                        t0 = tp[0]; t1 = tp[1]; t2 = tp[2]; t3 = tp[3];
                                        cj = *(const float4 *)(ts + T_COLS * 16 + cl * 4);
                                        if (has_bias) bk = *(const float4 *)(t_ring + tslot * T_SLOT + cl * 4);
                                    } else {
                                        t0 = P.tab[tb + col]; t1 = P.tab[tb + col + 1]; t2 = P.tab[tb + col + 2]; t3 = P.tab[tb + col + 3];
                                        cj = *(const float4 *)(P.cj + tb + col);
                                        if (has_bias) bk = *(const float4 *)(Ly.bias + col);
                                    }
                                    float4 au = make_float4(t0.x, t1.x, t2.x, t3.x);
                                    if (P.aup) au = *(const float4 *)(P.aup + tb + col);
                                    const int b0 = (c2 + h2) * CPT + 4 * g;
                                    o.x = relax_coeff_fast(upper, dir, dirf, acc[b0], t0, au.x, cj.x, bk.x, gi, gb, sp_);
                                    o.y = relax_coeff_fast(upper, dir, dirf, acc[b0 + 1], t1, au.y, cj.y, bk.y, gi, gb, sp_);
                                    o.z = relax_coeff_fast(upper, dir, dirf, acc[b0 + 2], t2, au.z, cj.z, bk.z, gi, gb, sp_);
                                    o.w = relax_coeff_fast(upper, dir, dirf, acc[b0 + 3], t3, au.w, cj.w, bk.w, gi, gb, sp_);
                                    if (Ly.to_global) *(float4 *)(P.A_out + m * P.lda + col) = o;
                                }
                                v[4 * g] = o.x; v[4 * g + 1] = o.y; v[4 * g + 2] = o.z; v[4 * g + 3] = o.w;
                            }
                            // the two fp32 dot products of this slice join the binary64 bias (their roundings are part of cj)
                            sb += (double)gi + (double)gb;
                            spt = __fadd_ru(spt, sp_);
                            if (!Ly.to_global) {
                                if (wait_slot(23)) {
                                    put_chunk(ait % NA, v);
                                    publish(ait % NA);
                                    ++ait;
                                }
                            }
                        }
                    }
                    if constexpr (STAGED) {   // the pair's tables are consumed: the slot goes back to the producer
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars[T_EMPTY + tslot]));
                        ++tit;
                    }
                }
            }
            if (dead) break;
            // ---- the row's sums: the NSUB threads of a row add their shares (the arrays were cleared by the host;
            // two shares commute, so the result does not depend on their order)
            if (live) {
                atomicAdd(&P.rb[m], sb);
                atomicAdd(&P.rpen[m], (double)spt * 1.000002);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// Charge weights of the fused relaxation, one per (domain, column) of every fused layer and of the identity pass in
// front of the first contraction (see relax_coeff_fast): cj = eps * q + (gap + kappa) * max|z| + kappa * |bias|, all
// rounded upwards.  `ent` describes the blocks: offset and width inside a table row, q's per-domain stride, the bias,
// the contraction's rounding rate and whether the block is a ReLU (gap and intercept terms apply) or the top block.
struct PrepBlock { int off, n, relu; long q_ds; const float *bias; float eps; };
struct PrepParams { int n_blocks; PrepBlock blk[kMaxChain + 1]; };
__global__ void k_chain_prep(const __grid_constant__ PrepParams PP, int D, long nps, const float *__restrict__ zabs,
                             const float *__restrict__ q, float kappa, float *__restrict__ cj) {
    const int bi = blockIdx.y;
    const PrepBlock &B = PP.blk[bi];
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * B.n) return;
    const int d = (int)(t / B.n), j = (int)(t % B.n);
    const long o = (long)d * nps + B.off + j;
    const float qv = q[(long)d * B.q_ds + B.off + j];
    float c = __fmul_ru(B.eps, qv);
    if (B.bias) c = __fmaf_ru(kappa, fabsf(B.bias[j]), c);
    if (B.relu) c = __fmaf_ru(1.9073487e-7f /* 1.6 * 2^-23 */ + kappa * 1.001f, zabs[o], c);
    cj[o] = c;
}

}  // namespace chain

// Rounding rate of a fused contraction of length K against S = |A||W|: operand split 0.75 * 2^-20 (see
// nyb200_umma.cu); K/8 main steps of at most one fp32 ulp of the accumulated magnitude each; 2K/8 cross steps whose
// accumulator never exceeds 2^-10 S (|Al| <= 2^-11 |A|, |Wl| <= 2^-11 |W|); one rounding for main + cross.
double chain_eps(int K) {
    const int kc = (K + chain::BK - 1) / chain::BK;
    const double u23 = 1.1920928955078125e-07, u24 = 5.9604644775390625e-08;
    const double rep = 0.75 * 9.5367431640625e-07;
    const double main_steps = (double)(kc * (chain::BK / 8)) * u23;
    const double cross_steps = (double)(kc * 2 * (chain::BK / 8)) * u23 * 9.765625e-04 * 1.001;
    return rep + main_steps + cross_steps + u24 * 1.001;
}

// The constants of the charge weights (see k_chain_prep): kappa covers the fp32 dot products of the epilogue, which run
// over at most 16 columns per slice, plus the 2^-40 share of the binary64 additions; the rate of table block `block`
// is that of the contraction its relaxed coefficients enter (the unfused Linear_0 contraction for block 0, a fused one
// otherwise, the first fused one for the top block L-1).
float chain_kappa() { return 16.f * 5.9604645e-8f * 1.001f + 9.1e-13f; }
float chain_cj_eps(const Net &net, int L, int block) {
    const NetView &nv = net.v;
    const double eps = block == 0 ? umma_eps(nv.dims[1]) * 1.000001 : chain_eps(nv.dims[block + 1]) * 1.000001;
    (void)L;
    return (float)(eps * 1.0000002);
}

// Can the pass that starts at Linear_{L-1}'s output (L layers below it) run its contractions k = L-1 .. 1 fused?
bool chain_eligible(const Net &net, int L) {
    const NetView &nv = net.v;
    if (L < 2 || L - 1 > chain::kMaxChain) return false;
    if (nv.dims[L] > chain::BN) return false;
    for (int k = 0; k < L; ++k)
        if (net.is_conv(k) || net.skip_of(k) >= 0) return false;
    for (int k = 1; k < L; ++k)
        if (nv.dims[k] > chain::BN || (nv.dims[k] & 3) || (nv.pre_off[k - 1] & 3)) return false;
    return true;
}

// Launches the fused chain for the pass over layers L-1 .. 1 of the resident batch; the relaxed rows that enter
// Linear_0's contraction arrive in A_out, the row sums in p.rb / p.rpen.  eps0 is the rounding rate of that last,
// unfused contraction (charged by the relaxation in front of it).
int launch_chain(nyb200_engine *e, Net &net, const Batch &b, BatchPtrs &p, int L, bool identity_seed, bool shared_box,
                 float *A_out, double eps0, int *derr) {
    using namespace chain;
    const NetView &nv = net.v;
    Params P;  // ~5 KB, passed by value
    memset(&P, 0, sizeof(P));
    P.n_layers = L - 1;
    P.M = b.D * b.R; P.R = b.R; P.S = b.S;
    P.seed_identity = identity_seed ? 1 : 0;
    P.K_top = nv.dims[L];
    P.spec = p.spec;
    P.top_bias = nv.b[L - 1];
    P.top_off = nv.pre_off[L - 1];
    P.top_q_ds = nv.nps;
    P.top_eps = (float)(chain_eps(nv.dims[L]) * 1.000001 * 1.0000002);
    float *cj = p.cj;   // written by the interval pass of this run, or prepared below
    if (!cj) {
        cj = (float *)ws_get(e, "chain_cj", (size_t)b.D * nv.nps * 4);
        if (!cj) return NYB200_ERR_OOM;
    }
    P.tab = p.tab; P.zabs = p.zabs; P.q = p.q; P.aup = p.alpha_up; P.nps = nv.nps; P.cj = cj;
    PrepParams PP;
    memset(&PP, 0, sizeof(PP));
    int max_n = nv.dims[L];
    P.A_out = A_out; P.lda = p.lda; P.rb = p.rb; P.rpen = p.rpen; P.err = derr;
    for (int l = 0; l < L - 1; ++l) {
        const int k = L - 1 - l;  // contraction with W_k: K = dims[k + 1], N = dims[k]; then ReLU k-1 and the charges of lin k-1
        Layer &Ly = P.layer[l];
        memcpy(&Ly.tm_hi, net.umma[k].tm_hi, sizeof(CUtensorMap));
        memcpy(&Ly.tm_lo, net.umma[k].tm_lo, sizeof(CUtensorMap));
        Ly.K = nv.dims[k + 1]; Ly.N = nv.dims[k];
        Ly.relu_off = nv.pre_off[k - 1];
        Ly.q_ds = (k - 1 == 0 && shared_box) ? 0 : nv.nps;
        Ly.bias = nv.b[k - 1];
        const double eps = (k - 1 >= 1) ? chain_eps(nv.dims[k]) * 1.000001 : eps0;
        Ly.eps = (float)(eps * 1.0000002);
        Ly.to_global = (k == 1) ? 1 : 0;
        PrepBlock &B = PP.blk[l];
        B.off = Ly.relu_off; B.n = Ly.N; B.relu = 1; B.q_ds = Ly.q_ds; B.bias = Ly.bias; B.eps = Ly.eps;
        max_n = Ly.N > max_n ? Ly.N : max_n;
    }
    {
        PrepBlock &B = PP.blk[L - 1];  // the identity pass in front of the first contraction
        B.off = P.top_off; B.n = P.K_top; B.relu = 0; B.q_ds = P.top_q_ds; B.bias = P.top_bias; B.eps = P.top_eps;
        PP.n_blocks = L;
    }
    // kappa: the fp32 dot products run over at most 8 columns per slice (CPT of the narrowest epilogue slice is 8, of the
    // widest 16: charge the widest), plus the 2^-40 share of the binary64 additions
    const float kappa = chain_kappa();
    if (!p.cj) {
        dim3 grid((unsigned)(((long)b.D * max_n + 255) / 256), (unsigned)PP.n_blocks);
        k_chain_prep<<<grid, 256, 0, e->stream>>>(PP, b.D, (long)nv.nps, p.zabs, p.q, kappa, cj);
        e->launches++;
    }
    static std::mutex attr_mu;
    static bool attr_set[64] = {false};
    {
        std::lock_guard<std::mutex> g(attr_mu);
        const int dev = (e->device >= 0 && e->device < 64) ? e->device : 0;
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(k_chain<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
                cudaFuncSetAttribute(k_chain<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
                return set_err(e, NYB200_ERR_INTERNAL, "cannot raise the dynamic shared-memory limit");
            attr_set[dev] = true;
        }
    }
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, e->device);
    if (e->reserve_sms > 0 && sms > e->reserve_sms) sms -= e->reserve_sms;   // left to a concurrent collective
    const int tiles = (P.M + BM - 1) / BM;
    const int grid = tiles < sms ? tiles : sms;
    // a 128-row tile spans at most (BM - 2) / R + 2 domains; the table ring holds MAXD of them
    const bool staged = (BM - 2) / b.R + 2 <= MAXD;
    cudaError_t ls = staged ? launch_pdl(k_chain<4, true>, dim3(grid), dim3(Cfg<4>::THREADS), SMEM_BYTES, e, P)
                            : launch_pdl(k_chain<4, false>, dim3(grid), dim3(Cfg<4>::THREADS), SMEM_BYTES, e, P);
    if (ls != cudaSuccess) return set_err(e, NYB200_ERR_INTERNAL, "fused chain launch failed");
    e->launches++;
    return NYB200_OK;
}

}  // namespace nyb
