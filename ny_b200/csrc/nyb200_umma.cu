// tcgen05 contraction for the CROWN backward pass: C[M x N] = A[M x K] * W[K x N], fp32 in and out,
// computed as three TF32 tensor-core products on split operands (A = Ah + Al, W = Wh + Wl;
// Ah*Wh + Ah*Wl + Al*Wh) with fp32 accumulators in tensor memory.
//
// Layout of one CTA (persistent, one per SM, 512 threads, register budget re-split with setmaxnreg):
//   warp 0      TMA producer: streams the pre-split, pre-transposed weight tiles Wh^T, Wl^T
//               (K-major, 128-byte swizzle) into shared memory, one 32-wide K chunk per stage.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=256, K=8, kind::tf32),
//               commits each stage back to the producers and each finished chunk to the epilogue.
//   warp 2      allocates / frees the 512 tensor-memory columns (two 128x256 fp32 accumulators).
//   warps 4-11  epilogue: a K range is accumulated in tensor memory only over a short chain
//               (CHUNK_STAGES stages of 12 MMA steps each); each finished chunk is read with tcgen05.ld (one
//               TMEM lane = one output row per thread, 128 columns per warp) and added in fp32
//               registers, alternating between the two accumulators so that the drain of one chunk
//               overlaps the MMAs of the next; the row sums are stored after the last chunk.
//   warps 12-15 A producers: each thread owns one row of the 128-row tile, takes 32 fp32 of it
//               (prefetched one stage ahead), splits every value into TF32 high and low parts and
//               writes both to shared memory in the swizzled K-major layout the tensor core reads.
//               The fp32 tile itself arrives by TMA in a two-deep ring of 16 KB staging buffers (warp 0
//               issues it next to the weight tiles), so the producers read their rows from shared
//               memory; with one row per lane a direct global load touches 32 sectors per instruction
//               and the load/store unit becomes the pipeline's bottleneck.  Operands a tensor map
//               cannot describe (unaligned base or row stride, the channel-strided convolution form)
//               take the direct loads.
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code, stops issuing
// work, frees its tensor memory and returns.
//
// Rounding model used for the soundness penalty (charged by the caller as eps * |A| . q):
//   representation: Ah, Wh are exact TF32 values; Al = rn_tf32(A - Ah), |A - Ah - Al| <= 2^-22 |A|
//   (same for W), the product Al*Wl (<= 2^-22 |A||W|) is dropped: total <= 0.75 * 2^-20 |A||W|;
//   accumulation: each tcgen05.mma step adds 8 exact products to the fp32 accumulator; the model
//   assumes the step's error is at most one fp32 ulp of the magnitude sum accumulated so far
//   (truncating adder), i.e. <= 2^-23 * (accumulated magnitude) per step.  Inside a chain the eight
//   cross-term steps are issued first, while the accumulator holds only terms of size 2^-10 S, so they
//   cost 8 * 2^-33 S; the four Ah*Wh steps cost 4 * 2^-23 S.  The chunk sums are added in
//   round-to-nearest fp32 (2^-24 * S each).  A chain holds CHUNK_STAGES stages: with two (the default) the
//   second stage's eight cross-term steps meet a full-size accumulator, so a chain costs
//   (8 + 8) * 2^-23 of its own magnitude instead of 4 * 2^-23, and the kernel hands an accumulator to the
//   epilogue half as often: 12% off the contraction time of the 8 x 256 network for a rate of 2.9e-6 instead of
//   1.7e-6 at K = 256.  Keeping the chain short (instead of 12 * K/32 steps) is what keeps the certified bounds
//   within 1e-4 of the binary64 path; a batch whose charge still shows is re-evaluated in binary64 by the caller.
#include <cuda.h>

#include <cstdlib>

#include "nyb200_internal.cuh"
#include "nyb200_tcgen05.cuh"

namespace nyb {

namespace umma {

constexpr int BM = 128, BN = 256, BK = 32, STAGES = 2;
constexpr int A_BYTES = BM * BK * 4;   // 16 KB per half
constexpr int B_BYTES = BN * BK * 4;   // 32 KB per half
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr int RAW_STAGES = 2;           // fp32 A tiles in flight between the TMA and the split
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RAW_STAGES * A_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
static_assert(SMEM_BYTES <= 232448, "more than the 227 KB a CTA can opt into");
constexpr int THREADS = 512;
// Register budget after the roles re-split it with setmaxnreg: 4 control warps, 8 epilogue warps, 4 producer warps.
// setmaxnreg.inc blocks until the registers it asks for have been released by the other warps' setmaxnreg.dec, so
// the targets must fit what the CTA was launched with (65536 / THREADS per thread); no bounded wait can catch a
// shortfall.
constexpr int REGS_LAUNCH = 65536 / THREADS, REGS_CONTROL = 40, REGS_EPILOGUE = 184, REGS_PRODUCER = 104;
static_assert(4 * 32 * REGS_CONTROL + 8 * 32 * REGS_EPILOGUE + 4 * 32 * REGS_PRODUCER <= THREADS * REGS_LAUNCH,
              "setmaxnreg targets exceed the CTA's register allocation: the epilogue's setmaxnreg.inc would block");
// K stages (of 32) accumulated in one tensor-memory chain before the chunk is drained: two for contractions of
// eight stages or more (K > 224), where halving the hand-offs to the epilogue pays (12% of the contraction time of
// the 8 x 256 network), one for shorter ones, which hand over at most seven times per tile anyway and whose callers
// (convolutions, narrow layers on small boxes) are the ones sensitive to the rounding rate.  The rounding model
// follows the value in use.
static int chunk_stages_cfg(int K) { return (K + BK - 1) / BK >= 8 ? 2 : 1; }
}  // namespace umma

using namespace umma;

// Splits W [K x N] (row-major) into TF32 high/low parts stored transposed and K-padded:
// Wh_T, Wl_T are [N x Kpad] row-major with zeros for k >= K.
__global__ void k_split_weights(const float *__restrict__ W, int K, int N, int Kpad, float *__restrict__ Wh,
                                float *__restrict__ Wl) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)N * Kpad) return;
    int n = (int)(t / Kpad), k = (int)(t % Kpad);
    float w = (k < K) ? W[(long)k * N + n] : 0.f;
    float h = rn_tf32(w);
    float l = rn_tf32(w - h);
    Wh[t] = h;
    Wl[t] = l;
}

__global__ void __launch_bounds__(THREADS, 1)
k_umma_tf32x3(const __grid_constant__ CUtensorMap tm_hi, const __grid_constant__ CUtensorMap tm_lo,
              const __grid_constant__ CUtensorMap tm_a, const float *__restrict__ A, int lda, float *__restrict__ C,
              int ldc, int M, int N, int K, int chunk_stages, int *__restrict__ err, int a_plane, int a_tma,
              const __grid_constant__ ConcFuse cf) {
    extern __shared__ unsigned char smem_raw[];
    // aligned by an offset (not by a cast through an integer) so that the compiler keeps treating it as shared memory
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *raw_base = smem + STAGES * STAGE_BYTES;  // RAW_STAGES fp32 A tiles (128-byte swizzle, as TMA wrote them)
    unsigned long long *bars = (unsigned long long *)(raw_base + RAW_STAGES * A_BYTES);
    // barrier indices
    const int FULL_A = 0, FULL_B = STAGES, EMPTY = 2 * STAGES, ACC_FULL = 3 * STAGES, ACC_EMPTY = 3 * STAGES + 2;
    const int RAW_FULL = 3 * STAGES + 4, RAW_EMPTY = RAW_FULL + RAW_STAGES;
    unsigned *tmem_slot = (unsigned *)(bars + 3 * STAGES + 4 + 2 * RAW_STAGES);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    pdl_trigger();   // the next kernel of the stream may be scheduled; it waits for this one's completion itself
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    int total_tiles = m_tiles * n_tiles;
    int k_stages = (K + BK - 1) / BK;
    int n_chunks = (k_stages + chunk_stages - 1) / chunk_stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[FULL_A + s]), 128);
            mbar_init(smem_u32(&bars[FULL_B + s]), 1);
            mbar_init(smem_u32(&bars[EMPTY + s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars[ACC_FULL + b]), 1);
            mbar_init(smem_u32(&bars[ACC_EMPTY + b]), 256);
        }
        for (int b = 0; b < RAW_STAGES; ++b) {
            mbar_init(smem_u32(&bars[RAW_FULL + b]), 1);
            mbar_init(smem_u32(&bars[RAW_EMPTY + b]), 128);
        }
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
    pdl_wait();      // everything above touched only this CTA's shared and tensor memory
    unsigned tmem_base = *tmem_slot;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_CONTROL));
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ weight producer (TMA)
            unsigned it = 0;
            // The fp32 A tile of pipeline step `step` (tile t, K stage ks) into the staging ring, once the producers
            // have taken the tile that used the slot before.  It runs one step ahead of the weight tiles.
            auto stage_a = [&](unsigned step, int t, int ks) -> bool {
                int rb = step % RAW_STAGES;
                unsigned rph = (step / RAW_STAGES) & 1;
                if (!mbar_wait(smem_u32(&bars[RAW_EMPTY + rb]), rph ^ 1)) return false;
                unsigned rbar = smem_u32(&bars[RAW_FULL + rb]);
                mbar_expect_tx(rbar, A_BYTES);
                tma_load_2d(smem_u32(raw_base + rb * A_BYTES), &tm_a, ks * BK, (t / n_tiles) * BM, rbar);
                return true;
            };
            if (a_tma && (int)blockIdx.x < total_tiles && !stage_a(0, blockIdx.x, 0)) { atomicExch(err, 6); *abort_flag = 1; }
            for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
                int tn = t % n_tiles;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
                    if (a_tma) {
                        int nks = ks + 1, nt = t;
                        if (nks == k_stages) { nks = 0; nt = t + gridDim.x; }
                        if (nt < total_tiles && !stage_a(it + 1, nt, nks)) { atomicExch(err, 6); *abort_flag = 1; break; }
                    }
                    int s = it % STAGES;
                    unsigned ph = (it / STAGES) & 1;
                    if (!mbar_wait(smem_u32(&bars[EMPTY + s]), ph ^ 1)) { atomicExch(err, 1); *abort_flag = 1; break; }
                    unsigned char *st = smem + s * STAGE_BYTES;
                    unsigned bar = smem_u32(&bars[FULL_B + s]);
                    mbar_expect_tx(bar, 2 * B_BYTES);
                    tma_load_2d(smem_u32(st + 2 * A_BYTES), &tm_hi, ks * BK, tn * BN, bar);
                    tma_load_2d(smem_u32(st + 2 * A_BYTES + B_BYTES), &tm_lo, ks * BK, tn * BN, bar);
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            unsigned it = 0, chunk_it = 0;
            bool failed = false;
            for (int t = blockIdx.x; t < total_tiles && !*abort_flag && !failed; t += gridDim.x) {
                // a partial column tile only multiplies the columns it has (rounded up to the MMA granule of 16)
                int n_eff = min(BN, (N - (t % n_tiles) * BN + 15) & ~15);
                unsigned idesc = make_idesc(BM, n_eff);
                for (int ch = 0; ch < n_chunks && !failed; ++ch, ++chunk_it) {
                    int buf = chunk_it & 1;
                    unsigned aph = (chunk_it >> 1) & 1;
                    if (!mbar_wait(smem_u32(&bars[ACC_EMPTY + buf]), aph ^ 1)) { atomicExch(err, 2); *abort_flag = 1; failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
                    int ks_end = min(k_stages, (ch + 1) * chunk_stages);
                    for (int ks = ch * chunk_stages; ks < ks_end; ++ks, ++it) {
                        int s = it % STAGES;
                        unsigned ph = (it / STAGES) & 1;
                        if (!mbar_wait(smem_u32(&bars[FULL_A + s]), ph) || !mbar_wait(smem_u32(&bars[FULL_B + s]), ph)) {
                            atomicExch(err, 3); *abort_flag = 1; failed = true; break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        unsigned char *st = smem + s * STAGE_BYTES;
                        unsigned long long a_hi = make_desc(smem_u32(st)), a_lo = make_desc(smem_u32(st + A_BYTES));
                        unsigned long long b_hi = make_desc(smem_u32(st + 2 * A_BYTES));
                        unsigned long long b_lo = make_desc(smem_u32(st + 2 * A_BYTES + B_BYTES));
                        // Small products first: the eight cross-term steps (|Al*Wh|, |Ah*Wl| <= 2^-10 |A||W|)
                        // run while the accumulator is still small, so only the four Ah*Wh steps round at
                        // the scale of S.
                        bool first = (ks == ch * chunk_stages);
#pragma unroll
                        for (int k4 = 0; k4 < BK / 8; ++k4) {
                            unsigned long long adv = (unsigned long long)(k4 * 2);  // 8 TF32 = 32 bytes = 2 x 16 B
                            mma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, (first && k4 == 0) ? 0u : 1u);
                            mma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                        }
#pragma unroll
                        for (int k4 = 0; k4 < BK / 8; ++k4) {
                            unsigned long long adv = (unsigned long long)(k4 * 2);
                            mma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
                        mma_commit(smem_u32(&bars[EMPTY + s]));
                    }
                    if (!failed) mma_commit(smem_u32(&bars[ACC_FULL + buf]));
                }
            }
        }
    } else if (warp < 12) {
        // ---------------------------------------------------------------- epilogue (8 warps)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_EPILOGUE));
        int q = warp & 3, half = (warp - 4) >> 2;
        unsigned chunk_it = 0;
        bool dead = false;
        for (int t = blockIdx.x; t < total_tiles && !dead; t += gridDim.x) {
            int tm = t / n_tiles, tn = t % n_tiles;
            const int col0 = tn * BN + half * 128;
            const int ncols = min(128, N - col0);
            float sum[128];
#pragma unroll
            for (int j = 0; j < 128; ++j) sum[j] = 0.f;
            for (int ch = 0; ch < n_chunks; ++ch, ++chunk_it) {
                int buf = chunk_it & 1;
                unsigned aph = (chunk_it >> 1) & 1;
                bool ok = mbar_wait(smem_u32(&bars[ACC_FULL + buf]), aph);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) { atomicExch(err, 4); *abort_flag = 1; } dead = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ncols > 0)
#pragma unroll
                for (int c = 0; c < 128; c += 32) {
                    if (c >= ncols) break;
                    unsigned r[32];
                    unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN + half * 128 + c);
                    tmem_ld32(taddr, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) sum[c + j] += __uint_as_float(r[j]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(smem_u32(&bars[ACC_EMPTY + buf]));
            }
            if (dead) break;
            int row = tm * BM + q * 32 + lane;
            if (a_plane > 0) {
                // transposed convolution: the products go out tap-major, C[(m * N + tap) * a_plane + p], so that
                // lanes (consecutive pixels p) write consecutive words and the col2im gather reads them the same way
                if (row < M && ncols > 0) {
                    float *cb = C + ((long)(row / a_plane) * N + col0) * a_plane + (row % a_plane);
#pragma unroll
                    for (int j = 0; j < 128; ++j) if (j < ncols) cb[(long)j * a_plane] = sum[j];
                }
            }
            if (cf.on && a_plane == 0 && row < M) {
                // fused concretisation: this thread's columns of the finished row against the input box
                double s = 0.0, sa = 0.0;
                bool bad = false;
                if (ncols > 0) {
                    const int d = row / cf.R, rr = row - d * cf.R;
                    const bool upper = rr >= cf.S;
                    const float *xl = cf.in_lo + (long)d * cf.box_ds + col0, *xu = cf.in_hi + (long)d * cf.box_ds + col0;
                    const bool vec = ncols == 128 && (((reinterpret_cast<uintptr_t>(xl) | reinterpret_cast<uintptr_t>(xu)) & 15) == 0);
                    auto term = [&](float a, float l, float u) {
                        const bool nonneg = !(__float_as_uint(a) >> 31) || (__float_as_uint(a) & 0x7fffffffu) == 0;
                        const float x = (nonneg != upper) ? l : u;
                        bad |= !(fabsf(a) < 1e10f);  // is_crown_coeff_safe, crates/ny-core/src/gemm.rs:127
                        // a zero factor contributes nothing, whatever the other one is (no 0 * inf)
                        const double c = (a != 0.f && x != 0.f) ? (double)a * (double)x : 0.0;
                        s += c; sa += fabs(c);
                    };
                    if (vec) {
#pragma unroll
                        for (int j = 0; j < 128; j += 4) {
                            const float4 l = *(const float4 *)(xl + j), u = *(const float4 *)(xu + j);
                            term(sum[j], l.x, u.x); term(sum[j + 1], l.y, u.y); term(sum[j + 2], l.z, u.z); term(sum[j + 3], l.w, u.w);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 128; ++j) if (j < ncols) term(sum[j], xl[j], xu[j]);
                    }
                }
                double *slot = cf.part + ((long)row * cf.slots + tn * 2 + half) * 2;
                slot[0] = s; slot[1] = sa;
                if (bad) cf.bad[row] = 1;
            }
            if (a_plane > 0 || (cf.on && !cf.store)) {
            } else if (row < M && ncols > 0) {
                float *crow = C + (long)row * ldc + col0;
                if (ncols == 128 && ((reinterpret_cast<uintptr_t>(crow) & 31) == 0)) {
                    // 32-byte stores: every instruction writes whole sectors of this thread's row
#pragma unroll
                    for (int j = 0; j < 128; j += 8)
                        asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(crow + j), "f"(sum[j]),
                                     "f"(sum[j + 1]), "f"(sum[j + 2]), "f"(sum[j + 3]), "f"(sum[j + 4]), "f"(sum[j + 5]),
                                     "f"(sum[j + 6]), "f"(sum[j + 7])
                                     : "memory");
                } else if (ncols == 128 && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
                    for (int j = 0; j < 128; j += 4) *(float4 *)(crow + j) = make_float4(sum[j], sum[j + 1], sum[j + 2], sum[j + 3]);
                } else if ((reinterpret_cast<uintptr_t>(crow) & 15) == 0) {
                    // partial column tile: whole 16-byte groups of this thread's row, then the ragged tail
#pragma unroll
                    for (int j = 0; j < 128; j += 4) {
                        if (j + 3 < ncols) *(float4 *)(crow + j) = make_float4(sum[j], sum[j + 1], sum[j + 2], sum[j + 3]);
                        else {
                            if (j < ncols) crow[j] = sum[j];
                            if (j + 1 < ncols) crow[j + 1] = sum[j + 1];
                            if (j + 2 < ncols) crow[j + 2] = sum[j + 2];
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 128; ++j) if (j < ncols) crow[j] = sum[j];
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- A producers (split to TF32 hi/lo)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_PRODUCER));
        int r = threadIdx.x - 384;  // row of the tile owned by this thread
        unsigned it = 0;
        bool dead = false;
        float4 v[8];
        auto load_stage = [&](int t, int ks) {
            int row = (t / n_tiles) * BM + r;
            int k0 = ks * BK;
            if (a_plane > 0) {
                // Channel-strided operand (transposed convolution): GEMM row = (coefficient row m, pixel p),
                // element k = channel k of that pixel, stored at A[m * lda + k * a_plane + p].  Lanes hold
                // consecutive pixels, so every k is one coalesced load across the warp.
                const float *base = A + (long)(row / a_plane) * lda + (row % a_plane);
                const bool in = row < M;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    int k = k0 + c * 4;
                    float4 x;
                    x.x = (in && k < K) ? base[(long)k * a_plane] : 0.f;
                    x.y = (in && k + 1 < K) ? base[(long)(k + 1) * a_plane] : 0.f;
                    x.z = (in && k + 2 < K) ? base[(long)(k + 2) * a_plane] : 0.f;
                    x.w = (in && k + 3 < K) ? base[(long)(k + 3) * a_plane] : 0.f;
                    v[c] = x;
                }
                return;
            }
            const float *arow = A + (long)row * lda;
            if (row < M && k0 + BK <= K && ((reinterpret_cast<uintptr_t>(arow + k0) & 15) == 0)) {
                // whole, aligned chunk (the usual case): eight unconditional 16-byte loads
#pragma unroll
                for (int c = 0; c < 8; ++c) v[c] = *(const float4 *)(arow + k0 + c * 4);
                return;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                int k = k0 + c * 4;
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row < M) {
                    if (k + 3 < K && ((reinterpret_cast<uintptr_t>(arow + k) & 15) == 0)) x = *(const float4 *)(arow + k);
                    else {
                        if (k < K) x.x = arow[k];
                        if (k + 1 < K) x.y = arow[k + 1];
                        if (k + 2 < K) x.z = arow[k + 2];
                        if (k + 3 < K) x.w = arow[k + 3];
                    }
                }
                v[c] = x;
            }
        };
        // Staged form: this thread's row of the fp32 tile of pipeline step `step`, out of the TMA ring.  Chunk c of
        // row r sits at chunk c ^ (r & 7) of the row's 128 bytes; a quarter-warp reads eight different chunks.
        auto take_staged = [&](unsigned step) -> bool {
            int rb = step % RAW_STAGES;
            unsigned rph = (step / RAW_STAGES) & 1;
            if (!mbar_wait(smem_u32(&bars[RAW_FULL + rb]), rph)) return false;
            const float *raw = (const float *)(raw_base + rb * A_BYTES);
#pragma unroll
            for (int c = 0; c < 8; ++c) v[c] = *(const float4 *)(raw + r * 32 + ((c ^ (r & 7)) << 2));
            // The slot is refilled by the async proxy (TMA) once all 128 threads have arrived: order this thread's
            // generic-proxy reads before that write.  Without the fence later tiles of a CTA were seen to read a
            // refilled slot whenever the tensor core, not the loads, paced the pipeline.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&bars[RAW_EMPTY + rb]));
            return true;
        };
        if ((int)blockIdx.x < total_tiles) {
            if (a_tma) { if (!take_staged(0)) { atomicExch(err, 7); *abort_flag = 1; dead = true; } }
            else load_stage(blockIdx.x, 0);
        }
        for (int t = blockIdx.x; t < total_tiles && !dead; t += gridDim.x) {
            for (int ks = 0; ks < k_stages; ++ks, ++it) {
                int s = it % STAGES;
                unsigned ph = (it / STAGES) & 1;
                if (!mbar_wait(smem_u32(&bars[EMPTY + s]), ph ^ 1)) { atomicExch(err, 5); *abort_flag = 1; dead = true; break; }
                unsigned char *st = smem + s * STAGE_BYTES;
                float *ah = (float *)st, *al = (float *)(st + A_BYTES);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float4 x = v[c];
                    float4 h = make_float4(rn_tf32(x.x), rn_tf32(x.y), rn_tf32(x.z), rn_tf32(x.w));
                    float4 l = make_float4(rn_tf32(x.x - h.x), rn_tf32(x.y - h.y), rn_tf32(x.z - h.z), rn_tf32(x.w - h.w));
                    int off = r * 32 + ((c ^ (r & 7)) << 2);  // in floats: row * 128 B + swizzled 16 B chunk
                    *(float4 *)(ah + off) = h;
                    *(float4 *)(al + off) = l;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(smem_u32(&bars[FULL_A + s]));
                // prefetch the next stage's row segment while the tensor core works on this one
                int nks = ks + 1, nt = t;
                if (nks == k_stages) { nks = 0; nt = t + gridDim.x; }
                if (nt < total_tiles) {
                    if (a_tma) { if (!take_staged(it + 1)) { atomicExch(err, 7); *abort_flag = 1; dead = true; break; } }
                    else load_stage(nt, nks);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || !p) return nullptr;
    fn = (EncodeTiledFn)p;
    return fn;
}

// Tensor map over a [rows x kpad] fp32 matrix (K contiguous): box 32 (K) x 256 (rows), 128-byte swizzle,
// out-of-range elements read as zero.
static int make_tmap(CUtensorMap *tm, const float *base, int rows, int kpad, int ld = 0, int box_rows = BN) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return 1;
    cuuint64_t dims[2] = {(cuuint64_t)kpad, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(ld > 0 ? ld : kpad) * 4};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2;
}

int umma_prepare_layer(nyb200_engine *e, const float *W, int K, int N, UmmaLayer *out) {
    int kpad = (K + BK - 1) / BK * BK;
    size_t n = (size_t)N * kpad;
    float *wh = nullptr, *wl = nullptr;
    if (cudaMalloc(&wh, n * 4) != cudaSuccess) return NYB200_ERR_OOM;
    if (cudaMalloc(&wl, n * 4) != cudaSuccess) { cudaFree(wh); return NYB200_ERR_OOM; }
    k_split_weights<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(W, K, N, kpad, wh, wl);
    e->launches++;
    out->wh = wh; out->wl = wl; out->K = K; out->N = N; out->kpad = kpad;
    static_assert(sizeof(CUtensorMap) == sizeof(out->tm_hi), "tensor map storage size");
    if (make_tmap((CUtensorMap *)out->tm_hi, wh, N, kpad) || make_tmap((CUtensorMap *)out->tm_lo, wl, N, kpad))
        return set_err(e, NYB200_ERR_INTERNAL, "cuTensorMapEncodeTiled failed");
    return NYB200_OK;
}

int launch_umma(nyb200_engine *e, const UmmaLayer &L, int M, const float *A, int lda, float *C, int ldc, int *err,
                int a_plane, const ConcFuse *cf) {
    // the attribute is a per-device property of the function: set it once on every device that launches it
    static std::mutex attr_mu;
    static bool attr_set[64] = {false};
    {
        std::lock_guard<std::mutex> g(attr_mu);
        const int dev = (e->device >= 0 && e->device < 64) ? e->device : 0;
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(k_umma_tf32x3, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
                return set_err(e, NYB200_ERR_INTERNAL, "cannot raise the dynamic shared-memory limit");
            attr_set[dev] = true;
        }
    }
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, e->device);
    if (e->reserve_sms > 0 && sms > e->reserve_sms) sms -= e->reserve_sms;   // left to a concurrent collective
    int tiles = ((M + BM - 1) / BM) * ((L.N + BN - 1) / BN);
    int grid = tiles < sms ? tiles : sms;
    // The fp32 operand goes through TMA when a tensor map can describe it: rows of K contiguous values, base and row
    // stride multiples of 16 bytes.  Columns past K and rows past M read as zero, like the direct loads.
    alignas(64) CUtensorMap tm_a;
    int a_tma = 0;
    if (a_plane == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (lda & 3) == 0 && lda >= L.K) {
        if (make_tmap(&tm_a, A, M, L.K, lda, BM)) return set_err(e, NYB200_ERR_INTERNAL, "cuTensorMapEncodeTiled failed for the A operand");
        a_tma = 1;
    } else {
        tm_a = *(const CUtensorMap *)L.tm_hi;  // unused by the kernel in this form; any valid map
    }
    ConcFuse none;
    if (launch_pdl(k_umma_tf32x3, dim3(grid), dim3(THREADS), SMEM_BYTES, e, *(const CUtensorMap *)L.tm_hi,
                   *(const CUtensorMap *)L.tm_lo, tm_a, A, lda, C, ldc, M, L.N, L.K, L.chain > 0 ? L.chain : chunk_stages_cfg(L.K), err,
                   a_plane, a_tma, cf ? *cf : none) != cudaSuccess)
        return set_err(e, NYB200_ERR_INTERNAL, "contraction kernel launch failed");
    e->launches++;
    return NYB200_OK;
}

// (W+^T | W-^T) as a row-major [n_in x 2 n_out] matrix from W [n_out x n_in].
__global__ void k_build_wpm(const float *__restrict__ W, int n_in, int n_out, float *__restrict__ out) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)n_in * 2 * n_out) return;
    int k = (int)(t / (2 * n_out)), n = (int)(t % (2 * n_out));
    float w = W[(long)(n % n_out) * n_in + k];
    out[t] = (n < n_out) ? fmaxf(w, 0.f) : fminf(w, 0.f);
}

int umma_prepare_forward_layer(nyb200_engine *e, const float *W, int n_in, int n_out, UmmaLayer *out) {
    float *tmp = nullptr;
    size_t n = (size_t)n_in * 2 * n_out;
    if (cudaMalloc(&tmp, n * 4) != cudaSuccess) return NYB200_ERR_OOM;
    k_build_wpm<<<(unsigned)((n + 255) / 256), 256, 0, e->stream>>>(W, n_in, n_out, tmp);
    e->launches++;
    int st = umma_prepare_layer(e, tmp, n_in, 2 * n_out, out);
    // interval products keep one stage per chain: their slack is compared against every unstable neuron's width
    // and compounds through the layers, where the coefficient products' charge is only compared against the bound
    out->chain = 1;
    cudaStreamSynchronize(e->stream);
    cudaFree(tmp);
    return st;
}

// Interval bounds of Linear_k from Fl = zl (W+|W-) and Fu = zu (W+|W-), valid for 0 <= zl <= zu:
// lo = W+ zl + W- zu + b, hi = W+ zu + W- zl + b, q = |W| zu = W+ zu - W- zu.  Every product carries a
// rounding of at most eps times the sum of its own term magnitudes, each of which is bounded by q, so
// both ends move outward by eps * q (q itself inflated by its own relative error) before the directed cast.
__global__ void k_ibp_combine(int D, int n_out, const float *__restrict__ Fl, const float *__restrict__ Fu, int ldf,
                              const float *__restrict__ bias, double eps, float *__restrict__ raw_lo,
                              float *__restrict__ raw_hi, float *__restrict__ q, long out_ds) {
    long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)D * n_out) return;
    int d = (int)(t / n_out), o = (int)(t % n_out);
    double pl = Fl[(long)d * ldf + o], nl = Fl[(long)d * ldf + n_out + o];
    double pu = Fu[(long)d * ldf + o], nu = Fu[(long)d * ldf + n_out + o];
    double b = bias ? (double)bias[o] : 0.0;
    double qq = (fabs(pu) + fabs(nu)) / (1.0 - 2.0 * eps);
    double slack = eps * qq + 2.3e-16 * (qq + fabs(b));
    float lf = __double2float_rd(pl + nu + b - slack);
    float hf = __double2float_ru(pu + nl + b + slack);
    if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
    raw_lo[(long)d * out_ds + o] = lf;
    raw_hi[(long)d * out_ds + o] = hf;
    q[(long)d * out_ds + o] = __double2float_ru(qq);
}

void launch_ibp_combine(nyb200_engine *e, int D, int n_out, const float *Fl, const float *Fu, int ldf, const float *bias,
                        double eps, float *raw_lo, float *raw_hi, float *q, long out_ds) {
    long total = (long)D * n_out;
    k_ibp_combine<<<(unsigned)((total + 255) / 256), 256, 0, e->stream>>>(D, n_out, Fl, Fu, ldf, bias, eps, raw_lo, raw_hi, q,
                                                                          out_ds);
    e->launches++;
}

// Worst-case relative rounding of this kernel's product against S = |A||W| (see the model above).
double umma_eps(int K, int chain) {
    int k_stages = (K + BK - 1) / BK;
    const int CS = chain > 0 ? chain : chunk_stages_cfg(K);
    int cs = k_stages < CS ? k_stages : CS;
    int chunks = (k_stages + CS - 1) / CS;
    const double u23 = 1.1920928955078125e-07, u24 = 5.9604644775390625e-08;
    double rep = 0.75 * 9.5367431640625e-07;                    // operand split, 0.75 * 2^-20
    double chain_main = (double)(cs * (BK / 8)) * u23;          // Ah*Wh steps round at the scale of S
    // the cross-term steps of a chain's first stage meet an accumulator of size 2^-10 S, those of its later
    // stages a full-size one
    double chain_cross = (double)((BK / 8) * 2) * u23 * ((double)(cs - 1) + 9.765625e-04 /* 2^-10 */);
    return rep + chain_main + chain_cross + (double)chunks * u24;
}

}  // namespace nyb
