// tcgen05 contraction for the CROWN backward pass: C[M x N] = A[M x K] * W[K x N], fp32 in and out,
// computed as three TF32 tensor-core products on split operands (A = Ah + Al, W = Wh + Wl;
// Ah*Wh + Ah*Wl + Al*Wh) with fp32 accumulators in tensor memory.
//
// Layout of one CTA (persistent, one per SM, 384 threads):
//   warp 0      TMA producer: streams the pre-split, pre-transposed weight tiles Wh^T, Wl^T
//               (K-major, 128-byte swizzle) into shared memory, one 32-wide K chunk per stage.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=256, K=8, kind::tf32),
//               commits each stage back to the producers and each finished tile to the epilogue.
//   warp 2      allocates / frees the 512 tensor-memory columns (two 128x256 fp32 accumulators).
//   warps 4-7   epilogue: tcgen05.ld the accumulator (one TMEM lane = one output row per thread)
//               and store the fp32 rows to global memory; overlaps the next tile's MMAs.
//   warps 8-11  A producers: each thread owns one row of the 128-row tile, loads 32 fp32 of it,
//               splits every value into TF32 high and low parts and writes both to shared memory
//               in the swizzled K-major layout the tensor core reads.
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code, stops issuing
// work, frees its tensor memory and returns.
//
// Rounding model used for the soundness penalty (charged by the caller as eps * |A| . q):
//   representation: Ah, Wh are exact TF32 values; Al = rn_tf32(A - Ah), |A - Ah - Al| <= 2^-22 |A|
//   (same for W), the product Al*Wl (<= 2^-22 |A||W|) is dropped: total <= 0.75 * 2^-20 |A||W|;
//   accumulation: each tcgen05.mma step adds 8 exact products to the fp32 accumulator; the model
//   assumes the step's error is at most one fp32 ulp of the magnitude sum accumulated so far
//   (truncating adder), i.e. <= 2^-23 * S per step, so a chain of n steps is within n * 2^-23 * S.
#include <cuda.h>

#include "nyb200_internal.cuh"

namespace nyb {

namespace umma {

constexpr int BM = 128, BN = 256, BK = 32, STAGES = 2;
constexpr int A_BYTES = BM * BK * 4;   // 16 KB per half
constexpr int B_BYTES = BN * BK * 4;   // 32 KB per half
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr int THREADS = 384;
constexpr unsigned SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the limit expires.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (it > 1024) __nanosleep(64);
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap *tm, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tm), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// K-major, 128-byte swizzle shared-memory operand descriptor: start address >> 4 in bits [0,14),
// leading byte offset (unused for this layout) = 1 in [16,30), stride byte offset = 1024 B (8 rows of
// 128 B) >> 4 in [32,46), descriptor version 1 in [46,48), layout type 2 (128B swizzle) in [61,64).
__device__ __forceinline__ unsigned long long make_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);
    d |= 1ull << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor: D fp32 (bits [4,6) = 1), A and B TF32 (format 2 at [7,10) and [10,13)),
// both K-major, N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ unsigned make_idesc(int m, int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                         unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Round an fp32 value to the nearest TF32 value (10 explicit mantissa bits); ties away from zero.
__device__ __forceinline__ float rn_tf32(float x) {
    unsigned b = __float_as_uint(x);
    if ((b & 0x7f800000u) == 0x7f800000u) return x;
    b = (b + 0x1000u) & 0xffffe000u;
    return __uint_as_float(b);
}

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
              const float *__restrict__ A, int lda, float *__restrict__ C, int ldc, int M, int N, int K,
              int *__restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long *bars = (unsigned long long *)(smem + STAGES * STAGE_BYTES);
    // barrier indices
    const int FULL_A = 0, FULL_B = STAGES, EMPTY = 2 * STAGES, ACC_FULL = 3 * STAGES, ACC_EMPTY = 3 * STAGES + 2;
    unsigned *tmem_slot = (unsigned *)(bars + 3 * STAGES + 4);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    int total_tiles = m_tiles * n_tiles;
    int k_stages = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[FULL_A + s]), 128);
            mbar_init(smem_u32(&bars[FULL_B + s]), 1);
            mbar_init(smem_u32(&bars[EMPTY + s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars[ACC_FULL + b]), 1);
            mbar_init(smem_u32(&bars[ACC_EMPTY + b]), 128);
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
    unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- weight producer (TMA)
        if (lane == 0) {
            unsigned it = 0;
            for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
                int tn = t % n_tiles;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
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
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            unsigned idesc = make_idesc(BM, BN);
            unsigned it = 0, tile_it = 0;
            for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x, ++tile_it) {
                int buf = tile_it & 1;
                unsigned aph = (tile_it >> 1) & 1;
                if (!mbar_wait(smem_u32(&bars[ACC_EMPTY + buf]), aph ^ 1)) { atomicExch(err, 2); *abort_flag = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
                bool failed = false;
                for (int ks = 0; ks < k_stages; ++ks, ++it) {
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
#pragma unroll
                    for (int k4 = 0; k4 < BK / 8; ++k4) {
                        unsigned long long adv = (unsigned long long)(k4 * 2);  // 8 TF32 = 32 bytes = 2 x 16 B
                        unsigned acc0 = (ks > 0 || k4 > 0) ? 1u : 0u;
                        mma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, acc0);
                        mma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                        mma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                    }
                    mma_commit(smem_u32(&bars[EMPTY + s]));
                }
                if (failed) break;
                mma_commit(smem_u32(&bars[ACC_FULL + buf]));
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------------------------------------------------------- epilogue
        int q = warp & 3;
        unsigned tile_it = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_it) {
            int tm = t / n_tiles, tn = t % n_tiles;
            int buf = tile_it & 1;
            unsigned aph = (tile_it >> 1) & 1;
            bool ok = mbar_wait(smem_u32(&bars[ACC_FULL + buf]), aph);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) { atomicExch(err, 4); *abort_flag = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int row = tm * BM + q * 32 + lane;
            float *crow = C + (long)row * ldc + tn * BN;
            int ncols = min(BN, N - tn * BN);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                unsigned r[32];
                unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN + c);
                tmem_ld32(taddr, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < M && c < ncols) {
                    if (c + 32 <= ncols && ((ldc & 3) == 0)) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *(float4 *)(crow + c + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                     __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (c + j < ncols) crow[c + j] = __uint_as_float(r[j]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(smem_u32(&bars[ACC_EMPTY + buf]));
        }
    } else if (warp >= 8) {
        // ---------------------------------------------------------------- A producers (split to TF32 hi/lo)
        int r = threadIdx.x - 256;  // row of the tile owned by this thread
        unsigned it = 0;
        bool dead = false;
        for (int t = blockIdx.x; t < total_tiles && !dead; t += gridDim.x) {
            int tm = t / n_tiles;
            int row = tm * BM + r;
            const float *arow = A + (long)row * lda;
            for (int ks = 0; ks < k_stages; ++ks, ++it) {
                int s = it % STAGES;
                unsigned ph = (it / STAGES) & 1;
                if (!mbar_wait(smem_u32(&bars[EMPTY + s]), ph ^ 1)) { atomicExch(err, 5); *abort_flag = 1; dead = true; break; }
                unsigned char *st = smem + s * STAGE_BYTES;
                float *ah = (float *)st, *al = (float *)(st + A_BYTES);
                int k0 = ks * BK;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float v[4] = {0.f, 0.f, 0.f, 0.f};
                    int k = k0 + c * 4;
                    if (row < M) {
                        if (k + 3 < K && ((lda & 3) == 0)) {
                            float4 x = *(const float4 *)(arow + k);
                            v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) if (k + j < K) v[j] = arow[k + j];
                        }
                    }
                    float h[4], l[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) { h[j] = rn_tf32(v[j]); l[j] = rn_tf32(v[j] - h[j]); }
                    int off = r * 32 + ((c ^ (r & 7)) << 2);  // in floats: row * 128 B + swizzled 16 B chunk
                    *(float4 *)(ah + off) = make_float4(h[0], h[1], h[2], h[3]);
                    *(float4 *)(al + off) = make_float4(l[0], l[1], l[2], l[3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(smem_u32(&bars[FULL_A + s]));
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
static int make_tmap(CUtensorMap *tm, const float *base, int rows, int kpad) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return 1;
    cuuint64_t dims[2] = {(cuuint64_t)kpad, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)kpad * 4};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BN};
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

int launch_umma(nyb200_engine *e, const UmmaLayer &L, int M, const float *A, int lda, float *C, int ldc, int *err) {
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_umma_tf32x3, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return set_err(e, NYB200_ERR_INTERNAL, "cannot raise the dynamic shared-memory limit");
        attr_set = true;
    }
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, e->device);
    int tiles = ((M + BM - 1) / BM) * ((L.N + BN - 1) / BN);
    int grid = tiles < sms ? tiles : sms;
    k_umma_tf32x3<<<grid, THREADS, SMEM_BYTES, e->stream>>>(*(const CUtensorMap *)L.tm_hi, *(const CUtensorMap *)L.tm_lo, A,
                                                            lda, C, ldc, M, L.N, L.K, err);
    e->launches++;
    return NYB200_OK;
}

// Worst-case relative rounding of this kernel's product against S = |A||W| (see the model above).
double umma_eps(int K) {
    int steps = ((K + BK - 1) / BK) * (BK / 8) * 3;
    return 0.75 * 9.5367431640625e-07 /* 2^-20 */ + (double)steps * 1.1920928955078125e-07 /* 2^-23 */;
}

}  // namespace nyb
