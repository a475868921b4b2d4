// Inline-PTX building blocks shared by the tcgen05 kernels: bounded mbarrier waits, TMA tile loads, shared-memory
// operand and instruction descriptors for kind::tf32, MMA issue / commit, tensor-memory loads, TF32 rounding.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace nyb {
namespace umma {

constexpr unsigned WAIT_HINT_NS = 20000;                 // per probe: up to 20 us parked
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;    // per wait: about two seconds of SM clock

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
// Bounded wait: returns false when the limit expires.  Every probe carries a suspend-time hint, so a waiting warp is
// parked by the hardware until the phase completes (or the hint runs out) instead of competing for issue slots with
// the warps that do the work; the bound is on elapsed SM cycles (about two seconds), read only between probes.
__device__ __forceinline__ bool mbar_probe(unsigned bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// sleep_ns > 0: the caller is a role that runs ahead of the work (a producer, the MMA issuer waiting for operands);
// after a failed probe it sleeps that long, so that it does not take issue slots from the warps it is waiting for.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, unsigned sleep_ns = 0) {
    if (mbar_probe(bar, parity, WAIT_HINT_NS)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (sleep_ns) __nanosleep(sleep_ns);
        if (mbar_probe(bar, parity, WAIT_HINT_NS)) return true;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
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

// Round an fp32 value to the nearest TF32 value (10 explicit mantissa bits), ties away from zero.
__device__ __forceinline__ float rn_tf32(float x) {
    // Half an ulp of the 10-bit mantissa added to the magnitude bits, then the 13 low bits cleared: the value
    // cvt.rna.tf32.f32 returns (a carry into the exponent is the correct rounding to the next binade or to
    // infinity; infinities and NaNs keep their class), in two full-rate integer instructions instead of one
    // conversion-pipe instruction.
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}


}  // namespace umma
}  // namespace nyb
