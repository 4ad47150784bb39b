// Pieces shared by the decode GEMV kernels (qgemv.cu, qgemv_k.cu): the bounded mbarrier wait
// and the 1-D bulk copy that feed their per-warp shared-memory rings.
#pragma once

#include "tpb_internal.h"

namespace tpb_gemv {

constexpr long long kWaitLimitCycles = 2000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: false when the limit ran out (status word written).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t *status,
                                          uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u && clock64() - t0 > kWaitLimitCycles) {
            atomicCAS(status, 0u, code);
            return false;
        }
    }
}
// Exact int -> float for |v| < 2^22 on the ALU/FMA pipes: 0x4B400000 is 1.5 * 2^23 as a float, where
// one unit in the last place is 1, so adding v to the bit pattern adds v to the value.  The
// cvt instruction gives the same bits but issues at a quarter of the rate, which made it the
// limiter of the GEMVs with several activation rows (one conversion per block, row and column).
constexpr int kI2FMagicBits = 0x4B400000;
constexpr float kI2FMagic = 12582912.0f;
__device__ __forceinline__ float i2f_small(int v) { return __int_as_float(v + kI2FMagicBits) - kI2FMagic; }

// Untiled bulk copy global -> shared; both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

}  // namespace tpb_gemv
