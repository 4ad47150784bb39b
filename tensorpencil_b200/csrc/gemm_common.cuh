// Device helpers shared by the tcgen05 GEMM kernels: PTX wrappers (mbarrier, TMA,
// tcgen05), descriptor builders and the tile configuration.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdint>
#include <cstring>

#include "tpb_internal.h"

namespace tpb_gemm {

constexpr int BM = 128;            // rows of q per tile (= UMMA M)
constexpr int BK = 128;            // int8 elements (= bytes) of K per stage: one 128B swizzle row
constexpr int UMMA_K = 32;         // K of one tcgen05.mma.kind::i8
constexpr int kThreads = 192;      // 6 warps
constexpr long long kWaitLimitCycles = 2000000000ll;  // ~1 s: far beyond any legitimate wait

enum OutKind { OUT_F32 = 0, OUT_BF16 = 1, OUT_S32 = 2 };

template <int BN>
struct TileCfg {
    static constexpr int kStageBytesA = BM * BK;
    static constexpr int kStageBytesB = BN * BK;
    static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers (power of two >= 32)
    // epilogue staging: 4 warps x 2 buffers x (32 rows x 128 bytes)
    static constexpr int kStagingBytes = 4 * 2 * 4096;
    // tiles + staging + barriers (full/empty per stage, full/empty per accumulator)
    // + TMEM base slot + abort flag, plus 1 KB slack to align the tiles to 1024 bytes.
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

constexpr int kMaxPeers = 7;  // world size <= 8

struct GemmParams {
    void *y;
    long long ldy;
    const float *act_scale;
    const float *w_scale;
    const int32_t *act_sum;  // non-null: subtract 8 * act_sum[row] (unsigned-nibble weights)
    int m, n, k;
    uint32_t *status;
    // Fused all-gather: every output piece is also written, at the same (row, column)
    // and with the same ldy, into these peer-mapped buffers (other GPUs' copies of y).
    int n_peers;
    void *peer_y[kMaxPeers];
    // Or one NVSwitch multicast address of y (same row, column and ldy): a single
    // multimem store lands in every GPU's copy, this GPU's included.
    void *mc_y;
    // Gated residual (epilogue mode 3, f32 only): y is the residual stream x and the
    // epilogue stores x + gate[col] * (acc * act_scale * w_scale) back into it.
    const float *gate;
    // Paired weights (two-CTA kernel, PAIR mode): the scales of the second weight; the output is
    // silu(gate projection) * (up projection), n columns wide.
    const float *w_scale2 = nullptr;
    // Diagnosis only (TPB_GEMM_ABLATE, two-CTA kernel): bit 0 = issue no loads of q, bit 1 = no loads
    // of w, bit 2 = no epilogue (accumulators are handed back unread), bit 3 = the epilogue only
    // reads the accumulators out of tensor memory, bit 4 = it also converts and stages them in
    // shared memory but issues no stores.  Results are meaningless; the timings show what each
    // part of the pipeline costs the tensor pipe.
    int ablate;
};

// ---- PTX wrappers -----------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
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

// Bounded wait.  Returns false when the limit ran out or another role already
// gave up; the caller then leaves its loop.  `code` identifies the waiter.
// `relaxed` waiters (roles with slack: epilogue, TMA producer) sleep between polls so
// they do not take issue slots from the warps doing the work; latency-critical waiters
// (MMA issue, unpack) poll flat out.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                            uint32_t *status, uint32_t code, bool relaxed) {
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (relaxed) __nanosleep(it < 8 ? 32 : 128);
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                atomicCAS(status, 0u, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          uint32_t *status, uint32_t code, bool relaxed = false) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code, relaxed);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets row (lane
// base + t), registers 0..31 = columns col..col+31.
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Same wait, but naming the destination registers of the load as in/out operands
// so that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tc_wait_ld_dep(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                   "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]),
                   "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]),
                   "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]),
                   "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void st_global_v4(void *addr, uint4 v) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void multimem_st_v4(void *addr, uint4 v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// TMA store of one staged box (shared -> global); rows/columns outside the tensor are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle
// layout TMA writes: rows of 128 bytes, 8-row groups 1024 bytes apart.
//   bits  0-13 start address >> 4     bits 16-29 leading byte offset >> 4 (unused here)
//   bits 32-45 stride byte offset >> 4 (1024)   bits 46-47 descriptor version (1)
//   bits 61-63 layout (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::i8: int32 accumulate, A signed int8, B signed or
// unsigned int8, both K-major, N at bits 17-22 (N/8), M at bits 24-28 (M/16).
template <int BN>
__device__ __forceinline__ uint32_t make_idesc_i8(bool b_unsigned) {
    uint32_t d = 0;
    d |= 2u << 4;                       // accumulator format S32
    d |= 1u << 7;                       // A: signed 8-bit
    d |= (b_unsigned ? 0u : 1u) << 10;  // B: signed / unsigned 8-bit
    d |= (uint32_t)(BN >> 3) << 17;
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}

// ---- CTA-pair (cta_group::2) helpers ------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// cluster-window address of `addr` (a shared::cta address) in CTA `rank`
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are counted on a barrier that may live in
// the peer CTA of the pair (cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc2_commit(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
                 : "memory");
}
__device__ __forceinline__ void tc2_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// kind::i8, M = 256 across the pair, N = 256, both operands K-major
__device__ __forceinline__ uint32_t make_idesc2_i8(bool b_unsigned) {
    uint32_t d = 0;
    d |= 2u << 4;
    d |= 1u << 7;
    d |= (b_unsigned ? 0u : 1u) << 10;
    d |= (uint32_t)(256 >> 3) << 17;
    d |= (uint32_t)(256 >> 4) << 24;
    return d;
}

// Epilogue of one 128 x BN tile for one warp (32 accumulator rows starting at
// TMEM address t_row): load 32 columns at a time (the next load in flight while
// the current columns are processed), dequantise, stage 32 rows x 128 bytes in the
// warp's swizzled staging buffer and hand each full piece to a TMA store.
// PEERS is the epilogue mode.  3 = gated residual: read the tile of y, add gate[col] times
// the dequantised result, store it back (GemmParams::gate).  Modes of the fused all-gather:
// 1 = also write every piece to GemmParams::peer_y with plain
// stores; 2 = write every piece once, to the multicast address GemmParams::mc_y, instead of
// the local TMA store.  A template parameter so that the ordinary kernels carry none of it.
template <int BN, int OUT, int PEERS = 0, bool LEAN = false, bool ONE_STG = LEAN>
__device__ __forceinline__ void epilogue_tile(uint32_t t_row, const GemmParams &p, const CUtensorMap *tma_y,
                                              uint32_t stg, uint32_t my_row_off, uint32_t sw, uint32_t &n_store,
                                              int row0, int n0, float as, int corr, int lane,
                                              const float *w_scale_in = nullptr) {
    const float *w_scale = w_scale_in != nullptr ? w_scale_in : p.w_scale;   // the weight's scales (several weights per launch)
    // LEAN (the gated mode with eight epilogue warps, 168 registers per thread): the accumulators are read through
    // one register buffer instead of two and the residual one piece ahead instead of two.  ONE_STG (eight epilogue
    // warps, 4 KB of staging each): a piece is staged in one buffer, whose previous store must have been read out first.
    constexpr bool kOneTmemBuf = LEAN;
    uint32_t ra[32], rb[32];
    tc_ld_32x32(t_row, ra);
    // Gated residual: the 32 x 32 pieces of the residual stream this warp updates, read kPre pieces ahead of
    // their use with whole-line loads (eight lanes per 128-byte row segment, four rows per instruction) and
    // turned into "one row per lane" through the staging buffer.  A lane reading its own row 16 bytes at a
    // time touches 32 half-used sectors per warp instruction: K = 3072 took 87 us that way against 38 us for
    // the plain GEMM (more of those loads in flight made it worse: 102 us).  L2-only loads: the tile is
    // rewritten below through the TMA (async proxy), which does not update a line such a load would leave in
    // L1, and a dependent kernel that was launched early on this SM could then read the old values from it.
    constexpr int kPre = LEAN ? 1 : 2;
    float4 xr[PEERS == 3 ? kPre : 1][8];
    auto load_residual = [&](int c, float4 (&dst)[8]) {
        const int col = n0 + c * 32 + 4 * (lane & 7);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int r = row0 + 4 * i + (lane >> 3);
            dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < p.m && col < p.n)
                dst[i] = __ldcg(reinterpret_cast<const float4 *>(static_cast<const float *>(p.y) + (size_t)r * (size_t)p.ldy + col));
        }
    };
    if (PEERS == 3) {
#pragma unroll
        for (int c = 0; c < kPre && c < BN / 32; c++) load_residual(c, xr[c]);
    }
    // The 32 per-column scales of a piece (and the gate values in the gated mode), loaded one piece ahead
    // of their use into two register sets.  Loaded where they were used, inside the conversion loop, each of
    // the eight loads of a piece stalled its first multiply for an L1 round trip: half the epilogue's time
    // (measured at K = 256, where the epilogue is all there is).
    // (The gated mode, which also keeps residual pieces in registers, has room for one set only: it loads a
    // piece's scales at the top of the piece, ahead of the wait for the accumulators.)
    constexpr bool kTwoSets = PEERS != 3;
    float4 wsa[8], wsb[kTwoSets ? 8 : 1], gta[PEERS == 3 ? 8 : 1];
    auto load_scales = [&](int c, float4 (&w)[8]) {
        const int col0 = n0 + c * 32;
#pragma unroll
        for (int g = 0; g < 8; g++) {
            w[g] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (OUT != OUT_S32 && col0 + 4 * g < p.n) w[g] = __ldg(reinterpret_cast<const float4 *>(w_scale + col0 + 4 * g));
            if (PEERS == 3) {
                gta[g] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (col0 + 4 * g < p.n) gta[g] = __ldcg(reinterpret_cast<const float4 *>(p.gate + col0 + 4 * g));
            }
        }
    };
    if (kTwoSets) load_scales(0, wsa);
#pragma unroll
    for (int c = 0; c < BN / 32; c++) {
        uint32_t(&cur)[32] = (!kOneTmemBuf && (c & 1)) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        float4(&wsc)[8] = (kTwoSets && (c & 1)) ? reinterpret_cast<float4(&)[8]>(wsb) : wsa;
        float4(&gtc)[PEERS == 3 ? 8 : 1] = gta;
        if (kTwoSets) {
            if (c + 1 < BN / 32) load_scales(c + 1, (c & 1) ? wsa : reinterpret_cast<float4(&)[8]>(wsb));
        } else {
            load_scales(c, wsa);
        }
        tc_wait_ld_dep(cur);  // columns 32c.. are in `cur`
        if (!kOneTmemBuf && c + 1 < BN / 32) tc_ld_32x32(t_row + (uint32_t)((c + 1) * 32), nxt);
        const int col0 = n0 + c * 32;
        // first piece of a 128-byte staging row: make sure the TMA store that last
        // read this buffer (two stores ago) is done with it
        const bool first_piece = OUT != OUT_BF16 || (c & 1) == 0;
        const uint32_t buf = stg + (ONE_STG ? 0u : (n_store & 1u) * 4096u) + my_row_off;
        // Warp-uniform: does this 128-byte-wide piece reach into the tensor at all?
        // Skipped pieces touch neither the staging buffers nor the buffer counter,
        // so "all but the latest store have finished reading" keeps meaning "the
        // other buffer's store".
        const int scol = (OUT == OUT_BF16 && (c & 1)) ? col0 - 32 : col0;
        const bool do_store = row0 < p.m && scol < p.n && !(p.ablate & 8);
        if (!do_store) {
            if (kOneTmemBuf && c + 1 < BN / 32) tc_ld_32x32(t_row + (uint32_t)((c + 1) * 32), ra);
            continue;
        }
        if (first_piece) {
            if (lane == 0) {
                if (ONE_STG) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // one staging buffer
                else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
            __syncwarp();
        }
        if (OUT == OUT_S32) {
#pragma unroll
            for (int g = 0; g < 8; g++)
                st_shared_v4(buf + ((((uint32_t)g) ^ sw) << 4), cur[4 * g] - corr, cur[4 * g + 1] - corr,
                             cur[4 * g + 2] - corr, cur[4 * g + 3] - corr);
        } else if (OUT == OUT_F32) {
            float4 xrow[PEERS == 3 ? 8 : 1];
            if (PEERS == 3) {
                // the piece loaded ahead, through the (free) staging buffer: rows x 16-byte chunks in, this lane's row out
                const uint32_t sbase = stg + (ONE_STG ? 0u : (n_store & 1u) * 4096u);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t r = (uint32_t)(4 * i + (lane >> 3));
                    const float4 v = xr[PEERS == 3 ? c % kPre : 0][i];
                    st_shared_v4(sbase + r * 128u + ((((uint32_t)lane & 7u) ^ (r & 7u)) << 4), __float_as_uint(v.x),
                                 __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
                }
                __syncwarp();
#pragma unroll
                for (int g = 0; g < 8; g++) {
                    const uint4 v = ld_shared_v4(buf + ((((uint32_t)g) ^ sw) << 4));
                    xrow[g] = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
                }
                __syncwarp();   // every lane has its row before anybody overwrites the buffer with results
            }
#pragma unroll
            for (int g = 0; g < 8; g++) {
                const float4 ws = wsc[g];
                float v0 = __fmul_rn(__fmul_rn(__int2float_rn((int)cur[4 * g] - corr), as), ws.x);
                float v1 = __fmul_rn(__fmul_rn(__int2float_rn((int)cur[4 * g + 1] - corr), as), ws.y);
                float v2 = __fmul_rn(__fmul_rn(__int2float_rn((int)cur[4 * g + 2] - corr), as), ws.z);
                float v3 = __fmul_rn(__fmul_rn(__int2float_rn((int)cur[4 * g + 3] - corr), as), ws.w);
                if (PEERS == 3) {
                    // this lane's row of the residual stream (loaded ahead, see above); the tile is written
                    // back by this warp's own TMA store below, nobody else touches it
                    const float4 gt = gtc[PEERS == 3 ? g : 0];
                    const float4 xv = xrow[PEERS == 3 ? g : 0];
                    v0 = __fmaf_rn(gt.x, v0, xv.x);
                    v1 = __fmaf_rn(gt.y, v1, xv.y);
                    v2 = __fmaf_rn(gt.z, v2, xv.z);
                    v3 = __fmaf_rn(gt.w, v3, xv.w);
                }
                st_shared_v4(buf + ((((uint32_t)g) ^ sw) << 4), __float_as_uint(v0), __float_as_uint(v1),
                             __float_as_uint(v2), __float_as_uint(v3));
            }
            if (PEERS == 3 && c + kPre < BN / 32) load_residual(c + kPre, xr[PEERS == 3 ? c % kPre : 0]);
        } else {
            // bf16: 64 columns make one 128-byte row; this chunk fills pieces 4*(c&1) .. +3
#pragma unroll
            for (int g = 0; g < 4; g++) {
                const float4 w0 = wsc[2 * g], w1 = wsc[2 * g + 1];
                const float wsv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float lo = __fmul_rn(__fmul_rn(__int2float_rn((int)cur[8 * g + 2 * e] - corr), as), wsv[2 * e]);
                    const float hi = __fmul_rn(__fmul_rn(__int2float_rn((int)cur[8 * g + 2 * e + 1] - corr), as), wsv[2 * e + 1]);
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                    pk[e] = *reinterpret_cast<const uint32_t *>(&b2);
                }
                const uint32_t piece = (uint32_t)(4 * (c & 1) + g);
                st_shared_v4(buf + ((piece ^ sw) << 4), pk[0], pk[1], pk[2], pk[3]);
            }
        }
        // one accumulator buffer: the next piece is requested now that this one's values are used up
        if (kOneTmemBuf && c + 1 < BN / 32) tc_ld_32x32(t_row + (uint32_t)((c + 1) * 32), ra);
        const bool last_piece = OUT != OUT_BF16 || (c & 1) == 1;
        if (last_piece) {
            // generic-proxy writes -> visible to the async proxy, then one lane stores
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (PEERS != 2 && lane == 0 && !(p.ablate & 16)) {
                tma_store_2d(tma_y, stg + (ONE_STG ? 0u : (n_store & 1u) * 4096u), scol, row0);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (PEERS == 1 || PEERS == 2) {
                // The staged piece (32 rows x 128 bytes) goes to the peers with plain
                // 16-byte stores: eight lanes cover one 128-byte row, so every store
                // instruction writes four whole rows' segments.
                constexpr int kElemsPerChunk = OUT == OUT_BF16 ? 8 : 4;
                constexpr int kElemBytes = OUT == OUT_BF16 ? 2 : 4;
                const uint32_t sbase = stg + (ONE_STG ? 0u : (n_store & 1u) * 4096u);
                const int chunk = lane & 7;
                const int gcol = scol + chunk * kElemsPerChunk;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = 4 * i + (lane >> 3);
                    const uint4 v = ld_shared_v4(sbase + (uint32_t)r * 128u + ((uint32_t)(chunk ^ (r & 7)) << 4));
                    const int grow = row0 + r;
                    if (grow < p.m && gcol < p.n) {
                        const size_t off = ((size_t)grow * (size_t)p.ldy + (size_t)gcol) * kElemBytes;
                        if (PEERS == 2) {
                            multimem_st_v4(static_cast<char *>(p.mc_y) + off, v);
                        } else {
#pragma unroll
                            for (int pr = 0; pr < kMaxPeers; pr++)
                                if (pr < p.n_peers) st_global_v4(static_cast<char *>(p.peer_y[pr]) + off, v);
                        }
                    }
                }
            }
            n_store++;
        }
    }
}

// sigmoid with the fast exponential and reciprocal: the same two instructions, in the same order,
// as the stand-alone SiLU / sigmoid ops (prep_common.cuh), so that fusing changes no bit.
__device__ __forceinline__ float sigmoid_fast_ep(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}

// Epilogue of the paired-weight tile: accumulator columns 0..127 hold the gate projection of
// output columns n0 .. n0+127, columns 128..255 the up projection of the same ones.  Both are
// dequantised as in epilogue_tile, out = (g * sigmoid(g)) * u in f32 (the arithmetic of the
// stand-alone siluMul on f32 operands, src/models/dit_cuda.zig:513), then f32 or bf16, staged
// and stored like any other tile.
template <int OUT>
__device__ __forceinline__ void epilogue_pair(uint32_t t_row, const GemmParams &p, const CUtensorMap *tma_y,
                                              uint32_t stg, uint32_t my_row_off, uint32_t sw, uint32_t &n_store,
                                              int row0, int n0, float as, int lane) {
    static_assert(OUT == OUT_F32 || OUT == OUT_BF16, "paired epilogue writes f32 or bf16");
    uint32_t rg[32], ru[32];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const int col0 = n0 + c * 32;
        const int scol = (OUT == OUT_BF16 && (c & 1)) ? col0 - 32 : col0;
        const bool do_store = row0 < p.m && scol < p.n;   // warp-uniform
        if (!do_store) continue;
        tc_ld_32x32(t_row + (uint32_t)(c * 32), rg);
        tc_ld_32x32(t_row + (uint32_t)(128 + c * 32), ru);
        // the piece's scales while the accumulators are on their way (loaded inside the loop below, each
        // load stalled its first multiply for an L1 round trip)
        float4 wgv[8], wuv[8];
#pragma unroll
        for (int g = 0; g < 8; g++) {
            wgv[g] = wuv[g] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col0 + 4 * g < p.n) {
                wgv[g] = __ldg(reinterpret_cast<const float4 *>(p.w_scale + col0 + 4 * g));
                wuv[g] = __ldg(reinterpret_cast<const float4 *>(p.w_scale2 + col0 + 4 * g));
            }
        }
        tc_wait_ld_dep(rg);
        tc_wait_ld_dep(ru);
        const bool first_piece = OUT != OUT_BF16 || (c & 1) == 0;
        const uint32_t buf = stg + (n_store & 1u) * 4096u + my_row_off;
        if (first_piece) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
        }
        float o[32];
#pragma unroll
        for (int g = 0; g < 8; g++) {
            const float4 wg = wgv[g], wu = wuv[g];
            const float wgs[4] = {wg.x, wg.y, wg.z, wg.w}, wus[4] = {wu.x, wu.y, wu.z, wu.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float vg = __fmul_rn(__fmul_rn(__int2float_rn((int)rg[4 * g + e]), as), wgs[e]);
                const float vu = __fmul_rn(__fmul_rn(__int2float_rn((int)ru[4 * g + e]), as), wus[e]);
                o[4 * g + e] = __fmul_rn(__fmul_rn(vg, sigmoid_fast_ep(vg)), vu);
            }
        }
        if (OUT == OUT_F32) {
#pragma unroll
            for (int g = 0; g < 8; g++)
                st_shared_v4(buf + ((((uint32_t)g) ^ sw) << 4), __float_as_uint(o[4 * g]), __float_as_uint(o[4 * g + 1]),
                             __float_as_uint(o[4 * g + 2]), __float_as_uint(o[4 * g + 3]));
        } else {
#pragma unroll
            for (int g = 0; g < 4; g++) {
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(o[8 * g + 2 * e], o[8 * g + 2 * e + 1]);
                    pk[e] = *reinterpret_cast<const uint32_t *>(&b2);
                }
                const uint32_t piece = (uint32_t)(4 * (c & 1) + g);
                st_shared_v4(buf + ((piece ^ sw) << 4), pk[0], pk[1], pk[2], pk[3]);
            }
        }
        const bool last_piece = OUT != OUT_BF16 || (c & 1) == 1;
        if (last_piece) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(tma_y, stg + (n_store & 1u) * 4096u, scol, row0);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            n_store++;
        }
    }
}

// ---- host side: tensor maps ------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Looks the map up in the handle's cache, or encodes it and remembers it.  `key` names everything
// the encoding depends on.
template <typename Encode>
inline int tpb_tensor_map_cached(tpb_handle_t h, CUtensorMap *map, const uint64_t (&key)[5], Encode encode) {
    static_assert(sizeof(CUtensorMap) <= sizeof(tpb_map_slot::map), "tensor map larger than a cache slot");
    uint64_t hsh = 0x9E3779B97F4A7C15ull;
    for (int i = 0; i < 5; i++) hsh = (hsh ^ key[i]) * 0xFF51AFD7ED558CCDull, hsh ^= hsh >> 29;
    tpb_map_slot &slot = h->map_cache[hsh % TPB_MAP_CACHE_SLOTS];
    if (slot.valid && slot.key[0] == key[0] && slot.key[1] == key[1] && slot.key[2] == key[2] &&
        slot.key[3] == key[3] && slot.key[4] == key[4]) {
        memcpy(map, slot.map, sizeof(CUtensorMap));
        return TPB_OK;
    }
    const int rc = encode(map);
    if (rc != TPB_OK) return rc;
    for (int i = 0; i < 5; i++) slot.key[i] = key[i];
    memcpy(slot.map, map, sizeof(CUtensorMap));
    slot.valid = true;
    return TPB_OK;
}

// 2-D uint8 tensor [rows][k] (k contiguous), box = 128 bytes x box_rows, 128B swizzle,
// out-of-range rows read as zero.
inline int make_kmajor_map(tpb_handle_t h, CUtensorMap *map, const void *base, int64_t rows, int64_t k,
                    int box_rows) {
    const uint64_t key[5] = {(uint64_t)reinterpret_cast<uintptr_t>(base), (uint64_t)rows, (uint64_t)k,
                             (uint64_t)box_rows, 0x100u};
    return tpb_tensor_map_cached(h, map, key, [&](CUtensorMap *out) {
        const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)k};
        const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
        const cuuint32_t estride[2] = {1, 1};
        const CUresult r = reinterpret_cast<EncodeTiledFn>(h->encode_tiled)(
            out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estride,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return tpb_fail(h, TPB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) rows=%lld k=%lld", (int)r,
                            (long long)rows, (long long)k);
        return (int)TPB_OK;
    });
}

// Output tensor [m][ldy] (row-major), box = 128 bytes x 32 rows, 128B swizzle: the
// epilogue's staging layout.
template <int OUT>
inline int make_out_map(tpb_handle_t h, CUtensorMap *map, const GemmParams &p) {
    const uint64_t key[5] = {(uint64_t)reinterpret_cast<uintptr_t>(p.y), (uint64_t)p.m, (uint64_t)p.n,
                             (uint64_t)p.ldy, 0x200u + (uint64_t)OUT};
    return tpb_tensor_map_cached(h, map, key, [&](CUtensorMap *out) {
        const int esz = OUT == OUT_BF16 ? 2 : 4;
        const CUtensorMapDataType dt = OUT == OUT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                       : OUT == OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                        : CU_TENSOR_MAP_DATA_TYPE_INT32;
        const cuuint64_t gdim[2] = {(cuuint64_t)p.n, (cuuint64_t)p.m};
        const cuuint64_t gstride[1] = {(cuuint64_t)p.ldy * esz};
        const cuuint32_t box[2] = {(cuuint32_t)(128 / esz), 32u};
        const cuuint32_t estride[2] = {1, 1};
        const CUresult r = reinterpret_cast<EncodeTiledFn>(h->encode_tiled)(
            out, dt, 2, p.y, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return tpb_fail(h, TPB_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed (%d) m=%d n=%d ldy=%lld", (int)r,
                            p.m, p.n, p.ldy);
        return (int)TPB_OK;
    });
}

}  // namespace tpb_gemm
