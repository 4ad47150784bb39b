// GGUF Q8_0 decode GEMV for 1..8 activation rows with the activations held in registers
// for the whole kernel and the weight streamed past them once (sm_100a).
//
// Why a second Q8_0 kernel.  In the dp4a kernel (qgemv.cu) a lane owns a K position and
// re-reads that position's quantised activations from shared memory for every group of
// weight rows: 64 bytes per lane, activation row and row group.  With several activation
// rows those shared-memory reads, and the instructions around them, set the pace (measured:
// 128-bit shared loads with distinct addresses take 8 cycles per warp instruction on this
// part, dp4a issues at half rate and shares its pipe with the f32 work).  Here the roles are
// swapped.  Every consumer warp owns a fixed slice of K; a lane keeps its part of the
// activations of that slice in registers from start to end, laid out as the B operand of
// mma.sync.m16n8k32 (8 activation rows on the n side: two registers per Q8_0 block), and
// each Q8_0 block of 16 weight rows is one A operand: four shared-memory words per lane and
// one MMA give the 16 x 8 exact int32 block sums that the dp4a kernel needs 8 dp4a per row
// and activation row for.  The per-block scaling stays the reference's
// (src/gpu/cuda/elt.zig:1984-2005):
//   acc += float(sumi) * (d_w * d_x)   in f32, block after block.
// Rows too long for the registers (more than 12 block pairs per warp) are taken in several
// passes over K: a pass streams one K range of all the CTA's rows, and the passes after the
// first add to the y the first one wrote.
//
// Data path.  One CTA per SM owns a contiguous range of weight rows.  Four producer warps stream
// them in stages of 16 rows x one K segment with one 1-D bulk copy per row (cp.async.bulk,
// completion on the stage's "full" mbarrier, no multicast) into a ring that fills most of
// shared memory; they start before griddepcontrol.wait, so under programmatic dependent launch
// the ring fills while the previous kernel drains.  (Four warps, four rows each, because a warp
// gets a bulk copy under way only every ~225 cycles: measured, one warp issuing all sixteen
// copies of every stage capped the kernel at 3.4 TB/s.  The register file hands out registers
// to warps in fours, so warps 17..19 cost nothing.)  The warps whose K slice lies in a stage's
// segment wait for it, multiply, write their 16 x 8 partial sums to a small buffer and arrive
// on the stage's "empty" mbarrier.  When the last segment of a row group has been released,
// the first producer warp -- which has to wait for that anyway before it may refill the slot -- adds
// the partials in warp order (a fixed order: results do not depend on timing), applies
// `scale`, and stores y.  No warp ever waits for another consumer warp.
//
// Rows in shared memory sit at a pitch of 4 words modulo 32 banks, so the 8 rows x 4 words an
// A fragment load touches fall in 32 different banks.
//
// Quant bytes of the first block of a pair start 2 bytes into a word (34-byte blocks).  The
// MMA sums over k, so any order of the 32 positions will do as long as A and B agree: the
// first block of every pair uses the order "bytes of the aligned words 1..7, then the two
// half words at the ends", which costs one funnel shift in one lane out of four, and the
// activations are loaded into that order once, at the start.
#include <cuda_fp16.h>

#include "qgemv_common.cuh"

using namespace tpb_gemv;

namespace {

constexpr int kBlockBytes = 34;
constexpr int kPairBytes = 68;
constexpr int kConsumers = 16;                 // consumer warps 0..15
constexpr int kProducers = 4;                  // producer warps 16..19, four rows of every stage each
constexpr int kThreadsMma = (kConsumers + kProducers) * 32;
constexpr int kStageRows = 16;                 // weight rows per stage = m of the MMA
constexpr int kActRows = 8;                    // activation rows = n of the MMA
constexpr int kPartFloats = kStageRows * kActRows;   // partial sums of one warp for one stage

struct MmaGemvParams {
    float *y;
    const uint8_t *w;
    const float *xd;   // activation block scales [m][nblk]
    const int8_t *xq;  // activation quants [m][cols]
    float scale;
    int rows, cols, nblk, m;
    int npass;         // passes over K (each covers a contiguous range of whole 8-block units)
    int nseg;          // K segments per pass and row group (divides kConsumers)
    int pitch;         // bytes between rows of a stage
    int stages;        // ring depth
    int rgbuf;         // row groups of partial sums kept
    int debug;         // TPB_GEMV_MMA_DEBUG (diagnosis): bit 0 = consumers skip the arithmetic
    uint32_t *status;
};

// Pass p of a row covers blocks [pass_blk0(p), pass_blk0(p + 1)); K segment s of a pass covers
// [seg_blk0(s), seg_blk0(s + 1)) of those.  Both are whole units of 8 blocks (272 bytes, a multiple of 16).
__host__ __device__ inline int pass_blk0(int nblk, int npass, int p) { return (int)((long long)(nblk / 8) * p / npass) * 8; }
__host__ __device__ inline int seg_blk0(int pb0, int pb1, int nseg, int s) {
    return pb0 + (int)((long long)((pb1 - pb0) / 8) * s / nseg) * 8;
}
// pairs [lo, hi) of consumer `wi` (0 .. wps-1) inside a segment of `pairs` block pairs
__host__ __device__ inline int warp_pair0(int pairs, int wps, int wi) { return (int)((long long)pairs * wi / wps); }

// C[16 weight rows][8 activation rows] = A[16][32] * B[32][8], int8 -> int32, C starts at zero.
// Lane (g = lane / 4, t = lane % 4): a0/a2 = weight row g, k = 4t.. and 16+4t..; a1/a3 = weight row
// g + 8; b0/b1 = activation row g, same k; c0,c1 = row g x activation rows 2t, 2t+1; c2,c3 = row g + 8.
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Shared-memory loads by 32-bit shared address: one address register instead of a generic pointer pair.
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float f16lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))); }
__device__ __forceinline__ float f16hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }

// 20 warps: 65536 / 640 = 102 registers per thread, 96 after rounding to the allocation unit.
template <int NP>
__global__ void __launch_bounds__(kThreadsMma, 1) q8_0_gemv_mma_kernel(const MmaGemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nblk = p.nblk;
    const int S = p.stages;
    const int stage_bytes = kStageRows * p.pitch;
    const size_t row_bytes = (size_t)nblk * kBlockBytes;

    uint8_t *ring = smem;
    float *s_dx = reinterpret_cast<float *>(smem + (size_t)S * stage_bytes);       // [8][nblk]
    float *s_part = s_dx + (size_t)kActRows * nblk;                                 // [rgbuf][kConsumers][128]
    const uint32_t bars = smem_u32(s_part + (size_t)p.rgbuf * kConsumers * kPartFloats);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };

    const int wps = kConsumers / p.nseg;  // consumer warps per K segment
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(kProducers));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(wps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this CTA's rows and its stages: (pass, row group, segment), row groups of 16 rows
    const int r_begin = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int n_rg = (r_end - r_begin + kStageRows - 1) / kStageRows;
    const int total = p.npass * n_rg * p.nseg;

    if (warp >= kConsumers) {
        // ---------------- producers (the first one also reduces) ----------------
        const int pw = warp - kConsumers;
        constexpr int kRowsPerProducer = kStageRows / kProducers;
        auto issue = [&](int i) {  // whole warp: lane r starts the copy of this warp's r-th row of stage i
            const int v = i / p.nseg, seg = i - v * p.nseg;      // v = row-group visit: pass * n_rg + rg
            const int pass = v / n_rg, rg = v - pass * n_rg;
            const int row0 = r_begin + rg * kStageRows;
            const int nrow = min(kStageRows, r_end - row0);
            const int pb0 = pass_blk0(nblk, p.npass, pass), pb1 = pass_blk0(nblk, p.npass, pass + 1);
            const int b0 = seg_blk0(pb0, pb1, p.nseg, seg), b1 = seg_blk0(pb0, pb1, p.nseg, seg + 1);
            const uint32_t bytes = (uint32_t)(b1 - b0) * kBlockBytes;
            const int slot = i % S;
            const uint32_t bar = full_bar(slot);
            const int my_rows = max(0, min(kRowsPerProducer, nrow - pw * kRowsPerProducer));
            if (lane == 0)   // every producer warp arrives, also with nothing to copy (the barrier counts four)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (uint32_t)my_rows)
                             : "memory");
            __syncwarp();
            const int r = pw * kRowsPerProducer + lane;
            const uint32_t dst = smem_u32(ring + (size_t)slot * stage_bytes);
            const uint8_t *src = p.w + (size_t)row0 * row_bytes + (size_t)b0 * kBlockBytes;
            if (lane < my_rows) bulk_g2s(dst + (uint32_t)(r * p.pitch), src + (size_t)r * row_bytes, bytes, bar);
        };
        auto reduce = [&](int v) {  // all lanes: y of one row-group visit from the consumers' partial sums
            // a warp's partials: [16 weight rows][8 activation rows]; this lane: row lane / 2, activation rows 4 (lane % 2) ..
            const int pass = v / n_rg, rg = v - pass * n_rg;
            const float *part = s_part + (size_t)(v % p.rgbuf) * kConsumers * kPartFloats + 4 * lane;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kConsumers; w++) {
                const float4 v = *reinterpret_cast<const float4 *>(part + w * kPartFloats);
                sum.x += v.x;
                sum.y += v.y;
                sum.z += v.z;
                sum.w += v.w;
            }
            const int row = r_begin + rg * kStageRows + (lane >> 1);
            const int m0 = 4 * (lane & 1);
            if (row < r_end) {
                // later passes add to what this same lane stored in the pass before
                const float v4[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (m0 + e < p.m) {
                        float *dst = p.y + (size_t)(m0 + e) * p.rows + row;
                        *dst = pass == 0 ? v4[e] * p.scale : fmaf(v4[e], p.scale, *dst);
                    }
            }
        };
        // weights are constants: the ring starts filling before the previous kernel has finished
        for (int i = 0; i < S && i < total; i++) issue(i);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        bool ok = true;
        for (int j = 0; j < total && ok; j++) {
            // stage j has been consumed by its warps
            ok = mbar_wait(empty_bar(j % S), (uint32_t)(j / S) & 1u, p.status, (7u << 24) | (uint32_t)(j % S));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // Partial sums are added before this warp's part of the refill goes out, and the refilled
            // stage is not "full" without it: no consumer can overwrite a partial that is still needed.
            if (pw == 0 && j % p.nseg == p.nseg - 1) reduce(j / p.nseg);
            __syncwarp();
            if (j + S < total) {
                // order the consumers' generic-proxy reads of the slot before the async-proxy refill
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue(j + S);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    const int seg = warp / wps, wi = warp - seg * wps;

    asm volatile("griddepcontrol.wait;" ::: "memory");
    // activation scales of all 8 (padded) rows -> shared memory; consumers only
    // (the loads of four rounds go out together: a round trip to L2 each would cost a microsecond)
    for (int i0 = threadIdx.x; i0 < kActRows * nblk; i0 += 4 * kConsumers * 32) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * kConsumers * 32;
            const int m = i / nblk;
            v[u] = (i < kActRows * nblk && m < p.m) ? __ldcg(p.xd + (size_t)m * nblk + (i - m * nblk)) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * kConsumers * 32;
            if (i < kActRows * nblk) s_dx[i] = v[u];
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");

    const uint32_t hi_rows = 8u * (uint32_t)p.pitch;   // weight row g + 8
    const uint32_t dx_next = 4u * (uint32_t)nblk;      // next activation row's scales
    bool ok = true;
  for (int pass = 0; pass < p.npass && ok; pass++) {
    const int pb0 = pass_blk0(nblk, p.npass, pass), pb1 = pass_blk0(nblk, p.npass, pass + 1);
    const int sb0 = seg_blk0(pb0, pb1, p.nseg, seg), sb1 = seg_blk0(pb0, pb1, p.nseg, seg + 1);
    const int seg_pairs = (sb1 - sb0) / 2;
    const int pp0 = warp_pair0(seg_pairs, wps, wi), pp1 = warp_pair0(seg_pairs, wps, wi + 1);
    const int np = pp1 - pp0;  // <= NP (checked by the host)
    // this lane's part of the B operand: activation row g, K positions of its pairs in this pass
    // Lane (g, t) loads words t and 4+t of both blocks of each pair (all loads independent, so they
    // go out together), then the first block is put into the order "aligned words 1..7 of the
    // weight block, then its two end halves": slot j holds activation bytes 4j-2 .. 4j+1, i.e. the
    // high half of word j-1 and the low half of word j; slot 0 holds bytes 0, 1, 30, 31.  The
    // neighbouring words come from the neighbouring lanes of the same activation row.
    uint32_t b[NP][4];
#pragma unroll
    for (int q = 0; q < NP; q++) {
        b[q][0] = b[q][1] = b[q][2] = b[q][3] = 0u;
        if (q < np && g < p.m) {
            const int blk = sb0 + 2 * (pp0 + q);
            const uint32_t *x0 = reinterpret_cast<const uint32_t *>(p.xq + (size_t)g * p.cols + (size_t)blk * 32);
            b[q][0] = __ldcg(x0 + t);
            b[q][1] = __ldcg(x0 + 4 + t);
            b[q][2] = __ldcg(x0 + 8 + t);    // second block: word-aligned in the weight row, natural order
            b[q][3] = __ldcg(x0 + 12 + t);
        }
    }
#pragma unroll
    for (int q = 0; q < NP; q++) {
        // all 32 lanes take part in the shuffles (q < np is warp-uniform)
        if (q < np) {
            const uint32_t w_lo = b[q][0], w_hi = b[q][1];
            const int prev = (lane & ~3) | ((t + 3) & 3);                 // lane (g, t-1), wrapping to t = 3
            const uint32_t p_lo = __shfl_sync(0xffffffffu, w_lo, prev);   // word t-1      (t = 0: word 3)
            const uint32_t p_hi = __shfl_sync(0xffffffffu, w_hi, prev);   // word 3+t      (t = 0: word 7)
            // slot t: t >= 1 -> words (t-1, t); t = 0 -> low half of word 0, high half of word 7
            b[q][0] = t == 0 ? ((w_lo & 0x0000ffffu) | (p_hi & 0xffff0000u)) : __funnelshift_r(p_lo, w_lo, 16);
            // slot 4+t: words (3+t, 4+t); word 3+t is lane t-1's second word, for t = 0 lane 3's first
            b[q][1] = __funnelshift_r(t == 0 ? p_lo : p_hi, w_hi, 16);
        }
    }
    // shared addresses relative to a stage: this warp's first pair in weight row g, word t
    const uint32_t ring_u32 = smem_u32(ring) + (uint32_t)(pp0 * kPairBytes) + (uint32_t)(g * p.pitch) + 4u * (uint32_t)t;
    // activation scales of activation rows 2t and 2t+1, this warp's first block
    const uint32_t dx_u32 = smem_u32(s_dx + (size_t)(2 * t) * nblk + sb0 + 2 * pp0);

    for (int rg = 0; rg < n_rg && ok; rg++) {
        const int v = pass * n_rg + rg;
        const int i = v * p.nseg + seg;
        const int slot = i % S;
        ok = mbar_wait(full_bar(slot), (uint32_t)(i / S) & 1u, p.status, (8u << 24) | (uint32_t)slot);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t wl = ring_u32 + (uint32_t)(slot * stage_bytes), wh = wl + hi_rows;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int q = 0; q < NP; q++) {
            if (q < np && !(p.debug & 1)) {
                const uint32_t o = (uint32_t)(q * kPairBytes);
                // words t, 4+t, 8 (and 0 for the scale) of the first block, 9+t and 13+t of the second
                const uint32_t l0 = lds32(wl + o - 4u * t), l_lo = lds32(wl + o), l_hi = lds32(wl + o + 16);
                const uint32_t l8 = lds32(wl + o + 32 - 4u * t), l_v0 = lds32(wl + o + 36), l_v1 = lds32(wl + o + 52);
                const uint32_t h0 = lds32(wh + o - 4u * t), h_lo = lds32(wh + o), h_hi = lds32(wh + o + 16);
                const uint32_t h8 = lds32(wh + o + 32 - 4u * t), h_v0 = lds32(wh + o + 36), h_v1 = lds32(wh + o + 52);
                const float2 dxa = lds_f2(dx_u32 + 8u * q), dxb = lds_f2(dx_u32 + dx_next + 8u * q);
                int c0[4], c1[4];
                mma_s8(c0, t == 0 ? __funnelshift_r(l_lo, l8, 16) : l_lo, t == 0 ? __funnelshift_r(h_lo, h8, 16) : h_lo,
                       l_hi, h_hi, b[q][0], b[q][1]);
                mma_s8(c1, l_v0, h_v0, l_v1, h_v1, b[q][2], b[q][3]);
                // weight scales: f16 in the low half of word 0 (first block) and the high half of word 8 (second)
                const float dl0 = f16lo(l0), dl1 = f16hi(l8), dh0 = f16lo(h0), dh1 = f16hi(h8);
                acc[0] = fmaf(i2f_small(c0[0]), dl0 * dxa.x, acc[0]);
                acc[1] = fmaf(i2f_small(c0[1]), dl0 * dxb.x, acc[1]);
                acc[2] = fmaf(i2f_small(c0[2]), dh0 * dxa.x, acc[2]);
                acc[3] = fmaf(i2f_small(c0[3]), dh0 * dxb.x, acc[3]);
                acc[0] = fmaf(i2f_small(c1[0]), dl1 * dxa.y, acc[0]);
                acc[1] = fmaf(i2f_small(c1[1]), dl1 * dxb.y, acc[1]);
                acc[2] = fmaf(i2f_small(c1[2]), dh1 * dxa.y, acc[2]);
                acc[3] = fmaf(i2f_small(c1[3]), dh1 * dxb.y, acc[3]);
            }
        }
        // this warp's K slice of C[weight row][activation row]: rows g and g + 8, activation rows 2t, 2t+1
        float *part = s_part + ((size_t)(v % p.rgbuf) * kConsumers + warp) * kPartFloats;
        *reinterpret_cast<float2 *>(part + g * kActRows + 2 * t) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2 *>(part + (g + 8) * kActRows + 2 * t) = make_float2(acc[2], acc[3]);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(empty_bar(slot)) : "memory");
    }
  }
}

struct MmaPlan {
    int npass = 0, nseg = 0, pitch = 0, stages = 0, rgbuf = 0, max_pairs = 0;
    size_t smem = 0;
};

constexpr int kMaxPairs = 12;   // block pairs a consumer warp can keep in registers (largest instantiation)

// Ring geometry for `nblk` blocks per row: the fewest passes over K whose K slices fit the
// registers, then the fewest segments that still give a ring of at least 4 stages (else the
// deepest ring).  npass = 0 when nothing fits.
MmaPlan plan_mma(tpb_handle_t h, int nblk) {
    const size_t limit = (size_t)h->smem_optin - 1024;
    for (int npass = 1; npass <= 8; npass++) {
        if (nblk / 8 < npass) break;
        MmaPlan best;
        for (int nseg = 1; nseg <= kConsumers; nseg *= 2) {
            int seg_blocks = 0, max_pairs = 0;
            bool ok = true;
            const int wps = kConsumers / nseg;
            for (int ps = 0; ps < npass && ok; ps++) {
                const int pb0 = pass_blk0(nblk, npass, ps), pb1 = pass_blk0(nblk, npass, ps + 1);
                if ((pb1 - pb0) / 8 < nseg) ok = false;
                for (int sg = 0; sg < nseg && ok; sg++) {
                    const int nb = seg_blk0(pb0, pb1, nseg, sg + 1) - seg_blk0(pb0, pb1, nseg, sg);
                    seg_blocks = nb > seg_blocks ? nb : seg_blocks;
                    for (int wi = 0; wi < wps; wi++) {
                        const int n = warp_pair0(nb / 2, wps, wi + 1) - warp_pair0(nb / 2, wps, wi);
                        max_pairs = n > max_pairs ? n : max_pairs;
                    }
                }
            }
            if (!ok) break;
            if (max_pairs > kMaxPairs) continue;
            // rows at 4 words modulo 32 banks, 16-byte aligned
            int pitch_w = seg_blocks * kBlockBytes / 4;
            pitch_w += ((4 - pitch_w % 32) + 32) % 32;
            const int pitch = pitch_w * 4;
            const size_t stage = (size_t)kStageRows * pitch;
            const size_t fixed = (size_t)kActRows * nblk * 4 + 64 + 2 * 8 * 16;
            for (int stages = 8; stages >= 3; stages--) {
                const int rgbuf = (stages - 1 + nseg - 1) / nseg + 1;
                const size_t smem = stages * stage + fixed + (size_t)rgbuf * kConsumers * kPartFloats * 4;
                if (smem > limit) continue;
                if (best.npass == 0 || (best.stages < 4 && stages > best.stages)) {
                    best.npass = npass;
                    best.nseg = nseg;
                    best.pitch = pitch;
                    best.stages = stages;
                    best.rgbuf = rgbuf;
                    best.max_pairs = max_pairs;
                    best.smem = smem;
                }
                break;
            }
            if (best.npass != 0 && best.stages >= 4) break;
        }
        if (best.npass != 0) return best;
    }
    return MmaPlan();
}

template <int NP>
int launch_np(tpb_handle_t h, cudaStream_t st, const MmaGemvParams &p, size_t smem) {
    auto kern = q8_0_gemv_mma_kernel<NP>;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
    long long grid = ((long long)p.rows + kStageRows - 1) / kStageRows;
    if (grid > h->sm_count) grid = h->sm_count;
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3((unsigned)grid), dim3(kThreadsMma), smem, st, p));
    return TPB_OK;
}

}  // namespace

// True when the activation-stationary kernel can take this shape.
bool tpb_q8_0_gemv_mma_fits(tpb_handle_t h, int64_t rows, int64_t cols) {
    if (cols % 256 != 0 || rows < 1) return false;
    const MmaPlan pl = plan_mma(h, (int)(cols / 32));
    return pl.npass != 0;
}

int tpb_launch_q8_0_gemv_mma(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale, int64_t rows,
                             int64_t cols, const void *xq, int ng, int row_off, int n_total) {
    const int nblk = (int)(cols / 32);
    const MmaPlan pl = plan_mma(h, nblk);
    if (pl.npass == 0)
        return tpb_fail(h, TPB_ERR_INVALID_ARG, "q8_0 gemv: %lld columns do not fit the register-resident kernel",
                        (long long)cols);
    MmaGemvParams p;
    p.y = y;
    p.w = reinterpret_cast<const uint8_t *>(w);
    p.xd = reinterpret_cast<const float *>(xq) + (size_t)row_off * nblk;
    p.xq = reinterpret_cast<const int8_t *>(xq) + (size_t)n_total * nblk * 4 + (size_t)row_off * cols;
    p.scale = scale;
    p.rows = (int)rows;
    p.cols = (int)cols;
    p.nblk = nblk;
    p.m = ng;
    p.npass = pl.npass;
    p.nseg = pl.nseg;
    p.pitch = pl.pitch;
    p.stages = pl.stages;
    p.rgbuf = pl.rgbuf;
    p.status = h->d_status;
    {
        const char *e = getenv("TPB_GEMV_MMA_DEBUG");
        p.debug = e ? atoi(e) : 0;
        if (p.debug & 2) {   // experiment: rows of a stage 128-byte aligned (bank conflicts, aligned copies)
            const int pitch128 = (pl.pitch + 127) / 128 * 128;
            if ((size_t)pl.stages * kStageRows * (pitch128 - pl.pitch) + pl.smem <= (size_t)h->smem_optin - 1024) {
                p.pitch = pitch128;
                const_cast<MmaPlan &>(pl).smem += (size_t)pl.stages * kStageRows * (pitch128 - pl.pitch);
            } else {
                p.debug &= ~2;
            }
        }
    }
    if (pl.max_pairs <= 6) return launch_np<6>(h, st, p, pl.smem);
    return launch_np<kMaxPairs>(h, st, p, pl.smem);
}
