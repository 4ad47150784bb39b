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
//
// Data path.  One CTA per SM owns a contiguous range of weight rows.  A producer warp streams
// them in stages of 16 rows x one K segment with one 1-D bulk copy per row (cp.async.bulk,
// completion on the stage's "full" mbarrier, no multicast) into a ring that fills most of
// shared memory; it starts before griddepcontrol.wait, so under programmatic dependent launch
// the ring fills while the previous kernel drains.  The warps whose K slice lies in a stage's
// segment wait for it, multiply, write their 16 x 8 partial sums to a small buffer and arrive
// on the stage's "empty" mbarrier.  When the last segment of a row group has been released,
// the producer warp -- which has to wait for that anyway before it may refill the slot -- adds
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
constexpr int kConsumers = 16;                 // consumer warps; warp 16 is the producer
constexpr int kThreadsMma = (kConsumers + 1) * 32;
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
    int nseg;          // K segments per row group (divides kConsumers)
    int pitch;         // bytes between rows of a stage
    int stages;        // ring depth
    int rgbuf;         // row groups of partial sums kept
    uint32_t *status;
};

// K segment s of a row: blocks [seg_blk0(s), seg_blk0(s + 1)), always whole units of 8 blocks
// (272 bytes, a multiple of 16).
__host__ __device__ inline int seg_blk0(int nblk, int nseg, int s) { return (int)((long long)(nblk / 8) * s / nseg) * 8; }
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

// 17 warps x 32 lanes x 120 registers = 65280 of the SM's 65536: the register budget is stated
// directly (a launch bound of 544 threads makes the compiler settle for 96).
template <int NP>
__global__ void __maxnreg__(120) q8_0_gemv_mma_kernel(const MmaGemvParams p) {
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
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(wps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this CTA's rows and its stages: (row group, segment), row groups of 16 rows
    const int r_begin = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r_end = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int n_rg = (r_end - r_begin + kStageRows - 1) / kStageRows;
    const int total = n_rg * p.nseg;

    if (warp == kConsumers) {
        // ---------------- producer + reducer ----------------
        auto issue = [&](int i) {  // lane 0: copies of stage i
            const int rg = i / p.nseg, seg = i - rg * p.nseg;
            const int row0 = r_begin + rg * kStageRows;
            const int nrow = min(kStageRows, r_end - row0);
            const int b0 = seg_blk0(nblk, p.nseg, seg), b1 = seg_blk0(nblk, p.nseg, seg + 1);
            const uint32_t bytes = (uint32_t)(b1 - b0) * kBlockBytes;
            const int slot = i % S;
            const uint32_t bar = full_bar(slot);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (uint32_t)nrow)
                         : "memory");
            const uint32_t dst = smem_u32(ring + (size_t)slot * stage_bytes);
            const uint8_t *src = p.w + (size_t)row0 * row_bytes + (size_t)b0 * kBlockBytes;
            for (int r = 0; r < nrow; r++) bulk_g2s(dst + (uint32_t)(r * p.pitch), src + (size_t)r * row_bytes, bytes, bar);
        };
        auto reduce = [&](int rg) {  // all lanes: y for row group rg from the consumers' partial sums
            // a warp's partials: [16 weight rows][8 activation rows]; this lane: row lane / 2, activation rows 4 (lane % 2) ..
            const float *part = s_part + (size_t)(rg % p.rgbuf) * kConsumers * kPartFloats + 4 * lane;
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
                if (m0 + 0 < p.m) p.y[(size_t)(m0 + 0) * p.rows + row] = sum.x * p.scale;
                if (m0 + 1 < p.m) p.y[(size_t)(m0 + 1) * p.rows + row] = sum.y * p.scale;
                if (m0 + 2 < p.m) p.y[(size_t)(m0 + 2) * p.rows + row] = sum.z * p.scale;
                if (m0 + 3 < p.m) p.y[(size_t)(m0 + 3) * p.rows + row] = sum.w * p.scale;
            }
        };
        // weights are constants: the ring starts filling before the previous kernel has finished
        if (lane == 0)
            for (int i = 0; i < S && i < total; i++) issue(i);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        bool ok = true;
        for (int j = 0; j < total && ok; j++) {
            // stage j has been consumed by its warps
            ok = mbar_wait(empty_bar(j % S), (uint32_t)(j / S) & 1u, p.status, (7u << 24) | (uint32_t)(j % S));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (j % p.nseg == p.nseg - 1) reduce(j / p.nseg);
            __syncwarp();
            if (j + S < total && lane == 0) {
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
    const int sb0 = seg_blk0(nblk, p.nseg, seg), sb1 = seg_blk0(nblk, p.nseg, seg + 1);
    const int seg_pairs = (sb1 - sb0) / 2;
    const int pp0 = warp_pair0(seg_pairs, wps, wi), pp1 = warp_pair0(seg_pairs, wps, wi + 1);
    const int np = pp1 - pp0;  // <= NP (checked by the host)

    asm volatile("griddepcontrol.wait;" ::: "memory");
    // activation scales of all 8 (padded) rows -> shared memory; consumers only
    for (int i = threadIdx.x; i < kActRows * nblk; i += kConsumers * 32) {
        const int m = i / nblk;
        s_dx[i] = m < p.m ? __ldcg(p.xd + (size_t)m * nblk + (i - m * nblk)) : 0.0f;
    }
    // this lane's part of the B operand: activation row g, K positions of its pairs
    uint32_t b[NP][4];
#pragma unroll
    for (int q = 0; q < NP; q++) {
        b[q][0] = b[q][1] = b[q][2] = b[q][3] = 0u;
        if (q < np && g < p.m) {
            const int blk = sb0 + 2 * (pp0 + q);
            const uint32_t *x0 = reinterpret_cast<const uint32_t *>(p.xq + (size_t)g * p.cols + (size_t)blk * 32);
            // first block of the pair, in the order "aligned words 1..7, then the two end halves"
            const uint32_t lo_a = __ldcg(x0 + (t == 0 ? 0 : t - 1)), lo_b = __ldcg(x0 + (t == 0 ? 7 : t));
            b[q][0] = t == 0 ? ((lo_a & 0x0000ffffu) | (lo_b & 0xffff0000u)) : __funnelshift_r(lo_a, lo_b, 16);
            b[q][1] = __funnelshift_r(__ldcg(x0 + 3 + t), __ldcg(x0 + 4 + t), 16);
            // second block: word-aligned in the weight row, natural order
            b[q][2] = __ldcg(x0 + 8 + t);
            b[q][3] = __ldcg(x0 + 12 + t);
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");

    // shared addresses relative to a stage: this warp's first pair in weight row g, word t
    const uint32_t ring_u32 = smem_u32(ring) + (uint32_t)(pp0 * kPairBytes) + (uint32_t)(g * p.pitch) + 4u * (uint32_t)t;
    const uint32_t hi_rows = 8u * (uint32_t)p.pitch;   // weight row g + 8
    // activation scales of activation rows 2t and 2t+1, this warp's first block
    const uint32_t dx_u32 = smem_u32(s_dx + (size_t)(2 * t) * nblk + sb0 + 2 * pp0);
    const uint32_t dx_next = 4u * (uint32_t)nblk;

    bool ok = true;
    for (int rg = 0; rg < n_rg && ok; rg++) {
        const int i = rg * p.nseg + seg;
        const int slot = i % S;
        ok = mbar_wait(full_bar(slot), (uint32_t)(i / S) & 1u, p.status, (8u << 24) | (uint32_t)slot);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t wl = ring_u32 + (uint32_t)(slot * stage_bytes), wh = wl + hi_rows;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int q = 0; q < NP; q++) {
            if (q < np) {
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
        float *part = s_part + ((size_t)(rg % p.rgbuf) * kConsumers + warp) * kPartFloats;
        *reinterpret_cast<float2 *>(part + g * kActRows + 2 * t) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2 *>(part + (g + 8) * kActRows + 2 * t) = make_float2(acc[2], acc[3]);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(empty_bar(slot)) : "memory");
    }
}

struct MmaPlan {
    int nseg = 0, pitch = 0, stages = 0, rgbuf = 0, max_pairs = 0;
    size_t smem = 0;
};

// Ring geometry for `nblk` blocks per row, or nseg = 0 when the shape does not fit this kernel.
MmaPlan plan_mma(tpb_handle_t h, int nblk) {
    MmaPlan best;
    const size_t limit = (size_t)h->smem_optin - 1024;
    for (int nseg = 1; nseg <= kConsumers; nseg *= 2) {
        if (nblk / 8 < nseg) break;
        int seg_blocks = 0, max_pairs = 0;
        const int wps = kConsumers / nseg;
        for (int s = 0; s < nseg; s++) {
            const int b = seg_blk0(nblk, nseg, s + 1) - seg_blk0(nblk, nseg, s);
            seg_blocks = b > seg_blocks ? b : seg_blocks;
            for (int wi = 0; wi < wps; wi++) {
                const int n = warp_pair0(b / 2, wps, wi + 1) - warp_pair0(b / 2, wps, wi);
                max_pairs = n > max_pairs ? n : max_pairs;
            }
        }
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
            // prefer the fewest segments that still give >= 4 stages, else the deepest ring
            if (best.nseg == 0 || (best.stages < 4 && stages > best.stages)) {
                best.nseg = nseg;
                best.pitch = pitch;
                best.stages = stages;
                best.rgbuf = rgbuf;
                best.max_pairs = max_pairs;
                best.smem = smem;
            }
            break;
        }
        if (best.nseg != 0 && best.stages >= 4) break;
    }
    return best;
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
    return pl.nseg != 0 && pl.max_pairs <= 18;
}

int tpb_launch_q8_0_gemv_mma(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale, int64_t rows,
                             int64_t cols, const void *xq, int ng, int row_off, int n_total) {
    const int nblk = (int)(cols / 32);
    const MmaPlan pl = plan_mma(h, nblk);
    if (pl.nseg == 0 || pl.max_pairs > 18)
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
    p.nseg = pl.nseg;
    p.pitch = pl.pitch;
    p.stages = pl.stages;
    p.rgbuf = pl.rgbuf;
    p.status = h->d_status;
    if (pl.max_pairs <= 6) return launch_np<6>(h, st, p, pl.smem);
    if (pl.max_pairs <= 12) return launch_np<12>(h, st, p, pl.smem);
    return launch_np<18>(h, st, p, pl.smem);
}
