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
// each Q8_0 block of 8 weight rows is the upper half of an A operand (the lower half is zero):
// two shared-memory words per lane and one MMA give the 8 x 8 exact int32 block sums that the
// dp4a kernel needs 8 dp4a per row and activation row for.  (Eight rows, not the sixteen the
// instruction could take: a stage of whole rows is then half as large and the ring holds four of
// them.)  The per-block scaling stays the reference's
// (src/gpu/cuda/elt.zig:1984-2005):
//   acc += float(sumi) * (d_w * d_x)   in f32, block after block.
// Rows too long for the registers (more than 12 block pairs per warp) are taken in several
// passes over K: a pass streams one K range of all the CTA's rows, and the passes after the
// first add to the y the first one wrote.  Where that halves the number of passes, K is split
// across a cluster of two CTAs instead: both stream the same rows (twice as many as a lone CTA
// would own, so the 8-row stages divide them better), each its own half of K in one pass; the
// second CTA stores its sums into the first one's shared memory as it goes, and after one cluster
// barrier at the end the first CTA adds the two parts and writes y.
//
// Data path.  One CTA per SM owns a contiguous range of weight rows.  Four producer warps stream
// them in stages of 8 rows x one K segment with 1-D bulk copies (cp.async.bulk, completion on the
// stage's "full" mbarrier, no multicast) into a ring that fills most of shared memory; they start
// before griddepcontrol.wait, so under programmatic dependent launch the ring fills while the
// previous kernel drains.  What bounds this kernel is how fast copies can be issued, not the
// arithmetic: a warp gets a bulk copy under way only every few hundred cycles (more when memory is
// busy), and a producer's round "stage released -> fence -> expect -> copies" took 0.6 us per stage
// with one copy per row and 22 KB stages -- less than the memory system delivers.  Hence few, large
// copies: the fewest K segments that still leave four stages, and where a stage is whole rows
// (one pass, one segment, K not split) its rows, which are contiguous in the weight, come with ONE
// copy per group of rows (see plan_mma_ks for the bank arithmetic).  The warps whose K slice lies
// in a stage's segment wait for it, multiply, write their 8 x 8 partial sums to a small buffer and
// arrive on the stage's "empty" mbarrier.  When the last segment of a row group has been released
// and its refill is under way, the first producer warp adds the partials in warp order (a fixed
// order: results do not depend on timing), applies `scale` and stores y; the refilled stage counts
// as full only after that, so partial buffers are never overwritten early.  No warp ever waits for
// another consumer warp.  (Handing a stage back before the arithmetic, from registers, and letting
// the last consumer warp add the partials were both measured: slower.)
//
// Rows in shared memory start 4 words apart modulo 32 banks, so the 8 rows x 4 words an A fragment
// load touches fall in 32 different banks.
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
constexpr int kProducers = 4;                  // producer warps 16..19, two rows of every stage each
constexpr int kThreadsMma = (kConsumers + kProducers) * 32;
constexpr int kStageRows = 8;                  // weight rows per stage (rows 0..7 of the MMA's m side)
constexpr int kActRows = 8;                    // activation rows = n of the MMA
constexpr int kPartFloats = kStageRows * kActRows;

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
    int grp_rows;      // rows one bulk copy brings in (1, 2, 4 or 8; > 1 only when a stage is whole rows)
    int grp_shift;     // extra bytes before every further copy's rows (keeps the 8 rows on distinct banks)
    int stages;        // ring depth
    int rgbuf;         // row groups of partial sums kept
    int out_rg;        // K split: row groups of unscaled sums a CTA keeps for the final addition
    uint32_t *status;
};

// Pass p of a row covers blocks [pass_blk0(p), pass_blk0(p + 1)); K segment s of a pass covers
// [seg_blk0(s), seg_blk0(s + 1)) of those.  Both are whole units of 8 blocks (272 bytes, a multiple of 16).
// (32-bit arithmetic on purpose: nblk <= 2^19, p, s <= 16, and a 64-bit division costs hundreds of
// cycles on the GPU -- four of them per stage made the producer warps the bottleneck of the kernel.)
__host__ __device__ inline int pass_blk0(int nblk, int npass, int p) { return (nblk / 8) * p / npass * 8; }
__host__ __device__ inline int seg_blk0(int pb0, int pb1, int nseg, int s) { return pb0 + ((pb1 - pb0) / 8) * s / nseg * 8; }
// pairs [lo, hi) of consumer `wi` (0 .. wps-1) inside a segment of `pairs` block pairs
__host__ __device__ inline int warp_pair0(int pairs, int wps, int wi) { return pairs * wi / wps; }

// C[8 weight rows][8 activation rows] = A[8 (of 16)][32] * B[32][8], int8 -> int32, C starts at zero.
// Lane (g = lane / 4, t = lane % 4): a0/a2 = weight row g, k = 4t.. and 16+4t..; a1/a3 (rows 8..15)
// are zero; b0/b1 = activation row g, same k; c0, c1 = weight row g x activation rows 2t, 2t+1.
// The accumulators start at the bit pattern of 1.5 * 2^23 (kI2FMagicBits), so that each int32 result, read as a
// float, is that constant plus the block sum (|sum| <= 32 * 127 * 128 < 2^22): no integer-to-float conversion.
__device__ __forceinline__ void mma_s8(int &c0, int &c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    int c2, c3;
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%8,%5,%8}, {%6,%7}, {%9,%9,%8,%8};"
        : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
        : "r"(a0), "r"(a2), "r"(b0), "r"(b1), "r"(0), "r"(kI2FMagicBits));
    (void)c2;
    (void)c3;
}

// Two packed f32 values; each half rounds like the scalar instruction.
typedef unsigned long long f2;
__device__ __forceinline__ f2 pack2(float lo, float hi) {
    f2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ f2 pack2i(int lo, int hi) {
    f2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
__device__ __forceinline__ f2 sub2(f2 a, f2 b) {
    f2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
    f2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2 lds_f2x(uint32_t addr) {
    f2 v;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr));
    return v;
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

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 20 warps: 65536 / 640 = 102 registers per thread, 96 after rounding to the allocation unit.
// KS = CTAs per cluster = parts K is split into (1 or 2).
template <int NP, int KS>
__global__ void __cluster_dims__(KS, 1, 1) __launch_bounds__(kThreadsMma, 1) q8_0_gemv_mma_kernel(const MmaGemvParams p) {
    // pairs whose loads and MMAs are issued before any of their results is used: three while the registers
    // last (short K slices), two beyond -- a spill costs a trip to L2 here, the ring leaves almost no L1
    constexpr int kGroup = NP <= 6 ? 3 : 2;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nblk = p.nblk;
    const int S = p.stages;
    const int stage_bytes = kStageRows * p.pitch + (kStageRows / p.grp_rows) * p.grp_shift;
    const size_t row_bytes = (size_t)nblk * kBlockBytes;

    uint8_t *ring = smem;
    float *s_dx = reinterpret_cast<float *>(smem + (size_t)S * stage_bytes);       // [nblk][8 activation rows]
    float *s_part = s_dx + (size_t)kActRows * nblk;                                 // [rgbuf][kConsumers][8 weight rows x 8 activation rows]
    const uint32_t bars = smem_u32(s_part + (size_t)p.rgbuf * kConsumers * kPartFloats);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    // first block of every (pass, segment), plus one entry that closes the last segment of each pass:
    // s_seg[pass * (nseg + 1) + seg]; looked up instead of recomputed (integer divisions) per stage
    int *s_seg = reinterpret_cast<int *>(s_part + (size_t)p.rgbuf * kConsumers * kPartFloats) + 2 * 2 * 16;
    // K split: this CTA's passes are passes crank * npass .. of npass * KS over the whole row
    const int crank = KS > 1 ? (int)cluster_rank() : 0;
    const int npt = p.npass * KS;
    for (int e = threadIdx.x; e < p.npass * (p.nseg + 1); e += blockDim.x) {
        const int ps = e / (p.nseg + 1), sg = e - ps * (p.nseg + 1);
        const int gp = crank * p.npass + ps;
        s_seg[e] = seg_blk0(pass_blk0(nblk, npt, gp), pass_blk0(nblk, npt, gp + 1), p.nseg, sg);
    }
    float *s_out = reinterpret_cast<float *>(s_seg + 8 * 17);   // [KS][out_rg][8 weight rows][8 activation rows], KS > 1 only

    const int wps = kConsumers / p.nseg;  // consumer warps per K segment
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(kProducers + 1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(wps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // this CTA's rows and its stages: (pass, row group, segment), row groups of 8 rows
    // (the CTAs of a cluster share their rows)
    const int n_own = (int)gridDim.x / KS, own = (int)blockIdx.x / KS;
    const int r_base = p.rows / n_own, r_rem = p.rows % n_own;   // the first r_rem owners take one row more
    const int r_begin = own * r_base + min(own, r_rem);
    const int r_end = r_begin + r_base + (own < r_rem ? 1 : 0);
    const int n_rg = (r_end - r_begin + kStageRows - 1) / kStageRows;
    const int total = p.npass * n_rg * p.nseg;

    if (warp >= kConsumers) {
        // ---------------- producers (the first one also adds the partial sums) ----------------
        const int pw = warp - kConsumers;
        // the stage the next issue() fills: (pass, row group, segment), ring slot, all advanced by one per call
        int is_pass = 0, is_rg = 0, is_seg = 0, is_slot = 0;
        auto issue = [&]() {  // whole warp: lane l starts copy number pw + 4 l of the next stage (a copy = grp_rows rows)
            const int row0 = r_begin + is_rg * kStageRows;
            const int nrow = min(kStageRows, r_end - row0);
            const int b0 = s_seg[is_pass * (p.nseg + 1) + is_seg], b1 = s_seg[is_pass * (p.nseg + 1) + is_seg + 1];
            const uint32_t bytes = (uint32_t)(b1 - b0) * kBlockBytes;   // per row
            const uint32_t bar = full_bar(is_slot);
            const int cp = pw + kProducers * lane;                      // this lane's copy
            const int cp_row0 = cp * p.grp_rows;
            const int cp_rows = max(0, min(p.grp_rows, nrow - cp_row0));
            // rows of all this warp's copies (lanes 0 and 1; at most eight copies per stage)
            const int cp_rows1 = max(0, min(p.grp_rows, nrow - (cp_row0 + kProducers * p.grp_rows)));
            if (lane == 0)   // every producer warp arrives, also with nothing to copy (the barrier counts them all)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                             "r"(bytes * (uint32_t)(cp_rows + cp_rows1))
                             : "memory");
            __syncwarp();
            const uint32_t dst = smem_u32(ring) + (uint32_t)(is_slot * stage_bytes);
            const uint8_t *src = p.w + (size_t)row0 * row_bytes + (size_t)b0 * kBlockBytes;
            if (lane < 2 && cp_rows > 0)
                bulk_g2s(dst + (uint32_t)(cp_row0 * p.pitch + cp * p.grp_shift), src + (size_t)cp_row0 * row_bytes,
                         bytes * (uint32_t)cp_rows, bar);
            if (++is_slot == S) is_slot = 0;
            if (++is_seg == p.nseg) {
                is_seg = 0;
                if (++is_rg == n_rg) {
                    is_rg = 0;
                    is_pass++;
                }
            }
        };
        auto reduce = [&](int pass, int rg, int pbuf) {  // all lanes: y of one row-group visit from the consumers' partial sums
            // a warp's partials: [8 weight rows][8 activation rows]; this lane: row lane / 4, activation rows 2 (lane % 4) ..
            const float *part = s_part + (size_t)pbuf * kConsumers * kPartFloats + 2 * lane;
            float2 sum = make_float2(0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kConsumers; w++) {
                const float2 pv = *reinterpret_cast<const float2 *>(part + w * kPartFloats);
                sum.x += pv.x;
                sum.y += pv.y;
            }
            const int row = r_begin + rg * kStageRows + (lane >> 2);
            const int m0 = 2 * (lane & 3);
            if (KS > 1) {
                // Unscaled sums of this CTA's part of K.  Passes before the last accumulate here; the last one
                // sends the total to the cluster's first CTA, part `crank` of its s_out (a remote shared-memory
                // store: nothing waits for it, the cluster barrier at the end makes it visible), which adds
                // the parts and writes y.
                float2 *o = reinterpret_cast<float2 *>(s_out + ((size_t)crank * p.out_rg + rg) * kPartFloats + 2 * lane);
                if (pass != 0) {
                    const float2 prev = *o;
                    sum.x += prev.x;
                    sum.y += prev.y;
                }
                if (pass != p.npass - 1 || crank == 0) {
                    *o = sum;
                } else {
                    uint32_t ra;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(o)), "r"(0));
                    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(ra), "f"(sum.x), "f"(sum.y) : "memory");
                }
            } else if (row < r_end) {
                // later passes add to what this same lane stored in the pass before
                const float v2[2] = {sum.x, sum.y};
#pragma unroll
                for (int e = 0; e < 2; e++)
                    if (m0 + e < p.m) {
                        float *dst = p.y + (size_t)(m0 + e) * p.rows + row;
                        *dst = pass == 0 ? v2[e] * p.scale : fmaf(v2[e], p.scale, *dst);
                    }
            }
        };
        // weights are constants: the ring starts filling before the previous kernel has finished
        for (int i = 0; i < S && i < total; i++) {
            if (pw == 0 && lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_bar(is_slot)) : "memory");
            issue();
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        bool ok = true;
        // the stage whose release is awaited next: ring slot and phase, segment, row group, pass, partial buffer
        int w_slot = 0, w_seg = 0, w_rg = 0, w_pass = 0, w_pbuf = 0;
        uint32_t w_par = 0;
        for (int j = 0; j < total && ok; j++) {
            // stage j has been consumed by its warps
            ok = mbar_wait(empty_bar(w_slot), w_par, p.status, (7u << 24) | (uint32_t)w_slot);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t refill_bar = full_bar(is_slot);
            if (j + S < total) {
                // order the consumers' generic-proxy reads of the slot before the async-proxy refill
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue();
            }
            // The refill is under way; the first producer warp now adds the partial sums of a finished row
            // group and only then gives the refilled stage its last arrival: the stage is not "full" without
            // it, so no consumer can overwrite a partial that is still needed, and the copies did not have to
            // wait for the additions.
            if (pw == 0) {
                if (w_seg == p.nseg - 1) reduce(w_pass, w_rg, w_pbuf);
                __syncwarp();
                if (lane == 0 && j + S < total) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(refill_bar) : "memory");
            }
            if (++w_slot == S) {
                w_slot = 0;
                w_par ^= 1u;
            }
            if (++w_seg == p.nseg) {
                w_seg = 0;
                if (++w_pbuf == p.rgbuf) w_pbuf = 0;
                if (++w_rg == n_rg) {
                    w_rg = 0;
                    w_pass++;
                }
            }
        }
    } else {
    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    const int seg = warp / wps, wi = warp - seg * wps;

    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool ok = true;
    // this warp's next stage: ring slot and phase (it takes every nseg-th stage), partial buffer
    int c_slot = seg % S, c_pbuf = 0;
    uint32_t c_par = (uint32_t)(seg / S) & 1u;
  for (int pass = 0; pass < p.npass && ok; pass++) {
    const int sb0 = s_seg[pass * (p.nseg + 1) + seg], sb1 = s_seg[pass * (p.nseg + 1) + seg + 1];
    const int seg_pairs = (sb1 - sb0) / 2;
    const int pp0 = warp_pair0(seg_pairs, wps, wi), pp1 = warp_pair0(seg_pairs, wps, wi + 1);
    const int np = pp1 - pp0;  // <= NP (checked by the host)
    // this lane's part of the B operand: activation row g, K positions of its pairs in this pass.
    // A pair's 64 activation bytes are 16 words; lane (g, t) needs words t, 4+t (first block) and
    // 8+t, 12+t (second block).  It loads words 4t .. 4t+3 with one 16-byte load -- the quad then covers
    // the pair's 64 contiguous bytes, where four 4-byte loads per lane took four times as many
    // instructions with eight rows (eight cache lines) each, and with many activation rows that
    // address traffic alone cost microseconds before the first weight byte was used -- and the
    // quad transposes its 4 x 4 words with two exchange steps.
    uint32_t b[NP][4];
#pragma unroll
    for (int q = 0; q < NP; q++) {
        b[q][0] = b[q][1] = b[q][2] = b[q][3] = 0u;
        if (q < np && g < p.m) {
            const int blk = sb0 + 2 * (pp0 + q);
            const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(p.xq + (size_t)g * p.cols + (size_t)blk * 32) + t);
            b[q][0] = v.x; b[q][1] = v.y; b[q][2] = v.z; b[q][3] = v.w;
        }
    }
    {
        // Activation scales of this warp's blocks in this pass, all 8 (padded) activation rows, into the
        // warp's own part of s_dx ([block][activation row]: the four lanes t of a quad then read 32
        // contiguous bytes per block; row-major [m][nblk] put all four in one bank).  Issued after the
        // loads above so that the round trips overlap; nobody else reads this part, so a warp
        // barrier is all it takes.
        const int blk0 = sb0 + 2 * pp0;
        float v[kActRows];     // lane = block of the warp's slice (at most 2 NP <= 24 of them)
#pragma unroll
        for (int m = 0; m < kActRows; m++)
            v[m] = (lane < 2 * np && m < p.m) ? __ldcg(p.xd + (size_t)m * nblk + blk0 + lane) : 0.0f;
        if (lane < 2 * np) {
            float4 *d = reinterpret_cast<float4 *>(s_dx + (size_t)(blk0 + lane) * kActRows);
            d[0] = make_float4(v[0], v[1], v[2], v[3]);
            d[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
        __syncwarp();
    }
#pragma unroll
    for (int q = 0; q < NP; q++) {
        // all 32 lanes take part in the shuffles (q < np is warp-uniform)
        if (q < np) {
            {
                // 4 x 4 transpose inside the quad: b[q][j] of lane t = word 4t+j  ->  word 4j+t
                const bool hi2 = (t & 2) != 0, hi1 = (t & 1) != 0;
                const uint32_t x0 = hi2 ? b[q][0] : b[q][2], x1 = hi2 ? b[q][1] : b[q][3];
                const uint32_t y0 = __shfl_xor_sync(0xffffffffu, x0, 2), y1 = __shfl_xor_sync(0xffffffffu, x1, 2);
                if (hi2) { b[q][0] = y0; b[q][1] = y1; } else { b[q][2] = y0; b[q][3] = y1; }
                // now b[q][2a+c] = word 4((t&1)+2a) + 2(t>>1)+c; exchange the off-column with lane t^1
                const uint32_t z0 = __shfl_xor_sync(0xffffffffu, hi1 ? b[q][0] : b[q][1], 1);
                const uint32_t z1 = __shfl_xor_sync(0xffffffffu, hi1 ? b[q][2] : b[q][3], 1);
                if (hi1) { b[q][0] = z0; b[q][2] = z1; } else { b[q][1] = z0; b[q][3] = z1; }
            }
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
    const uint32_t ring_u32 = smem_u32(ring) + (uint32_t)(pp0 * kPairBytes) + (uint32_t)(g * p.pitch + (g / p.grp_rows) * p.grp_shift) + 4u * (uint32_t)t;
    // activation scales of activation rows 2t and 2t+1, this warp's first block
    const uint32_t dx_u32 = smem_u32(s_dx + (size_t)(sb0 + 2 * pp0) * kActRows + 2 * t);

    for (int rg = 0; rg < n_rg && ok; rg++) {
        ok = mbar_wait(full_bar(c_slot), c_par, p.status, (8u << 24) | (uint32_t)c_slot);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t wl = ring_u32 + (uint32_t)(c_slot * stage_bytes);
        f2 acc = 0ull;
        const f2 magic2 = pack2(kI2FMagic, kI2FMagic);
        // kGroup pairs at a time: first every load and both MMAs of each pair (independent of one
        // another, so the loads and the tensor-core latencies overlap), then the scaling.
#pragma unroll
        for (int q0 = 0; q0 < NP; q0 += kGroup) {
            int c[kGroup][4];
            uint32_t sc[kGroup][2];
#pragma unroll
            for (int u = 0; u < kGroup; u++) {
                const int q = q0 + u;
                if (q < NP && q < np) {
                    const uint32_t o = (uint32_t)(q * kPairBytes);
                    // words t, 4+t, 8 (and 0 for the scale) of the first block, 9+t and 13+t of the second
                    const uint32_t l0 = lds32(wl + o - 4u * t), l_lo = lds32(wl + o), l_hi = lds32(wl + o + 16);
                    const uint32_t l8 = lds32(wl + o + 32 - 4u * t), l_v0 = lds32(wl + o + 36), l_v1 = lds32(wl + o + 52);
                    mma_s8(c[u][0], c[u][1], t == 0 ? __funnelshift_r(l_lo, l8, 16) : l_lo, l_hi, b[q][0], b[q][1]);
                    mma_s8(c[u][2], c[u][3], l_v0, l_v1, b[q][2], b[q][3]);
                    sc[u][0] = l0;
                    sc[u][1] = l8;
                }
            }
#pragma unroll
            for (int u = 0; u < kGroup; u++) {
                const int q = q0 + u;
                if (q < NP && q < np) {
                    // scales of activation rows (2t, 2t+1) for the pair's first and second block
                    const f2 dx0 = lds_f2x(dx_u32 + 64u * q), dx1 = lds_f2x(dx_u32 + 64u * q + 32u);
                    // weight scales: f16 in the low half of word 0 (first block) and the high half of word 8 (second)
                    const float d0 = f16lo(sc[u][0]), d1 = f16hi(sc[u][1]);
                    // acc += float(sumi) * (d_w * d_x) for both activation rows at once (two-wide f32 instructions,
                    // each half rounded like the scalar one)
                    acc = fma2(sub2(pack2i(c[u][0], c[u][1]), magic2), mul2(pack2(d0, d0), dx0), acc);
                    acc = fma2(sub2(pack2i(c[u][2], c[u][3]), magic2), mul2(pack2(d1, d1), dx1), acc);
                }
            }
        }
        // this warp's K slice of C[weight row g][activation rows 2t, 2t+1]
        float *part = s_part + ((size_t)c_pbuf * kConsumers + warp) * kPartFloats;
        *reinterpret_cast<f2 *>(part + g * kActRows + 2 * t) = acc;
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(empty_bar(c_slot)) : "memory");
        c_slot += p.nseg;
        while (c_slot >= S) {
            c_slot -= S;
            c_par ^= 1u;
        }
        if (++c_pbuf == p.rgbuf) c_pbuf = 0;
    }
  }
    }
    if (KS > 1) {
        // Every thread of both CTAs gets here, also after a wait that gave up.  The barrier makes the sums
        // the other CTAs stored into the first CTA's shared memory complete and visible; they may leave.
        cluster_barrier();
        if (crank == 0) {
            const int nrows = r_end - r_begin;
            for (int i = threadIdx.x; i < nrows * p.m; i += blockDim.x) {
                const int m = i / nrows, r = i - m * nrows;
                float v = s_out[r * kActRows + m];
#pragma unroll
                for (int c = 1; c < KS; c++) v += s_out[(size_t)c * p.out_rg * kPartFloats + r * kActRows + m];
                p.y[(size_t)m * p.rows + r_begin + r] = v * p.scale;
            }
        }
    }
}

struct MmaPlan {
    int npass = 0, nseg = 0, pitch = 0, grp_rows = 1, grp_shift = 0, stages = 0, rgbuf = 0, max_pairs = 0;
    int ks = 1, out_rg = 0, grid = 0;
    size_t smem = 0;
};

constexpr int kMaxPairs = 12;   // block pairs a consumer warp can keep in registers (largest instantiation)

// Ring geometry for `nblk` blocks per row with K split over `ks` CTAs: the fewest passes over a
// CTA's part of K whose K slices fit the registers, then the fewest segments that still give a
// ring of at least 6 stages (else the deepest ring).  `extra` bytes of shared memory are kept free.
// npass = 0 when nothing fits.
MmaPlan plan_mma_ks(tpb_handle_t h, int nblk, int ks, size_t extra) {
    const size_t limit = (size_t)h->smem_optin - 1024 - extra;
    const int min_stages = 4;
    for (int npass = 1; npass <= 8 / ks; npass++) {
        if (nblk / 8 < npass * ks) break;
        MmaPlan best;
        for (int nseg = 1; nseg <= kConsumers; nseg *= 2) {
            int seg_blocks = 0, max_pairs = 0;
            bool ok = true;
            const int wps = kConsumers / nseg;
            for (int ps = 0; ps < npass * ks && ok; ps++) {
                const int pb0 = pass_blk0(nblk, npass * ks, ps), pb1 = pass_blk0(nblk, npass * ks, ps + 1);
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
            // Rows at 4 words modulo 32 banks, 16-byte aligned: by padding the pitch when every row comes
            // with its own copy.  A stage of whole rows (one pass, one segment, K not split) is contiguous
            // in the weight: its rows keep their pitch in memory, 4 u words modulo 32 with u = nblk / 8,
            // and come in copies of as many rows as fall on distinct banks that way (8 / gcd(u, 8)), every
            // further copy 16 bytes later.  Fewer, larger copies: the producers' issue rate was the limit
            // of the kernel with one copy per row and 22 KB stages.
            int pitch, grp_rows = 1, grp_shift = 0;
            if (npass * ks == 1 && nseg == 1) {
                const int u = (nblk / 8) % 8;
                int gcd = 8;
                while (u % gcd != 0) gcd /= 2;     // gcd(u, 8); u = 0 gives 8
                grp_rows = 8 / gcd;
                grp_shift = grp_rows > 1 ? 16 : 0;
            }
            if (grp_rows > 1) {
                pitch = seg_blocks * kBlockBytes;
            } else {
                int pitch_w = seg_blocks * kBlockBytes / 4;
                pitch_w += ((4 - pitch_w % 32) + 32) % 32;
                pitch = pitch_w * 4;
            }
            const size_t stage = (size_t)kStageRows * pitch + (size_t)(kStageRows / grp_rows) * grp_shift;
            const size_t fixed = (size_t)kActRows * nblk * 4 + 64 + 2 * 8 * 16 + 4 * 8 * 17;   // + the segment table
            for (int stages = 12; stages >= 3; stages--) {
                const int rgbuf = (stages - 1 + nseg - 1) / nseg + 1;
                const size_t smem = stages * stage + fixed + (size_t)rgbuf * kConsumers * kPartFloats * 4;
                if (smem > limit) continue;
                if (best.npass == 0 || (best.stages < min_stages && stages > best.stages)) {
                    best.npass = npass;
                    best.nseg = nseg;
                    best.pitch = pitch;
                    best.grp_rows = grp_rows;
                    best.grp_shift = grp_shift;
                    best.stages = stages;
                    best.rgbuf = rgbuf;
                    best.max_pairs = max_pairs;
                    best.smem = smem;
                }
                break;
            }
            if (best.npass != 0 && best.stages >= min_stages) break;
        }
        if (best.npass != 0) {
            best.ks = ks;
            return best;
        }
    }
    return MmaPlan();
}

constexpr int kMaxOutRg = 64;   // K split: row groups a cluster may own (16 KB of sums per CTA)

// One CTA per SM, each with all of K -- unless the rows need several passes over K and splitting K
// over a pair of CTAs halves them: then pairs of CTAs share twice as many rows.
MmaPlan plan_mma(tpb_handle_t h, int64_t rows, int nblk) {
    MmaPlan one = plan_mma_ks(h, nblk, 1, 0);
    long long grid = (rows + kStageRows - 1) / kStageRows;
    if (grid > h->sm_count) grid = h->sm_count;
    one.grid = (int)grid;
    const char *e = getenv("TPB_GEMV_KSPLIT");   // "0": never split K (measurements; read per launch)
    if (one.npass == 1 || h->sm_count < 2 || (e && e[0] == '0')) return one;
    long long owners = (rows + kStageRows - 1) / kStageRows;
    if (owners > h->sm_count / 2) owners = h->sm_count / 2;
    const int out_rg = (int)(((rows + owners - 1) / owners + kStageRows - 1) / kStageRows);
    if (out_rg > kMaxOutRg) return one;
    MmaPlan two = plan_mma_ks(h, nblk, 2, (size_t)2 * out_rg * kPartFloats * 4);
    if (two.npass == 0 || (one.npass != 0 && two.npass * 2 > one.npass)) return one;
    two.out_rg = out_rg;
    two.smem += (size_t)2 * out_rg * kPartFloats * 4;
    two.grid = (int)(2 * owners);
    return two;
}

template <int NP, int KS>
int launch_np(tpb_handle_t h, cudaStream_t st, const MmaGemvParams &p, const MmaPlan &pl) {
    auto kern = q8_0_gemv_mma_kernel<NP, KS>;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3((unsigned)pl.grid), dim3(kThreadsMma), pl.smem, st, p));
    return TPB_OK;
}

}  // namespace

// 0 when the activation-stationary kernel cannot take this shape, else the number of CTAs K is split over;
// *npass = its passes over K, *np_waste_pct = block pairs a warp's MMAs cover per pair it needs, in percent
// (the kernel is instantiated for 6, 9 and 12 pairs per warp).
int tpb_q8_0_gemv_mma_fits(tpb_handle_t h, int64_t rows, int64_t cols, int *npass, int *np_waste_pct) {
    if (cols % 256 != 0 || rows < 1) return 0;
    const MmaPlan pl = plan_mma(h, rows, (int)(cols / 32));
    if (pl.npass == 0) return 0;
    const int np = pl.max_pairs <= 6 ? 6 : pl.max_pairs <= 9 ? 9 : 12;
    if (npass) *npass = pl.npass;
    if (np_waste_pct) *np_waste_pct = pl.max_pairs > 0 ? 100 * np / pl.max_pairs : 100;
    return pl.ks;
}

int tpb_launch_q8_0_gemv_mma(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale, int64_t rows,
                             int64_t cols, const void *xq, int ng, int row_off, int n_total) {
    const int nblk = (int)(cols / 32);
    const MmaPlan pl = plan_mma(h, rows, nblk);
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
    p.grp_rows = pl.grp_rows;
    p.grp_shift = pl.grp_shift;
    p.stages = pl.stages;
    p.rgbuf = pl.rgbuf;
    p.out_rg = pl.out_rg;
    p.status = h->d_status;
    if (pl.ks == 2) {
        if (pl.max_pairs <= 6) return launch_np<6, 2>(h, st, p, pl);
        if (pl.max_pairs <= 9) return launch_np<9, 2>(h, st, p, pl);
        return launch_np<kMaxPairs, 2>(h, st, p, pl);
    }
    if (pl.max_pairs <= 6) return launch_np<6, 1>(h, st, p, pl);
    if (pl.max_pairs <= 9) return launch_np<9, 1>(h, st, p, pl);
    return launch_np<kMaxPairs, 1>(h, st, p, pl);
}
