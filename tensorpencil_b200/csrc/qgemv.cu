// GGUF Q8_0 decode GEMV family for sm_100a (CUDA cores, dp4a + warp reductions;
// HBM-bound: the weight matrix streams once for up to 8 activation rows).
//
// A Q8_0 row is k/32 blocks of 34 bytes (f16 d, then 32 int8); blocks are only
// 2-byte aligned, which is what makes per-lane global loads of them expensive.
// Here the weight never goes through the load/store unit on its way in: each
// warp streams its rows into a private shared-memory ring with 1-D bulk async
// copies (cp.async.bulk, completion on an mbarrier, no multicast), several
// stages ahead of the arithmetic.  A lane then takes a PAIR of adjacent blocks
// (68 bytes = 17 aligned words, lane stride 17 words => no bank conflicts): the
// second block's quants are already word-aligned, the first block's need one
// funnel shift per word.  Activations (int8 + per-block scale, the q8_1 form)
// sit in shared memory for the whole kernel and are reused across the R rows a
// warp handles at once.
//
// Arithmetic follows the reference kernel (src/gpu/cuda/elt.zig:1926-2006,
// :1663-1709): per block sumi = sum of 32 int8 products (exact), then
// acc += float(sumi) * (d_w * d_x) in f32, a butterfly reduction across the
// warp, and y = acc * scale.
#include <cuda_fp16.h>


#include "qgemv_common.cuh"

using namespace tpb_gemv;

namespace {

constexpr int kBlockBytes = 34;
constexpr int kPairsPerChunk = 32;                 // one block pair per lane
constexpr int kChunkBlocks = 2 * kPairsPerChunk;   // 64 blocks
constexpr int kChunkBytes = kChunkBlocks * kBlockBytes;  // 2176 per row (multiple of 16)
constexpr int kActPairBytes = 80;  // a block pair's 64 activation bytes + 16 pad: 16-byte reads at lane stride 80 hit distinct banks
__host__ __device__ constexpr int stage_bytes(int rows_per_group) { return rows_per_group * kChunkBytes; }

struct GemvParams {
    float *y;
    const uint8_t *w;
    const float *xd;   // activation block scales, row 0 of the group: [ng][nblk] with stride nblk
    const int8_t *xq;  // activation quants: [ng][cols]
    float scale;
    int rows, cols, nblk;
    uint32_t *status;
};

// M activation rows, R weight rows a warp processes together (compile time).
// ACT_SMEM: activations staged in shared memory.  Every warp of the grid owns a
// contiguous, nearly equal range of weight rows.
template <int M, int R, bool ACT_SMEM>
__global__ void __launch_bounds__(R == 2 ? 512 : 256, 1)
q8_0_gemv_q8n_kernel(const GemvParams p, const int stages) {
    constexpr int kRows = R;
    constexpr int kStageBytes = stage_bytes(R);
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_warps = blockDim.x >> 5;
    const int nblk = p.nblk;
    const int cols = p.cols;
    const size_t row_bytes = (size_t)nblk * kBlockBytes;

    // shared layout: [act q: M rows of (nblk/2) padded pairs][act d: M*nblk f32][per-warp: stages*kStageBytes][barriers]
    const size_t act_row = (size_t)(nblk / 2) * kActPairBytes;
    int8_t *s_q = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (ACT_SMEM ? (size_t)M * act_row : 0));
    uint8_t *ring0 = smem + (ACT_SMEM ? (size_t)M * act_row + (size_t)M * nblk * 4 : 0);
    uint8_t *ring = ring0 + (size_t)warp * stages * kStageBytes;
    const uint32_t bars = smem_u32(ring0 + (size_t)n_warps * stages * kStageBytes) + warp * stages * 8;

    // Each warp's barriers are used by that warp alone: initialise them, then start
    // streaming weights right away.  Weights are constants, so under programmatic
    // dependent launch this runs while the previous kernel in the stream is still
    // draining; activations and outputs are only touched after griddepcontrol.wait.
    if (lane == 0) {
        for (int s = 0; s < stages; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + 8 * s), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int cpr = (nblk + kChunkBlocks - 1) / kChunkBlocks;  // chunks per row
    const int gw = blockIdx.x * n_warps + warp;
    const int GW = gridDim.x * n_warps;
    const int my_r0 = (int)((long long)p.rows * gw / GW);        // this warp's rows: [my_r0, my_r1)
    const int my_r1 = (int)((long long)p.rows * (gw + 1) / GW);
    const int my_rg = (my_r1 - my_r0 + kRows - 1) / kRows;       // groups of up to R rows
    const int total = my_rg * cpr;

    auto issue = [&](int i) {
        // lane 0 only: start the copies of iteration i into its stage
        const int c = i % cpr;
        const int st = i % stages;
        const int row0 = my_r0 + (i / cpr) * kRows;
        const int nrow = min(kRows, my_r1 - row0);
        const int blocks = min(kChunkBlocks, nblk - c * kChunkBlocks);
        const uint32_t bytes = (uint32_t)blocks * kBlockBytes;
        const uint32_t bar = bars + 8 * st;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                     "r"(bytes * (uint32_t)nrow)
                     : "memory");
        const uint32_t dst = smem_u32(ring + (size_t)st * kStageBytes);
        for (int r = 0; r < nrow; r++)
            bulk_g2s(dst + r * kChunkBytes, p.w + (size_t)(row0 + r) * row_bytes + (size_t)c * kChunkBytes,
                     bytes, bar);
    };

    if (lane == 0)
        for (int i = 0; i < stages - 1 && i < total; i++) issue(i);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (ACT_SMEM) {
        const int4 *gq = reinterpret_cast<const int4 *>(p.xq);
        const int per_row = cols / 16;  // 16-byte pieces per activation row, 4 per block pair
        for (int i = threadIdx.x; i < M * per_row; i += blockDim.x) {
            const int m = i / per_row, c16 = i - m * per_row;
            *reinterpret_cast<int4 *>(s_q + (size_t)m * act_row + (size_t)(c16 >> 2) * kActPairBytes + (c16 & 3) * 16) =
                __ldcg(gq + i);
        }
        for (int i = threadIdx.x; i < M * nblk; i += blockDim.x) s_d[i] = __ldcg(p.xd + i);
    }
    __syncthreads();

    float acc[kRows][M];
#pragma unroll
    for (int r = 0; r < kRows; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = 0.0f;

    bool ok = true;
    for (int i = 0; i < total && ok; i++) {
        // the stage refilled here was consumed in iteration i-1 (warp-synchronous)
        if (lane == 0 && i + stages - 1 < total) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(i + stages - 1);
        }
        const int st = i % stages;
        ok = mbar_wait(bars + 8 * st, (uint32_t)(i / stages) & 1u, p.status, (4u << 24) | (uint32_t)st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;

        const int c = i % cpr;
        const int row0 = my_r0 + (i / cpr) * kRows;
        const int nrow = min(kRows, my_r1 - row0);
        const int blk0 = c * kChunkBlocks + 2 * lane;  // first block of this lane's pair
        const bool live = blk0 < nblk;                  // nblk is even
        if (live) {
            // weights: 17 aligned words per row, quants of block A funnel-shifted by 16 bits
            uint32_t wq[kRows][16];
            float wd[kRows][2];
            const uint8_t *stage = ring + (size_t)st * kStageBytes + lane * (2 * kBlockBytes);
#pragma unroll
            for (int r = 0; r < kRows; r++) {
                if (r < nrow) {
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(stage + r * kChunkBytes);
                    uint32_t t[17];
#pragma unroll
                    for (int j = 0; j < 17; j++) t[j] = src[j];
#pragma unroll
                    for (int j = 0; j < 8; j++) wq[r][j] = __funnelshift_r(t[j], t[j + 1], 16);
#pragma unroll
                    for (int j = 0; j < 8; j++) wq[r][8 + j] = t[9 + j];
                    wd[r][0] = __half2float(__ushort_as_half((unsigned short)(t[0] & 0xffffu)));
                    wd[r][1] = __half2float(__ushort_as_half((unsigned short)(t[8] >> 16)));
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) wq[r][j] = 0;
                    wd[r][0] = wd[r][1] = 0.0f;
                }
            }
#pragma unroll
            for (int m = 0; m < M; m++) {
                uint32_t xq[16];
                float xd0, xd1;
                if (ACT_SMEM) {
                    const int4 *a = reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)(blk0 >> 1) * kActPairBytes);
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        const int4 t = a[v];
                        xq[4 * v] = t.x; xq[4 * v + 1] = t.y; xq[4 * v + 2] = t.z; xq[4 * v + 3] = t.w;
                    }
                    const float2 d2 = *reinterpret_cast<const float2 *>(s_d + (size_t)m * nblk + blk0);
                    xd0 = d2.x;
                    xd1 = d2.y;
                } else {
                    const int4 *a = reinterpret_cast<const int4 *>(p.xq + (size_t)m * cols + (size_t)blk0 * 32);
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        // plain (L1-cached, coherent) load: every weight row re-reads these, and unlike a
                        // read-only-path load it cannot be moved above griddepcontrol.wait
                        const int4 t = a[v];
                        xq[4 * v] = t.x; xq[4 * v + 1] = t.y; xq[4 * v + 2] = t.z; xq[4 * v + 3] = t.w;
                    }
                    const float2 d2 = *reinterpret_cast<const float2 *>(p.xd + (size_t)m * nblk + blk0);
                    xd0 = d2.x;
                    xd1 = d2.y;
                }
#pragma unroll
                for (int r = 0; r < kRows; r++) {
                    // the sums start at the bit pattern of 1.5 * 2^23, so that they ARE their own float
                    // conversion plus that constant (|sum| <= 32 * 127 * 128 < 2^22): see i2f_small
                    int s0 = kI2FMagicBits, s1 = kI2FMagicBits;
#pragma unroll
                    for (int j = 0; j < 8; j++) s0 = __dp4a((int)wq[r][j], (int)xq[j], s0);
#pragma unroll
                    for (int j = 0; j < 8; j++) s1 = __dp4a((int)wq[r][8 + j], (int)xq[8 + j], s1);
                    acc[r][m] = fmaf(__int_as_float(s0) - kI2FMagic, wd[r][0] * xd0, acc[r][m]);
                    acc[r][m] = fmaf(__int_as_float(s1) - kI2FMagic, wd[r][1] * xd1, acc[r][m]);
                }
            }
        }
        __syncwarp();

        if (c == cpr - 1) {
            // row group finished: reduce across the warp, write, reset
#pragma unroll
            for (int r = 0; r < kRows; r++)
#pragma unroll
                for (int m = 0; m < M; m++) {
                    float v = acc[r][m];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0 && r < nrow) p.y[(size_t)m * p.rows + row0 + r] = v * p.scale;
                    acc[r][m] = 0.0f;
                }
        }
    }
}

// Fallback for shapes the bulk-copy path cannot take (row size not a multiple of
// 16 bytes, i.e. cols % 256 != 0): one warp per weight row, 16-bit global loads.
template <int M>
__global__ void __launch_bounds__(256)
q8_0_gemv_q8n_simple_kernel(const GemvParams p) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= p.rows) return;
    const uint8_t *wrow = p.w + (size_t)warp * p.nblk * kBlockBytes;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; m++) acc[m] = 0.0f;
    for (int b = lane; b < p.nblk; b += 32) {
        const unsigned short *blk = reinterpret_cast<const unsigned short *>(wrow + (size_t)b * kBlockBytes);
        const float dw = __half2float(__ushort_as_half(blk[0]));
        uint32_t wq[8];
#pragma unroll
        for (int j = 0; j < 8; j++) wq[j] = (uint32_t)blk[1 + 2 * j] | ((uint32_t)blk[2 + 2 * j] << 16);
#pragma unroll
        for (int m = 0; m < M; m++) {
            const int *xq = reinterpret_cast<const int *>(p.xq + (size_t)m * p.cols + (size_t)b * 32);
            int s = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) s = __dp4a((int)wq[j], xq[j], s);
            acc[m] = fmaf(i2f_small(s), dw * p.xd[(size_t)m * p.nblk + b], acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; m++) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) p.y[(size_t)m * p.rows + warp] = v * p.scale;
    }
}

// q8_1 activation quantiser: one warp per 32-element block
// (src/gpu/cuda/elt.zig:1226-1269).
__global__ void __launch_bounds__(256)
q8_1_quantize_kernel(const float *__restrict__ x, float *__restrict__ d, int8_t *__restrict__ qs,
                     int nblk) {
    const int blk = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (blk >= nblk) return;
    const float xi = x[(size_t)blk * 32 + lane];
    float amax = fabsf(xi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(127.0f, amax);
    qs[(size_t)blk * 32 + lane] = (int8_t)__float2int_rn(__fmul_rn(xi, inv));
    if (lane == 0) d[blk] = __fdiv_rn(amax, 127.0f);
}

// M = 1 GEMV in f32 arithmetic on un-quantised activations
// (src/gpu/cuda/elt.zig:671-727): one warp per row, x staged in shared memory.
__global__ void __launch_bounds__(256)
q8_0_gemv_f32_kernel(float *__restrict__ y, const float *__restrict__ x, const uint8_t *__restrict__ w,
                     float scale, int rows, int cols) {
    extern __shared__ __align__(16) uint8_t smem[];
    float *sx = reinterpret_cast<float *>(smem);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) sx[i] = x[i];
    __syncthreads();
    const int nblk = cols / 32;
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
        const uint8_t *wrow = w + (size_t)row * nblk * kBlockBytes;
        float acc = 0.0f;
        for (int b = lane; b < nblk; b += 32) {
            const unsigned short *blk = reinterpret_cast<const unsigned short *>(wrow + (size_t)b * kBlockBytes);
            const float dw = __half2float(__ushort_as_half(__ldg(blk)));
            const float *xb = sx + b * 32;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const unsigned short two = __ldg(blk + 1 + j);
                const float q0 = (float)(signed char)(two & 0xff);
                const float q1 = (float)(signed char)(two >> 8);
                acc = fmaf(q0 * dw, xb[2 * j], acc);
                acc = fmaf(q1 * dw, xb[2 * j + 1], acc);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) y[row] = acc * scale;
    }
}

// Launch with programmatic stream serialisation: the kernel may begin before the
// previous kernel in the stream has finished; it orders itself with griddepcontrol.wait.
template <typename Kern>
cudaError_t launch_pdl(Kern kern, int grid, int block, size_t smem, cudaStream_t st, const GemvParams &p,
                       int stages) {
    return tpb_launch_pdl(kern, dim3((unsigned)grid), dim3((unsigned)block), smem, st, p, stages);
}

// One (M, R) instantiation: fit activations + per-warp rings into the opt-in shared
// memory (as many stages as fit, at most 4; fewer warps next; activations left in
// global memory last) and launch one persistent CTA per SM.
// Diagnostic override of the launch shape: TPB_GEMV_CFG="R,warps,stages" (read at every launch,
// so one process can sweep shapes).
struct GemvOverride { int r = 0, warps = 0, stages = 0; };
static GemvOverride gemv_override() {
    GemvOverride v;
    if (const char *e = getenv("TPB_GEMV_CFG")) sscanf(e, "%d,%d,%d", &v.r, &v.warps, &v.stages);
    return v;
}

// Warps per CTA and stages per warp of the dp4a kernel for one rows-per-stage choice (stage = its bytes); 0 warps:
// the activations leave no room.  Every warp owns a contiguous range of whole rows, so the slowest warp
// carries ceil(rows / warps_total) rows.  Among the counts that fit (with >= 2 stages and the activations in
// shared memory) take the one with the best balance; ties go to more warps.  E.g. 5120 rows on 148 SMs:
// 16 warps -> 2.16 rows per warp (3 vs 2, 72 %), 12 warps -> 2.88 (96 %).
static void dp4a_plan(tpb_handle_t h, size_t act, int64_t rows, int stage, int max_warps, int *warps, int *stages) {
    const size_t limit = (size_t)h->smem_optin - 1024;
    *warps = 0;
    *stages = 0;
    double best_eff = -1.0;
    for (int w = max_warps; w >= max_warps / 2; w--) {
        int s_fit = 0;
        for (int s = 4; s >= 2; s--)
            if (act + (size_t)w * s * stage + (size_t)w * s * 8 + 64 <= limit) {
                s_fit = s;
                break;
            }
        if (s_fit == 0) continue;
        const double per_warp = (double)rows / ((double)h->sm_count * w);
        const double eff = per_warp >= 1.0 ? per_warp / (double)(long long)(per_warp + 0.999999) : per_warp;
        if (eff > best_eff + 0.02) {
            best_eff = eff;
            *warps = w;
            *stages = s_fit;
        }
    }
}

template <int M, int R>
int launch_q8n_cfg(tpb_handle_t h, cudaStream_t st, const GemvParams &p, int max_warps) {
    constexpr int kStage = stage_bytes(R);
    const size_t limit = (size_t)h->smem_optin - 1024;
    const size_t act = (size_t)M * (p.nblk / 2) * kActPairBytes + (size_t)M * p.nblk * 4;
    int warps = 0, stages = 0;
    bool act_smem = true;
    const GemvOverride ov = gemv_override();
    if (ov.r == R && ov.warps > 0 && ov.warps <= max_warps && ov.stages >= 2) {
        const size_t need = act + (size_t)ov.warps * ov.stages * kStage + (size_t)ov.warps * ov.stages * 8 + 64;
        if (need > limit) return tpb_fail(h, TPB_ERR_INVALID_ARG, "TPB_GEMV_CFG does not fit shared memory (%zu bytes)", need);
        int grid = (int)(((long long)p.rows + (long long)ov.warps * R - 1) / ((long long)ov.warps * R));
        if (grid > h->sm_count) grid = h->sm_count;
        auto kern = q8_0_gemv_q8n_kernel<M, R, true>;
        static tpb_per_device_once smem_set_ov;
        TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set_ov));
        TPB_CUDA(h, launch_pdl(kern, grid, ov.warps * 32, need, st, p, ov.stages));
        return TPB_OK;
    }
    dp4a_plan(h, act, p.rows, kStage, max_warps, &warps, &stages);
    if (stages == 0) {
        if (R == 2) return TPB_ERR_STATE;
        act_smem = false;
        warps = max_warps;
        stages = 3;
    }
    const size_t smem = (act_smem ? act : 0) + (size_t)warps * stages * kStage + (size_t)warps * stages * 8 + 64;
    // One persistent CTA per SM as soon as every warp gets at least one row group: leaving SMs
    // idle costs more bandwidth than an uneven last group.
    int grid = (int)(((long long)p.rows + (long long)warps * R - 1) / ((long long)warps * R));
    if (grid < 1) grid = 1;
    if (grid > h->sm_count) grid = h->sm_count;
    // the dynamic size varies per call: each instantiation opts in to the device maximum, once
    if (act_smem) {
        auto kern = q8_0_gemv_q8n_kernel<M, R, true>;
        static tpb_per_device_once smem_set;
        TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
        TPB_CUDA(h, launch_pdl(kern, grid, warps * 32, smem, st, p, stages));
    } else {
        auto kern = q8_0_gemv_q8n_kernel<M, R, false>;
        static tpb_per_device_once smem_set;
        TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
        TPB_CUDA(h, launch_pdl(kern, grid, warps * 32, smem, st, p, stages));
    }
    return TPB_OK;
}

template <int M>
int launch_q8n(tpb_handle_t h, cudaStream_t st, const GemvParams &p) {
    const size_t row_bytes = (size_t)p.nblk * kBlockBytes;
    if (row_bytes % 16 != 0) {
        const int block = 256;
        const int grid = (int)(((long long)p.rows * 32 + block - 1) / block);   // rows < 2^26 (checked at the entry)
        q8_0_gemv_q8n_simple_kernel<M><<<grid, block, 0, st>>>(p);
        TPB_CUDA(h, cudaGetLastError());
        return TPB_OK;
    }
    // Preferred: up to 16 warps with 2 weight rows each (more loads in flight, more latency
    // hiding).  When the activations leave too little shared memory for that, 8 warps with
    // 4 rows each (activations are re-read from shared memory once per R rows).
    if (gemv_override().r != 4) {
        const int rc = launch_q8n_cfg<M, 2>(h, st, p, 16);
        if (rc != TPB_ERR_STATE) return rc;  // TPB_ERR_STATE: did not fit, try the wider grouping
    }
    return launch_q8n_cfg<M, 4>(h, st, p, 8);
}

}  // namespace

int tpb_launch_q8_1_quantize(tpb_handle_t h, cudaStream_t st, const float *x, int64_t n_elems,
                             void *xq) {
    const int nblk = (int)(n_elems / 32);
    float *d = reinterpret_cast<float *>(xq);
    int8_t *qs = reinterpret_cast<int8_t *>(xq) + (size_t)nblk * 4;
    const int block = 256;
    const int grid = (nblk * 32 + block - 1) / block;
    q8_1_quantize_kernel<<<grid, block, 0, st>>>(x, d, qs, nblk);
    TPB_CUDA(h, cudaGetLastError());
    return TPB_OK;
}

int tpb_launch_q8_0_gemv_q8n(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale,
                             int64_t rows, int64_t cols, const void *xq, int ng, int row_off,
                             int n_total) {
    // Two kernels.  The dp4a streaming kernel below costs one dp4a per weight word and activation row: the fastest
    // for one row, 2-10 % slower with each further row, and much slower once its activations crowd the rings out of
    // shared memory.  The kernel that keeps the activations in registers and takes the block sums from mma.sync
    // (qgemv_mma.cu) costs the same whatever M is, but 0-4 us more than the dp4a kernel's single row (more where its
    // per-warp K slices are padded, K = 4096: 4 block pairs in MMAs built for 6, and where it needs two passes
    // over K).  Measured on ten decode shapes, M = 1 .. 8 (us, dp4a / mma): 17408 x 5120  17.6 19.1 21.0 23.8 /
    // 19.2-20.0;  5120 x 17408  21.1 22.9 25.4 / 19.9-21.4 (few long rows: the dp4a kernel's warps get 2.9 rows
    // for two-row stages);  32000 x 4096  22.6 22.7 24.8 26.7 29.9 / 27.1-28.7;  4096 x 14336  11.6 12.7 13.7 15.1
    // 16.9 26.7 / 15.3-16.2;  8192 x 28672  41.0 42.2 69.6 / 49.8-53.0;  28672 x 8192  41.4 42.4 43.6 47.9 /
    // 41.4-44.9.  The rule below follows that table.  TPB_GEMV_KERNEL=dp4a / mma forces one.
    {
        const char *e = getenv("TPB_GEMV_KERNEL");
        const bool force_dp4a = e != nullptr && e[0] == 'd', force_mma = e != nullptr && e[0] == 'm';
        const size_t act_bytes = (size_t)ng * (size_t)(cols / 64) * kActPairBytes + (size_t)ng * (size_t)(cols / 32) * 4;
        int npass = 1, waste_pct = 100;
        const int mma_ks = force_dp4a ? 0 : tpb_q8_0_gemv_mma_fits(h, rows, cols, &npass, &waste_pct);
        bool use_mma = false;
        if (mma_ks != 0 && !force_mma) {
            // the dp4a kernel at its best: fourteen warps with two two-row stages each fit beside the activations
            // (with fewer its time jumps: K = 14336 from the sixth activation row on, K = 28672 from the third)
            int warps = 0, stages = 0;
            dp4a_plan(h, act_bytes, rows, stage_bytes(2), 16, &warps, &stages);
            const bool roomy = warps != 0 && act_bytes + 14 * 2 * (size_t)stage_bytes(2) + 14 * 2 * 8 + 64 <=
                                                 (size_t)h->smem_optin - 1024;
            // share of its row slots that hold a row: rows come to a warp two at a time
            double slots = 1.0;
            if (roomy) {
                const double per_warp = (double)rows / ((double)h->sm_count * warps * 2);
                slots = per_warp >= 1.0 ? per_warp / (double)(long long)(per_warp + 0.999999) : 1.0;
            }
            const double mbytes = (double)rows * (double)(cols / 32) * kBlockBytes * 1e-6;
            const bool padded = waste_pct >= 140;
            const bool uneven = slots < 0.8 && mbytes >= 50.0;   // below that the fixed costs decide, not the balance
            if (!roomy) use_mma = true;
            else if (ng == 1) use_mma = mma_ks >= 2 && uneven;
            else if (uneven) use_mma = true;
            else if (ng == 2) use_mma = mbytes >= 200.0 && npass == 1;
            else if (ng == 3) use_mma = mbytes >= (padded ? 150.0 : 80.0);
            else if (ng == 4) use_mma = mbytes >= (padded ? 150.0 : 60.0);
            else use_mma = true;
        }
        if (mma_ks != 0 && (force_mma || use_mma))
            return tpb_launch_q8_0_gemv_mma(h, st, y, w, scale, rows, cols, xq, ng, row_off, n_total);
    }
    GemvParams p;
    const int nblk = (int)(cols / 32);
    p.y = y;
    p.w = reinterpret_cast<const uint8_t *>(w);
    // xq: f32 d[n_total * nblk], then int8 qs[n_total * cols]  (the reference's layout)
    p.xd = reinterpret_cast<const float *>(xq) + (size_t)row_off * nblk;
    p.xq = reinterpret_cast<const int8_t *>(xq) + (size_t)n_total * nblk * 4 + (size_t)row_off * cols;
    p.scale = scale;
    p.rows = (int)rows;
    p.cols = (int)cols;
    p.nblk = nblk;
    p.status = h->d_status;
    switch (ng) {
        case 1: return launch_q8n<1>(h, st, p);
        case 2: return launch_q8n<2>(h, st, p);
        case 3: return launch_q8n<3>(h, st, p);
        case 4: return launch_q8n<4>(h, st, p);
        case 5: return launch_q8n<5>(h, st, p);
        case 6: return launch_q8n<6>(h, st, p);
        case 7: return launch_q8n<7>(h, st, p);
        case 8: return launch_q8n<8>(h, st, p);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "q8_0_gemv_q8n: ng out of range");
}

int tpb_launch_q8_0_gemv_f32(tpb_handle_t h, cudaStream_t st, float *y, const float *x,
                             const void *w, float scale, int64_t rows, int64_t cols) {
    const size_t smem = (size_t)cols * 4;
    if (smem > (size_t)h->smem_optin)
        return tpb_fail(h, TPB_ERR_INVALID_ARG, "q8_0_gemv_f32: cols too large for shared memory");
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, q8_0_gemv_f32_kernel, h->smem_optin, smem_set));
    int grid = (int)((rows + 7) / 8);
    if (grid > h->sm_count * 4) grid = h->sm_count * 4;
    q8_0_gemv_f32_kernel<<<grid, 256, smem, st>>>(y, x, reinterpret_cast<const uint8_t *>(w), scale,
                                                  (int)rows, (int)cols);
    TPB_CUDA(h, cudaGetLastError());
    return TPB_OK;
}

// ---- allocation-free decode linear --------------------------------------------------
//
// Some hosts cannot let a plugin allocate: an engine that has handed the whole
// device to its own arena and accounts for every byte against a VRAM budget, or a
// decode loop that must not meet the implicit device synchronisation of
// cudaMalloc/cudaFree.  For them the quantised-activation scratch of the GEMV
// lives in this fixed array instead of a caller- or library-allocated buffer.
// Every GPU that loads the library carries the array until the process exits.
// All calls share it and it keeps the previous call's contents: two calls that
// overlap on the GPU (different streams, no ordering between them) race.
static __device__ __align__(256) unsigned char g_static_q8_scratch[TPB_STATIC_GEMV_SCRATCH_BYTES];

namespace {
// Device address of the array per device ordinal.  The array's name in host code
// is only a handle for the runtime, not a device pointer: the address has to be
// asked for, with the owning device current.
// Handles on different devices, or on different host threads, may get here at the same time:
// the table is atomic, and two racing look-ups store the same address.  tpb_create admits
// ordinals below TPB_MAX_DEVICES only, so the index never aliases.
std::atomic<void *> g_static_q8_ptr[TPB_MAX_DEVICES];

int static_scratch_setup(tpb_handle_t h, void **out) {
    void *ptr = g_static_q8_ptr[h->device].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        tpb_device_guard guard(h->device);
        TPB_CUDA(h, guard.err);
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_q8_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return tpb_fail(h, TPB_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s",
                            cudaGetErrorString(e));
        g_static_q8_ptr[h->device].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return TPB_OK;
}
}  // namespace

extern "C" int tpb_q8_0_gemv_static(tpb_handle_t h, tpb_stream_t stream, float *y, const float *x,
                                    int m, const void *w, float scale, int64_t rows, int64_t cols) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y && x && w, "q8_0_gemv_static: null pointer");
    TPB_CHECK_ARG(h, m >= 1 && m <= 8, "q8_0_gemv_static: m must be 1..8 (got %d)", m);
    TPB_CHECK_ARG(h, rows >= 0 && rows < (1ll << 26) && cols > 0 && cols % 32 == 0,
                  "q8_0_gemv_static: cols must be a multiple of 32 and rows below 2^26");
    TPB_CHECK_ARG(h, (int64_t)m * cols <= (int64_t)TPB_STATIC_GEMV_MAX_ELEMS,
                  "q8_0_gemv_static: m * cols = %lld exceeds the fixed scratch of %d elements",
                  (long long)((int64_t)m * cols), TPB_STATIC_GEMV_MAX_ELEMS);
    TPB_CHECK_ARG(h, tpb_aligned16(w) && tpb_aligned16(x), "q8_0_gemv_static: w and x must be 16-byte aligned");
    if (rows == 0) return TPB_OK;
    void *scratch = nullptr;
    int rc = static_scratch_setup(h, &scratch);
    if (rc != TPB_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // same two kernels as tpb_q8_1_quantize + tpb_q8_0_gemv_q8n, scratch in the fixed array
    rc = tpb_launch_q8_1_quantize(h, st, x, (int64_t)m * cols, scratch);
    if (rc != TPB_OK) return rc;
    return tpb_launch_q8_0_gemv_q8n(h, st, y, w, scale, rows, cols, scratch, m, 0, m);
}
