// Decode GEMV for the other GGUF block formats a checkpoint mixes with Q8_0 -- q4_0,
// iq4_nl, q4_k, q5_k (and q6_k further down) -- on the same streaming skeleton as the Q8_0 kernel (qgemv.cu): every
// warp owns a contiguous range of weight rows and streams them, R rows at a time, into a
// private shared-memory ring with 1-D bulk async copies (mbarrier completion, no
// multicast); q8_1 activations (int8 + per-32-block scale) stay in shared memory for the
// kernel's life; dp4a for the integer dots, f32 accumulation, warp butterfly, * scale.
// A second kernel with the same arithmetic behind one CTA-wide ring (kquant_gemv_ring_kernel,
// further down) takes the calls with one or two activation rows whose rows are long or many.
//
// The unit of work of a lane is 64 consecutive elements (two q8_1 activation blocks):
//   q4_0  a pair of 18-byte blocks (f16 d + 16 nibble bytes each; 36 bytes = 9 aligned
//         words, the first block's nibbles need one funnel shift per word); element j of a
//         block is the low nibble of byte j, element j+16 the high nibble; w = d*(n - 8);
//   q4_k  a quarter of a 144-byte super-block (f16 d, f16 dmin, 12 bytes of 6-bit
//         scales/mins, 128 nibble bytes): 32 bytes whose low nibbles are elements 0..31 of
//         the quarter and high nibbles elements 32..63; w = d*sc*n - dmin*m per 32;
//   q5_k  the same with a fifth bit per element from the 32-byte qh field (176 bytes).
// Block layouts: src/core/quants.zig:9-16 (ggml's).  Reference kernels these stand in for:
// src/gpu/cuda/elt.zig:2014-2110 (q4_0), :1831-1925 (q4_k), :1526-1713 (q5_k), dispatched
// from Backend.opGemvQuantQ8N (src/gpu/cuda/backend.zig:1719-1735).
//
// With sumi = sum(n * xq) over a 32-block (exact, dp4a) and S = dx * sum(xq) precomputed
// per activation block, the dequantised dot is
//   q4_0:  d * (dx * sumi - 8 * S)
//   q4_k / q5_k:  (d * sc) * (dx * sumi) - (dmin * m) * S
// which is what the kernels accumulate in f32.
#include <cuda_fp16.h>

#include "qgemv_common.cuh"

using namespace tpb_gemv;

namespace {

enum { FMT_Q4_0 = 1, FMT_Q4_K = 2, FMT_Q5_K = 3, FMT_IQ4_NL = 5 };

// A lane takes U 64-element units per pipeline stage (template parameter: 2, or 3 where that saves iterations
// per row -- K = 5120 is 80 units: two chunks of 64, the second a quarter full, or one chunk of 96).
constexpr int kActPairBytes = 80;   // a unit's 64 activation bytes + 16 pad (bank-conflict-free 16-byte reads)

template <int FMT> struct Fmt;
// bytes of one 64-element unit (a quarter super-block for the k-quants) and of a chunk of one row
template <> struct Fmt<FMT_Q4_0> { static constexpr int kUnitBytes = 36; };
template <> struct Fmt<FMT_IQ4_NL> { static constexpr int kUnitBytes = 36; };
template <> struct Fmt<FMT_Q4_K> { static constexpr int kUnitBytes = 36; };   // 144 / 4
template <> struct Fmt<FMT_Q5_K> { static constexpr int kUnitBytes = 44; };   // 176 / 4

struct KGemvParams {
    float *y;
    const uint8_t *w;
    const float *xd;   // activation block scales [ng][nblk]
    const int8_t *xq;  // activation quants [ng][cols]
    float scale;
    int rows, cols, nblk;  // nblk = cols / 32
    size_t row_bytes;
    uint32_t chunk_pitch;  // ring kernel: bytes between the rows of a stage
    uint32_t *status;
};

// unsigned bytes of a times signed bytes of b
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Four 4-bit indices (one per byte of idx, 0..15) -> the four signed bytes of ggml's
// kvalues_iq4nl table: two byte-permutes over the table halves, merged by the index's bit 3.
__device__ __forceinline__ uint32_t iq4nl_lookup(uint32_t idx) {
    constexpr uint32_t T0 = 0xBFAD9881u;  // -127 -104 -83 -65
    constexpr uint32_t T1 = 0xF6EADDCFu;  // -49 -35 -22 -10
    constexpr uint32_t T2 = 0x26190D01u;  // 1 13 25 38
    constexpr uint32_t T3 = 0x71594535u;  // 53 69 89 113
    const uint32_t t = idx & 0x07070707u;
    const uint32_t u = t | (t >> 4);                     // byte 0: b0 | b1 << 4, byte 2: b2 | b3 << 4
    const uint32_t sel = __byte_perm(u, 0, 0x4420);      // 16-bit selector b0, b1, b2, b3
    const uint32_t v_lo = __byte_perm(T0, T1, sel);
    const uint32_t v_hi = __byte_perm(T2, T3, sel);
    const uint32_t m = ((idx >> 3) & 0x01010101u) * 0xffu;
    return (v_lo & ~m) | (v_hi & m);
}
__device__ __forceinline__ float f16lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))); }
__device__ __forceinline__ float f16hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }

// The 6-bit scales and mins of sub-blocks 2j and 2j+1 (j = 0..3) of a q4_k / q5_k super-block, both pairs at
// once and without a branch; s0, s1, s2 are the three words of the 12-byte scales field.  ggml's
// get_scale_min_k4 read two sub-blocks at a time: bytes 2j, 2j+1 of the field are one 16-bit word, and
//   j < 2:  scale = byte & 63 of word j of s0,              min = byte & 63 of word j of s1
//   j >= 2: scale = (s2 word & 0x0f0f) | (s0 word >> 6 << 4), min = (s2 word >> 4 & 0x0f0f) | (s1 word >> 6 << 4)
// with "word" the 16-bit half number (j & 1) of each 32-bit word.
__device__ __forceinline__ void scale_min_k4_pair(int j, uint32_t s0, uint32_t s1, uint32_t s2, float &sc0, float &mn0,
                                                  float &sc1, float &mn1) {
    const uint32_t sh = (uint32_t)(j & 1) * 16u;
    const uint32_t a = (s0 >> sh) & 0xffffu, b = (s1 >> sh) & 0xffffu, c = (s2 >> sh) & 0xffffu;
    const bool upper = j >= 2;
    const uint32_t s16 = upper ? ((c & 0x0f0fu) | ((a & 0xc0c0u) >> 2)) : (a & 0x3f3fu);
    const uint32_t m16 = upper ? (((c >> 4) & 0x0f0fu) | ((b & 0xc0c0u) >> 2)) : (b & 0x3f3fu);
    sc0 = (float)(s16 & 0xffu);
    sc1 = (float)(s16 >> 8);
    mn0 = (float)(m16 & 0xffu);
    mn1 = (float)(m16 >> 8);
}

// The arithmetic of one pipeline stage: rows 0 .. nrow - 1 of `stage` (pitch bytes apart) hold chunk c of their
// weight rows; every lane decodes its U units of each row and adds their dot products with the M activation
// rows into acc.
template <int FMT, int M, int R, int U>
__device__ __forceinline__ void kq_stage_dot(const uint8_t *stage, const int pitch, const int nrow, const int c,
                                             const int n_units, const int lane, const int8_t *s_q, const size_t act_row,
                                             const float *s_d, const float *s_s, const int nblk, float (&acc)[R][M]) {
#pragma unroll
    for (int t = 0; t < U; t++) {
        const int ul = lane + 32 * t;                 // unit within the chunk
        const int unit = c * (32 * U) + ul;
        if (unit >= n_units) continue;
        // Decode this lane's 64 weights of each row: lo[8] = elements 0..31 as bytes (nibble,
        // plus the fifth bit for q5_k), hi[8] = elements 32..63 as bytes times 16 (the high
        // nibbles left where they are: one AND instead of shift + AND; the dot product is
        // then an exact multiple of 16), and the two (scale, offset) pairs.
        uint32_t lo[R][8], hi[R][8];
        float ws0[R], ws1[R], wo0[R], wo1[R];  // acc += ws * (dx * sumi) - wo * S
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (r < nrow) {
                if (FMT == FMT_IQ4_NL) {
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(stage + r * pitch + ul * 36);
                    uint32_t tw[9];
#pragma unroll
                    for (int j = 0; j < 9; j++) tw[j] = src[j];
                    // same 18-byte block pair as q4_0; the nibbles go through the value table and
                    // come out as signed bytes, so there is no offset term
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint32_t na = __funnelshift_r(tw[j], tw[j + 1], 16), nb = tw[5 + j];
                        lo[r][j] = iq4nl_lookup(na & 0x0f0f0f0fu);
                        lo[r][4 + j] = iq4nl_lookup((na >> 4) & 0x0f0f0f0fu);
                        hi[r][j] = iq4nl_lookup(nb & 0x0f0f0f0fu);
                        hi[r][4 + j] = iq4nl_lookup((nb >> 4) & 0x0f0f0f0fu);
                    }
                    ws0[r] = f16lo(tw[0]);
                    ws1[r] = f16hi(tw[4]);
                    wo0[r] = wo1[r] = 0.0f;
                } else if (FMT == FMT_Q4_0) {
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(stage + r * pitch + ul * 36);
                    uint32_t tw[9];
#pragma unroll
                    for (int j = 0; j < 9; j++) tw[j] = src[j];
                    // block A: d = tw[0] low half, nibble bytes 2..17; block B: d = tw[4] high half, bytes 20..35
                    uint32_t na[4], nb[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) na[j] = __funnelshift_r(tw[j], tw[j + 1], 16);
#pragma unroll
                    for (int j = 0; j < 4; j++) nb[j] = tw[5 + j];
                    // a block's elements 0..15 are its low nibbles, 16..31 its high nibbles; the
                    // high-nibble words carry a factor 16 that ws/16 below takes back
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        lo[r][j] = (na[j] & 0x0f0f0f0fu) << 4;
                        lo[r][4 + j] = na[j] & 0xf0f0f0f0u;
                        hi[r][j] = (nb[j] & 0x0f0f0f0fu) << 4;
                        hi[r][4 + j] = nb[j] & 0xf0f0f0f0u;
                    }
                    ws0[r] = f16lo(tw[0]);
                    ws1[r] = f16hi(tw[4]);
                    wo0[r] = 8.0f * ws0[r];
                    wo1[r] = 8.0f * ws1[r];
                    ws0[r] *= 0.0625f;
                    ws1[r] *= 0.0625f;
                } else {
                    constexpr int kSb = FMT == FMT_Q5_K ? 176 : 144;
                    constexpr int kQs = FMT == FMT_Q5_K ? 48 : 16;
                    const int j = lane & 3;  // quarter of the super-block (32 t is a multiple of 4)
                    const uint8_t *sb = stage + r * pitch + (ul >> 2) * kSb;
                    const uint4 hdr = *reinterpret_cast<const uint4 *>(sb);
                    const uint4 q0 = *reinterpret_cast<const uint4 *>(sb + kQs + 32 * j);
                    const uint4 q1 = *reinterpret_cast<const uint4 *>(sb + kQs + 32 * j + 16);
                    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                    for (int w = 0; w < 8; w++) {
                        lo[r][w] = qw[w] & 0x0f0f0f0fu;
                        hi[r][w] = qw[w] & 0xf0f0f0f0u;
                    }
                    if (FMT == FMT_Q5_K) {
                        // fifth bits: 16 for the low elements; 16 * 16 = 256 does not fit a byte for
                        // the (x16) high elements, so those go back to plain values
                        const uint4 h0 = *reinterpret_cast<const uint4 *>(sb + 16);
                        const uint4 h1 = *reinterpret_cast<const uint4 *>(sb + 32);
                        const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                        for (int w = 0; w < 8; w++) {
                            // bits 2j and 2j+1 of every qh byte, moved to bit 4 of the byte
                            const uint32_t t = hw[w] >> (2 * j);
                            lo[r][w] |= (t << 4) & 0x10101010u;
                            hi[r][w] = ((qw[w] >> 4) & 0x0f0f0f0fu) | ((t << 3) & 0x10101010u);
                        }
                    }
                    const float d = f16lo(hdr.x), dmin = f16hi(hdr.x);
                    float sc0, mn0, sc1, mn1;
                    scale_min_k4_pair(j, hdr.y, hdr.z, hdr.w, sc0, mn0, sc1, mn1);
                    ws0[r] = d * sc0;
                    wo0[r] = dmin * mn0;
                    ws1[r] = d * sc1 * (FMT == FMT_Q5_K ? 1.0f : 0.0625f);
                    wo1[r] = dmin * mn1;
                }
            } else {
#pragma unroll
                for (int w = 0; w < 8; w++) lo[r][w] = hi[r][w] = 0;
                ws0[r] = ws1[r] = wo0[r] = wo1[r] = 0.0f;
            }
        }
#pragma unroll
        for (int m = 0; m < M; m++) {
            uint32_t xq[16];
            const int4 *a = reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)unit * kActPairBytes);
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const int4 tt = a[v];
                xq[4 * v] = tt.x; xq[4 * v + 1] = tt.y; xq[4 * v + 2] = tt.z; xq[4 * v + 3] = tt.w;
            }
            const float2 d2 = *reinterpret_cast<const float2 *>(s_d + (size_t)m * nblk + 2 * unit);
            const float2 s2 = *reinterpret_cast<const float2 *>(s_s + (size_t)m * nblk + 2 * unit);
#pragma unroll
            for (int r = 0; r < R; r++) {
                int i0 = 0, i1 = 0;
#pragma unroll
                for (int w = 0; w < 8; w++)
                    i0 = FMT == FMT_IQ4_NL ? __dp4a((int)lo[r][w], (int)xq[w], i0) : dp4a_us(lo[r][w], xq[w], i0);
#pragma unroll
                for (int w = 0; w < 8; w++)
                    i1 = FMT == FMT_IQ4_NL ? __dp4a((int)hi[r][w], (int)xq[8 + w], i1) : dp4a_us(hi[r][w], xq[8 + w], i1);
                float tacc = acc[r][m];
                tacc = fmaf(ws0[r], d2.x * i2f_small(i0), tacc);
                tacc = fmaf(-wo0[r], s2.x, tacc);
                tacc = fmaf(ws1[r], d2.y * i2f_small(i1), tacc);
                tacc = fmaf(-wo1[r], s2.y, tacc);
                acc[r][m] = tacc;
            }
        }
    }
}

template <int FMT, int M, int R, int U>
__global__ void __launch_bounds__(512, 1)
kquant_gemv_q8n_kernel(const KGemvParams p, const int stages) {
    constexpr int kUnitsPerLane = U;
    constexpr int kUnitsPerChunk = 32 * U;
    constexpr int kChunkBytes = kUnitsPerChunk * Fmt<FMT>::kUnitBytes;
    constexpr int kStageBytes = R * kChunkBytes;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_warps = blockDim.x >> 5;
    const int nblk = p.nblk;
    const int cols = p.cols;
    const int n_units = cols / 64;

    // shared: [act q: M x n_units x 80][act d: M x nblk f32][act S = d * sum(q): M x nblk f32][rings][barriers]
    const size_t act_row = (size_t)n_units * kActPairBytes;
    int8_t *s_q = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * act_row);
    float *s_s = s_d + (size_t)M * nblk;
    uint8_t *ring0 = reinterpret_cast<uint8_t *>(s_s + (size_t)M * nblk);
    uint8_t *ring = ring0 + (size_t)warp * stages * kStageBytes;
    const uint32_t bars = smem_u32(ring0 + (size_t)n_warps * stages * kStageBytes) + warp * stages * 8;

    if (lane == 0) {
        for (int s = 0; s < stages; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + 8 * s), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int cpr = (n_units + kUnitsPerChunk - 1) / kUnitsPerChunk;  // chunks per row
    const int gw = blockIdx.x * n_warps + warp;
    const int GW = gridDim.x * n_warps;
    const int my_r0 = (int)((long long)p.rows * gw / GW);
    const int my_r1 = (int)((long long)p.rows * (gw + 1) / GW);
    const int my_rg = (my_r1 - my_r0 + R - 1) / R;
    const int total = my_rg * cpr;

    auto issue = [&](int i) {  // lane 0 only
        const int c = i % cpr;
        const int st = i % stages;
        const int row0 = my_r0 + (i / cpr) * R;
        const int nrow = min(R, my_r1 - row0);
        const int units = min(kUnitsPerChunk, n_units - c * kUnitsPerChunk);
        // whole super-blocks for the k-quants: the unit count is a multiple of 4 (cols % 256 == 0)
        const uint32_t bytes = (uint32_t)units * (uint32_t)Fmt<FMT>::kUnitBytes;
        const uint32_t bar = bars + 8 * st;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (uint32_t)nrow)
                     : "memory");
        const uint32_t dst = smem_u32(ring + (size_t)st * kStageBytes);
        for (int r = 0; r < nrow; r++)
            bulk_g2s(dst + r * kChunkBytes, p.w + (size_t)(row0 + r) * p.row_bytes + (size_t)c * kChunkBytes, bytes, bar);
    };

    if (lane == 0)
        for (int i = 0; i < stages - 1 && i < total; i++) issue(i);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const int4 *gq = reinterpret_cast<const int4 *>(p.xq);
        const int per_row = cols / 16;
        for (int i = threadIdx.x; i < M * per_row; i += blockDim.x) {
            const int m = i / per_row, c16 = i - m * per_row;
            *reinterpret_cast<int4 *>(s_q + (size_t)m * act_row + (size_t)(c16 >> 2) * kActPairBytes + (c16 & 3) * 16) =
                __ldcg(gq + i);
        }
        for (int i = threadIdx.x; i < M * nblk; i += blockDim.x) s_d[i] = __ldcg(p.xd + i);
    }
    __syncthreads();
    // S[m][b] = d[m][b] * sum of the block's 32 quants
    for (int i = threadIdx.x; i < M * nblk; i += blockDim.x) {
        const int m = i / nblk, b = i - m * nblk;
        const int4 *a = reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)(b >> 1) * kActPairBytes + (b & 1) * 32);
        const int4 t0 = a[0], t1 = a[1];
        int s = 0;
        s = __dp4a(t0.x, 0x01010101, s); s = __dp4a(t0.y, 0x01010101, s);
        s = __dp4a(t0.z, 0x01010101, s); s = __dp4a(t0.w, 0x01010101, s);
        s = __dp4a(t1.x, 0x01010101, s); s = __dp4a(t1.y, 0x01010101, s);
        s = __dp4a(t1.z, 0x01010101, s); s = __dp4a(t1.w, 0x01010101, s);
        s_s[i] = s_d[i] * (float)s;
    }
    __syncthreads();

    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = 0.0f;

    bool ok = true;
    for (int i = 0; i < total && ok; i++) {
        if (lane == 0 && i + stages - 1 < total) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(i + stages - 1);
        }
        const int st = i % stages;
        ok = mbar_wait(bars + 8 * st, (uint32_t)(i / stages) & 1u, p.status, (5u << 24) | (uint32_t)st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;

        const int c = i % cpr;
        const int row0 = my_r0 + (i / cpr) * R;
        const int nrow = min(R, my_r1 - row0);
        kq_stage_dot<FMT, M, R, U>(ring + (size_t)st * kStageBytes, kChunkBytes, nrow, c, n_units, lane, s_q, act_row, s_d, s_s,
                                   nblk, acc);
        __syncwarp();

        if (c == cpr - 1) {
#pragma unroll
            for (int r = 0; r < R; r++)
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

// ---- the same arithmetic behind a CTA-wide ring ------------------------------------------------
//
// With half the bytes per element of Q8_0 a warp of the kernel above has little left in flight: its
// private ring holds two stages, so every row pair costs it one full trip to HBM.  Here one producer
// warp streams stages of sixteen rows -- one row per consumer warp -- through a ring that takes all
// of shared memory, several stages ahead of the arithmetic; where a row is one chunk, a stage is one
// contiguous piece of the weight and comes with a single bulk copy.  full[s]: the copy's bytes have
// landed; empty[s]: all sixteen consumer warps are done with the stage.  Same sums in the same order
// as the kernel above with one row per stage.
constexpr int kRingRows = 16;

template <int FMT, int M, int U>
__global__ void __launch_bounds__(32 * (kRingRows + 1), 1)
kquant_gemv_ring_kernel(const KGemvParams p, const int stages) {
    constexpr int kUnitsPerChunk = 32 * U;
    constexpr int kChunkBytes = kUnitsPerChunk * Fmt<FMT>::kUnitBytes;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nblk = p.nblk;
    const int cols = p.cols;
    const int n_units = cols / 64;
    const int pitch = (int)p.chunk_pitch;
    const int stage_bytes = kRingRows * pitch;
    const bool whole_rows = (size_t)pitch == p.row_bytes;

    // shared: [act q: M x n_units x 80][act d: M x nblk f32][act S: M x nblk f32][ring][full barriers][empty barriers]
    const size_t act_row = (size_t)n_units * kActPairBytes;
    int8_t *s_q = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * act_row);
    float *s_s = s_d + (size_t)M * nblk;
    uint8_t *ring = reinterpret_cast<uint8_t *>(s_s + (size_t)M * nblk);
    const uint32_t full = smem_u32(ring + (size_t)stages * stage_bytes);
    const uint32_t empty = full + 8u * (uint32_t)stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full + 8 * s), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty + 8 * s), "r"(kRingRows));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int cpr = (n_units + kUnitsPerChunk - 1) / kUnitsPerChunk;  // chunks per row
    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int n_groups = (r1 - r0 + kRingRows - 1) / kRingRows;
    const int total = n_groups * cpr;

    if (warp == 0) {
        // ---------------- producer: the weights do not depend on the kernel before this one ----------------
        if (lane == 0) {
            for (int i = 0; i < total; i++) {
                const int st = i % stages;
                if (i >= stages) {
                    if (!mbar_wait(empty + 8 * st, (uint32_t)(i / stages - 1) & 1u, p.status, (7u << 24) | (uint32_t)st)) break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                const int c = i % cpr;
                const int row0 = r0 + (i / cpr) * kRingRows;
                const int nrow = min(kRingRows, r1 - row0);
                const int units = min(kUnitsPerChunk, n_units - c * kUnitsPerChunk);
                const uint32_t bytes = (uint32_t)units * (uint32_t)Fmt<FMT>::kUnitBytes;
                const uint32_t bar = full + 8 * st;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (uint32_t)nrow)
                             : "memory");
                const uint32_t dst = smem_u32(ring + (size_t)st * stage_bytes);
                if (whole_rows) {
                    bulk_g2s(dst, p.w + (size_t)row0 * p.row_bytes, bytes * (uint32_t)nrow, bar);
                } else {
                    for (int r = 0; r < nrow; r++)
                        bulk_g2s(dst + r * pitch, p.w + (size_t)(row0 + r) * p.row_bytes + (size_t)c * kChunkBytes, bytes, bar);
                }
            }
        }
        return;
    }

    // ---------------- consumers: warp w takes row w of every stage ----------------
    const int w = warp - 1;
    const int ctid = threadIdx.x - 32;
    constexpr int kConsumerThreads = 32 * kRingRows;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const int4 *gq = reinterpret_cast<const int4 *>(p.xq);
        const int per_row = cols / 16;
        for (int i = ctid; i < M * per_row; i += kConsumerThreads) {
            const int m = i / per_row, c16 = i - m * per_row;
            *reinterpret_cast<int4 *>(s_q + (size_t)m * act_row + (size_t)(c16 >> 2) * kActPairBytes + (c16 & 3) * 16) =
                __ldcg(gq + i);
        }
        for (int i = ctid; i < M * nblk; i += kConsumerThreads) s_d[i] = __ldcg(p.xd + i);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
    // S[m][b] = d[m][b] * sum of the block's 32 quants
    for (int i = ctid; i < M * nblk; i += kConsumerThreads) {
        const int m = i / nblk, b = i - m * nblk;
        const int4 *a = reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)(b >> 1) * kActPairBytes + (b & 1) * 32);
        const int4 t0 = a[0], t1 = a[1];
        int sum = 0;
        sum = __dp4a(t0.x, 0x01010101, sum); sum = __dp4a(t0.y, 0x01010101, sum);
        sum = __dp4a(t0.z, 0x01010101, sum); sum = __dp4a(t0.w, 0x01010101, sum);
        sum = __dp4a(t1.x, 0x01010101, sum); sum = __dp4a(t1.y, 0x01010101, sum);
        sum = __dp4a(t1.z, 0x01010101, sum); sum = __dp4a(t1.w, 0x01010101, sum);
        s_s[i] = s_d[i] * (float)sum;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");

    float acc[1][M];
#pragma unroll
    for (int m = 0; m < M; m++) acc[0][m] = 0.0f;

    bool ok = true;
    for (int i = 0; i < total && ok; i++) {
        const int st = i % stages;
        ok = mbar_wait(full + 8 * st, (uint32_t)(i / stages) & 1u, p.status, (8u << 24) | (uint32_t)st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int c = i % cpr;
        const int row = r0 + (i / cpr) * kRingRows + w;
        const bool valid = row < r1;
        if (valid)
            kq_stage_dot<FMT, M, 1, U>(ring + (size_t)st * stage_bytes + (size_t)w * pitch, pitch, 1, c, n_units, lane, s_q, act_row,
                                       s_d, s_s, nblk, acc);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty + 8 * st) : "memory");
        if (c == cpr - 1) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                float v = acc[0][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && valid) p.y[(size_t)m * p.rows + row] = v * p.scale;
                acc[0][m] = 0.0f;
            }
        }
    }
}

// ---- q6_k -----------------------------------------------------------------------------
//
// 210-byte super-blocks (ql[128] low nibbles, qh[64] two high bits, 16 int8 scales, f16 d;
// w = d * sc * (q - 32)) are only 2-byte aligned and a row of them is in general not a
// multiple of 16 bytes, while a bulk copy needs 16-byte aligned addresses and sizes.  A
// chunk is 16 super-blocks (3360 bytes = 210 x 16), so within a row every chunk starts at
// the same offset `mis` modulo 16: the copy starts `mis` bytes early and is rounded up to
// 16, and the lanes index from stage + mis.  (The rounding can read up to 14 bytes past a
// row -- the next row's, or, after the last row, whatever follows the weights in the same
// allocation; those bytes are never used.)  Fields are fetched as aligned words and funnel-
// shifted by the (even) byte offset.
//
// A lane's unit is 64 elements of one super-block: half n (0/1), sixteen positions
// l = 16 lh .. 16 lh + 15 of that half (lh = 0/1), and the four 32-element strides p --
// y[128n + 32p + l].  Each of the four 16-element runs is one scale group of the super-block and half of
// a q8_1 activation block.  With T = 32 * d_x * (sum of the run's sixteen activation quants), computed once
// per call into shared memory, a run adds (d * sc) * (d_x * sum(q * x_q)) - (d * sc) * T.
constexpr int kQ6Sb = 210;
constexpr int kQ6ChunkSb = 16;
constexpr int kQ6ChunkBytes = kQ6ChunkSb * kQ6Sb;     // 3360 = 210 x 16
constexpr int kQ6RowStage = kQ6ChunkBytes + 16 + 16;  // + alignment slack + words read past the last field

// 8 bytes at byte offset `off` (even) from the 4-byte aligned `base`
__device__ __forceinline__ uint2 ld8_unaligned(const uint8_t *base, int off) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(base + (off & ~3));
    const uint32_t sh = (uint32_t)(off & 3) * 8u;  // 0 or 16
    const uint32_t a = w[0], b = w[1], c = w[2];
    return make_uint2(__funnelshift_r(a, b, sh), __funnelshift_r(b, c, sh));
}
// 16 bytes at byte offset `off` (even) from the 4-byte aligned `base`
__device__ __forceinline__ uint4 ld16_unaligned(const uint8_t *base, int off) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(base + (off & ~3));
    const uint32_t sh = (uint32_t)(off & 3) * 8u;  // 0 or 16
    const uint32_t a = w[0], b = w[1], c = w[2], d = w[3], e = w[4];
    return make_uint4(__funnelshift_r(a, b, sh), __funnelshift_r(b, c, sh), __funnelshift_r(c, d, sh), __funnelshift_r(d, e, sh));
}

// The arithmetic of one q6_k pipeline stage: rows row0 .. row0 + nrow - 1 at `stage` (kQ6RowStage bytes apart, each
// starting its row's misalignment into its slot) hold chunk c; every lane decodes its two units of each row.
template <int M, int R>
__device__ __forceinline__ void q6k_stage_dot(const uint8_t *stage, const int row0, const int nrow, const size_t row_bytes,
                                              const int c, const int n_sb, const int lane, const int8_t *s_q,
                                              const size_t act_row, const float *s_d, const float *s_t, const int nblk,
                                              float (&acc)[R][M]) {
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const int ul = lane + 32 * t;              // 64 lane-units per chunk: 4 per super-block
        const int sb_l = ul >> 2;
        const int sb = c * kQ6ChunkSb + sb_l;
        if (sb >= n_sb) continue;
        const int n = (ul >> 1) & 1, lh = ul & 1;
        // q values of the four runs as unsigned bytes (0..63), four words each, and their scales
        uint32_t qv[R][4][4];
        float wsc[R][4];
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (r < nrow) {
                const uint32_t mis = (uint32_t)(((size_t)(row0 + r) * row_bytes) & 15u);
                const uint8_t *base = stage + r * kQ6RowStage;                               // 16-byte aligned
                const int o = (int)mis + sb_l * kQ6Sb;                                    // super-block offset (even)
                const uint4 la = ld16_unaligned(base, o + 64 * n + 16 * lh);        // low nibbles: run 0, high: run 2
                const uint4 lb = ld16_unaligned(base, o + 64 * n + 32 + 16 * lh);   // low: run 1, high: run 3
                const uint4 hb = ld16_unaligned(base, o + 128 + 32 * n + 16 * lh);  // two high bits of runs 0..3
                const uint32_t a4[4] = {la.x, la.y, la.z, la.w}, b4[4] = {lb.x, lb.y, lb.z, lb.w};
                const uint32_t h4[4] = {hb.x, hb.y, hb.z, hb.w};
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    qv[r][0][w] = (a4[w] & 0x0f0f0f0fu) | ((h4[w] << 4) & 0x30303030u);
                    qv[r][1][w] = (b4[w] & 0x0f0f0f0fu) | ((h4[w] << 2) & 0x30303030u);
                    qv[r][2][w] = ((a4[w] >> 4) & 0x0f0f0f0fu) | (h4[w] & 0x30303030u);
                    qv[r][3][w] = ((b4[w] >> 4) & 0x0f0f0f0fu) | ((h4[w] >> 2) & 0x30303030u);
                }
                // scales 8 n + lh + 0, 2, 4, 6 (one per run) from the eight bytes of this half; d behind them
                const uint2 sc8 = ld8_unaligned(base, o + 192 + 8 * n);
                const uint32_t sce = lh ? __byte_perm(sc8.x, sc8.y, 0x7531) : __byte_perm(sc8.x, sc8.y, 0x6420);
                const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(base + o + 208)));
#pragma unroll
                for (int pp = 0; pp < 4; pp++) wsc[r][pp] = d * (float)(int)(int8_t)(sce >> (8 * pp));
            } else {
#pragma unroll
                for (int pp = 0; pp < 4; pp++) {
#pragma unroll
                    for (int w = 0; w < 4; w++) qv[r][pp][w] = 0;
                    wsc[r][pp] = 0.0f;
                }
            }
        }
        const int u = 4 * sb + 2 * n + lh;     // lane-unit number within the row
#pragma unroll
        for (int m = 0; m < M; m++) {
            const float4 dx4 = *reinterpret_cast<const float4 *>(s_d + (size_t)m * nblk + 8 * sb + 4 * n);
            const float4 t4 = *reinterpret_cast<const float4 *>(s_t + ((size_t)m * 4 * n_sb + u) * 4);
            const float dxs[4] = {dx4.x, dx4.y, dx4.z, dx4.w}, ts[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
            for (int pp = 0; pp < 4; pp++) {
                // activation elements 256 sb + 128 n + 32 pp + 16 lh .. + 15
                const int e = 256 * sb + 128 * n + 32 * pp + 16 * lh;
                const int4 xv = *reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)(e >> 6) * kActPairBytes + (e & 63));
#pragma unroll
                for (int r = 0; r < R; r++) {
                    int sq = dp4a_us(qv[r][pp][0], (uint32_t)xv.x, 0);
                    sq = dp4a_us(qv[r][pp][1], (uint32_t)xv.y, sq);
                    sq = dp4a_us(qv[r][pp][2], (uint32_t)xv.z, sq);
                    sq = dp4a_us(qv[r][pp][3], (uint32_t)xv.w, sq);
                    float tacc = acc[r][m];
                    tacc = fmaf(wsc[r][pp], dxs[pp] * i2f_small(sq), tacc);
                    tacc = fmaf(-wsc[r][pp], ts[pp], tacc);
                    acc[r][m] = tacc;
                }
            }
        }
    }
}

template <int M, int R>
__global__ void __launch_bounds__(512, 1)
q6k_gemv_q8n_kernel(const KGemvParams p, const int stages) {
    constexpr int kStageBytes = R * kQ6RowStage;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_warps = blockDim.x >> 5;
    const int nblk = p.nblk;
    const int cols = p.cols;
    const int n_units = cols / 64;
    const int n_sb = cols / 256;

    const size_t act_row = (size_t)n_units * kActPairBytes;
    // shared: [act q: M x n_units x 80][act d: M x nblk f32][T: M x 4 n_sb lane-units x 4 runs f32][rings][barriers]
    int8_t *s_q = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * act_row);
    float *s_t = s_d + (size_t)M * nblk;
    uint8_t *ring0 = reinterpret_cast<uint8_t *>(s_t + (size_t)M * 16 * n_sb);
    uint8_t *ring = ring0 + (size_t)warp * stages * kStageBytes;
    const uint32_t bars = smem_u32(ring0 + (size_t)n_warps * stages * kStageBytes) + warp * stages * 8;

    if (lane == 0) {
        for (int s = 0; s < stages; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + 8 * s), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int cpr = (n_sb + kQ6ChunkSb - 1) / kQ6ChunkSb;
    const int gw = blockIdx.x * n_warps + warp;
    const int GW = gridDim.x * n_warps;
    const int my_r0 = (int)((long long)p.rows * gw / GW);
    const int my_r1 = (int)((long long)p.rows * (gw + 1) / GW);
    const int my_rg = (my_r1 - my_r0 + R - 1) / R;
    const int total = my_rg * cpr;

    auto issue = [&](int i) {  // lane 0 only
        const int c = i % cpr;
        const int st = i % stages;
        const int row0 = my_r0 + (i / cpr) * R;
        const int nrow = min(R, my_r1 - row0);
        const int sbs = min(kQ6ChunkSb, n_sb - c * kQ6ChunkSb);
        const uint32_t bar = bars + 8 * st;
        uint32_t tx = 0;
        for (int r = 0; r < nrow; r++) {
            const uint32_t mis = (uint32_t)(((size_t)(row0 + r) * p.row_bytes) & 15u);
            tx += (mis + (uint32_t)sbs * kQ6Sb + 15u) & ~15u;
        }
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx) : "memory");
        const uint32_t dst = smem_u32(ring + (size_t)st * kStageBytes);
        for (int r = 0; r < nrow; r++) {
            const size_t goff = (size_t)(row0 + r) * p.row_bytes + (size_t)c * kQ6ChunkBytes;
            const uint32_t mis = (uint32_t)(((size_t)(row0 + r) * p.row_bytes) & 15u);
            const uint32_t bytes = (mis + (uint32_t)sbs * kQ6Sb + 15u) & ~15u;
            bulk_g2s(dst + r * kQ6RowStage, p.w + goff - mis, bytes, bar);
        }
    };

    if (lane == 0)
        for (int i = 0; i < stages - 1 && i < total; i++) issue(i);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const int4 *gq = reinterpret_cast<const int4 *>(p.xq);
        const int per_row = cols / 16;
        for (int i = threadIdx.x; i < M * per_row; i += blockDim.x) {
            const int m = i / per_row, c16 = i - m * per_row;
            *reinterpret_cast<int4 *>(s_q + (size_t)m * act_row + (size_t)(c16 >> 2) * kActPairBytes + (c16 & 3) * 16) =
                __ldcg(gq + i);
        }
        for (int i = threadIdx.x; i < M * nblk; i += blockDim.x) s_d[i] = __ldcg(p.xd + i);
    }
    __syncthreads();
    // T[m][lane-unit u = 4 sb + 2 n + lh][run p] = 32 * d_x * sum of activation quants 256 sb + 128 n + 32 p + 16 lh .. + 15
    for (int i = threadIdx.x; i < M * 16 * n_sb; i += blockDim.x) {
        const int m = i / (16 * n_sb), j = i - m * 16 * n_sb;
        const int u = j >> 2, pp = j & 3;
        const int e = 64 * (u >> 1) * 2 + 32 * pp + 16 * (u & 1);   // 256 sb + 128 n = 128 (u >> 1)
        const int4 x = *reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)(e >> 6) * kActPairBytes + (e & 63));
        int sx = __dp4a(x.x, 0x01010101, 0);
        sx = __dp4a(x.y, 0x01010101, sx);
        sx = __dp4a(x.z, 0x01010101, sx);
        sx = __dp4a(x.w, 0x01010101, sx);
        s_t[i] = 32.0f * (s_d[(size_t)m * nblk + (e >> 5)] * (float)sx);
    }
    __syncthreads();

    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = 0.0f;

    bool ok = true;
    for (int i = 0; i < total && ok; i++) {
        if (lane == 0 && i + stages - 1 < total) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(i + stages - 1);
        }
        const int st = i % stages;
        ok = mbar_wait(bars + 8 * st, (uint32_t)(i / stages) & 1u, p.status, (6u << 24) | (uint32_t)st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;

        const int c = i % cpr;
        const int row0 = my_r0 + (i / cpr) * R;
        const int nrow = min(R, my_r1 - row0);
        q6k_stage_dot<M, R>(ring + (size_t)st * kStageBytes, row0, nrow, p.row_bytes, c, n_sb, lane, s_q, act_row, s_d, s_t, nblk, acc);
        __syncwarp();

        if (c == cpr - 1) {
#pragma unroll
            for (int r = 0; r < R; r++)
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

// q6_k behind the CTA-wide ring (see kquant_gemv_ring_kernel): one producer warp, stages of sixteen rows, one row per
// consumer warp; a row's slot starts 16-byte aligned and the row's chunk sits `mis` bytes into it, as above.
template <int M>
__global__ void __launch_bounds__(32 * (kRingRows + 1), 1)
q6k_gemv_ring_kernel(const KGemvParams p, const int stages) {
    constexpr int kStageBytes = kRingRows * kQ6RowStage;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nblk = p.nblk;
    const int cols = p.cols;
    const int n_units = cols / 64;
    const int n_sb = cols / 256;

    const size_t act_row = (size_t)n_units * kActPairBytes;
    int8_t *s_q = reinterpret_cast<int8_t *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)M * act_row);
    float *s_t = s_d + (size_t)M * nblk;
    uint8_t *ring = reinterpret_cast<uint8_t *>(s_t + (size_t)M * 16 * n_sb);
    const uint32_t full = smem_u32(ring + (size_t)stages * kStageBytes);
    const uint32_t empty = full + 8u * (uint32_t)stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full + 8 * s), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty + 8 * s), "r"(kRingRows));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int cpr = (n_sb + kQ6ChunkSb - 1) / kQ6ChunkSb;
    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int n_groups = (r1 - r0 + kRingRows - 1) / kRingRows;
    const int total = n_groups * cpr;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int i = 0; i < total; i++) {
                const int st = i % stages;
                if (i >= stages) {
                    if (!mbar_wait(empty + 8 * st, (uint32_t)(i / stages - 1) & 1u, p.status, (9u << 24) | (uint32_t)st)) break;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                const int c = i % cpr;
                const int row0 = r0 + (i / cpr) * kRingRows;
                const int nrow = min(kRingRows, r1 - row0);
                const int sbs = min(kQ6ChunkSb, n_sb - c * kQ6ChunkSb);
                const uint32_t bar = full + 8 * st;
                uint32_t tx = 0;
                for (int r = 0; r < nrow; r++) {
                    const uint32_t mis = (uint32_t)(((size_t)(row0 + r) * p.row_bytes) & 15u);
                    tx += (mis + (uint32_t)sbs * kQ6Sb + 15u) & ~15u;
                }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx) : "memory");
                const uint32_t dst = smem_u32(ring + (size_t)st * kStageBytes);
                for (int r = 0; r < nrow; r++) {
                    const size_t goff = (size_t)(row0 + r) * p.row_bytes + (size_t)c * kQ6ChunkBytes;
                    const uint32_t mis = (uint32_t)(((size_t)(row0 + r) * p.row_bytes) & 15u);
                    const uint32_t bytes = (mis + (uint32_t)sbs * kQ6Sb + 15u) & ~15u;
                    bulk_g2s(dst + r * kQ6RowStage, p.w + goff - mis, bytes, bar);
                }
            }
        }
        return;
    }

    // ---------------- consumers: warp w takes row w of every stage ----------------
    const int w = warp - 1;
    const int ctid = threadIdx.x - 32;
    constexpr int kConsumerThreads = 32 * kRingRows;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const int4 *gq = reinterpret_cast<const int4 *>(p.xq);
        const int per_row = cols / 16;
        for (int i = ctid; i < M * per_row; i += kConsumerThreads) {
            const int m = i / per_row, c16 = i - m * per_row;
            *reinterpret_cast<int4 *>(s_q + (size_t)m * act_row + (size_t)(c16 >> 2) * kActPairBytes + (c16 & 3) * 16) =
                __ldcg(gq + i);
        }
        for (int i = ctid; i < M * nblk; i += kConsumerThreads) s_d[i] = __ldcg(p.xd + i);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
    for (int i = ctid; i < M * 16 * n_sb; i += kConsumerThreads) {
        const int m = i / (16 * n_sb), j = i - m * 16 * n_sb;
        const int u = j >> 2, pp = j & 3;
        const int e = 128 * (u >> 1) + 32 * pp + 16 * (u & 1);
        const int4 x = *reinterpret_cast<const int4 *>(s_q + (size_t)m * act_row + (size_t)(e >> 6) * kActPairBytes + (e & 63));
        int sx = __dp4a(x.x, 0x01010101, 0);
        sx = __dp4a(x.y, 0x01010101, sx);
        sx = __dp4a(x.z, 0x01010101, sx);
        sx = __dp4a(x.w, 0x01010101, sx);
        s_t[i] = 32.0f * (s_d[(size_t)m * nblk + (e >> 5)] * (float)sx);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");

    float acc[1][M];
#pragma unroll
    for (int m = 0; m < M; m++) acc[0][m] = 0.0f;

    bool ok = true;
    for (int i = 0; i < total && ok; i++) {
        const int st = i % stages;
        ok = mbar_wait(full + 8 * st, (uint32_t)(i / stages) & 1u, p.status, (10u << 24) | (uint32_t)st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int c = i % cpr;
        const int row = r0 + (i / cpr) * kRingRows + w;
        const bool valid = row < r1;
        if (valid)
            q6k_stage_dot<M, 1>(ring + (size_t)st * kStageBytes + (size_t)w * kQ6RowStage, row, 1, p.row_bytes, c, n_sb, lane, s_q,
                                act_row, s_d, s_t, nblk, acc);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty + 8 * st) : "memory");
        if (c == cpr - 1) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                float v = acc[0][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && valid) p.y[(size_t)m * p.rows + row] = v * p.scale;
                acc[0][m] = 0.0f;
            }
        }
    }
}

// TPB_GEMVK_KERNEL=ring|warp forces one of the two kernels (read at every launch, for measurements).
static int k_kernel_override() {
    const char *e = getenv("TPB_GEMVK_KERNEL");
    if (e == nullptr) return 0;
    return e[0] == 'r' ? 1 : e[0] == 'w' ? 2 : 0;
}

template <int M>
int launch_q6k_ring(tpb_handle_t h, cudaStream_t st, const KGemvParams &p, int stages, size_t act) {
    const size_t smem = act + (size_t)stages * ((size_t)kRingRows * kQ6RowStage + 16) + 64;
    int grid = (int)((p.rows + kRingRows - 1) / kRingRows);
    if (grid > h->sm_count) grid = h->sm_count;
    auto kern = q6k_gemv_ring_kernel<M>;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(grid), dim3(32 * (kRingRows + 1)), smem, st, p, stages));
    return TPB_OK;
}

template <int M>
int launch_q6k_m(tpb_handle_t h, cudaStream_t st, const KGemvParams &p) {
    constexpr int R = 2;
    if constexpr (M <= 2) {
        // the ring kernel for one or two activation rows (see launch_fmt_m), where at least three stages fit
        const int force = k_kernel_override();
        const size_t act_r = (size_t)M * (p.cols / 64) * kActPairBytes + (size_t)M * p.nblk * 4 + (size_t)M * (p.cols / 16) * 4;
        const size_t limit_r = (size_t)h->smem_optin - 1024;
        const int s_r = act_r + 256 < limit_r ? (int)((limit_r - act_r - 256) / ((size_t)kRingRows * kQ6RowStage + 16)) : 0;
        // measured (us, per-warp rings / ring): K = 17408 -> N = 5120 28.9 / 23.5, 32000 x 4096 34.1 / 27.7, but
        // 17408 x 5120 22.2 / 27.8 and 8192 x 8192 14.9 / 15.6 at M = 1; at M = 2 4096 x 14336 19.4 / 15.9
        const bool many_rows = p.rows > 10 * 16 * h->sm_count;
        const bool pick = many_rows || p.cols >= (M == 1 ? 16384 : 8192);
        if (s_r >= 3 && (force == 1 || (force == 0 && pick))) return launch_q6k_ring<M>(h, st, p, s_r > 12 ? 12 : s_r, act_r);
    }
    constexpr int kStage = R * kQ6RowStage;
    const size_t limit = (size_t)h->smem_optin - 1024;
    const size_t act = (size_t)M * (p.cols / 64) * kActPairBytes + (size_t)M * p.nblk * 4 + (size_t)M * (p.cols / 16) * 4;
    int warps = 0, stages = 0;
    double best_eff = -1.0;
    for (int w = 16; w >= 4; w--) {
        int s_fit = 0;
        for (int s = 4; s >= 2; s--)
            if (act + (size_t)w * s * kStage + (size_t)w * s * 8 + 64 <= limit) {
                s_fit = s;
                break;
            }
        if (s_fit == 0) continue;
        const double per_warp = (double)p.rows / ((double)h->sm_count * w);
        const double eff = per_warp >= 1.0 ? per_warp / (double)(long long)(per_warp + 0.999999) : per_warp;
        if (eff > best_eff + 0.02) {
            best_eff = eff;
            warps = w;
            stages = s_fit;
        }
    }
    if (stages == 0)
        return tpb_fail(h, TPB_ERR_INVALID_ARG, "gguf_gemv: %d activation rows of %d columns do not fit shared memory",
                        M, p.cols);
    const size_t smem = act + (size_t)warps * stages * kStage + (size_t)warps * stages * 8 + 64;
    int grid = (int)(((long long)p.rows + (long long)warps * R - 1) / ((long long)warps * R));
    if (grid < 1) grid = 1;
    if (grid > h->sm_count) grid = h->sm_count;
    auto kern = q6k_gemv_q8n_kernel<M, R>;
    static tpb_per_device_once smem_set;   // the size varies per call: opt in to the device maximum, once
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(grid), dim3(warps * 32), smem, st, p, stages));
    return TPB_OK;
}

int launch_q6k(tpb_handle_t h, cudaStream_t st, const KGemvParams &p, int ng) {
    switch (ng) {
        case 1: return launch_q6k_m<1>(h, st, p);
        case 2: return launch_q6k_m<2>(h, st, p);
        case 3: return launch_q6k_m<3>(h, st, p);
        case 4: return launch_q6k_m<4>(h, st, p);
        case 5: return launch_q6k_m<5>(h, st, p);
        case 6: return launch_q6k_m<6>(h, st, p);
        case 7: return launch_q6k_m<7>(h, st, p);
        case 8: return launch_q6k_m<8>(h, st, p);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gguf_gemv: ng out of range");
}

template <int FMT, int M, int U>
int launch_fmt_mu(tpb_handle_t h, cudaStream_t st, const KGemvParams &p) {
    constexpr int R = 2;
    constexpr int kStage = R * 32 * U * Fmt<FMT>::kUnitBytes;
    const size_t limit = (size_t)h->smem_optin - 1024;
    const size_t act = (size_t)M * (p.cols / 64) * kActPairBytes + (size_t)M * p.nblk * 8;
    // Warps per CTA: every warp owns a contiguous range of whole rows; among the counts that
    // fit with >= 2 stages take the one whose ranges divide most evenly (ties: more warps).
    int warps = 0, stages = 0;
    double best_eff = -1.0;
    for (int w = 16; w >= 4; w--) {
        int s_fit = 0;
        for (int s = 4; s >= 2; s--)
            if (act + (size_t)w * s * kStage + (size_t)w * s * 8 + 64 <= limit) {
                s_fit = s;
                break;
            }
        if (s_fit == 0) continue;
        const double per_warp = (double)p.rows / ((double)h->sm_count * w);
        const double eff = per_warp >= 1.0 ? per_warp / (double)(long long)(per_warp + 0.999999) : per_warp;
        if (eff > best_eff + 0.02) {
            best_eff = eff;
            warps = w;
            stages = s_fit;
        }
    }
    if (stages == 0)
        return tpb_fail(h, TPB_ERR_INVALID_ARG, "gguf_gemv: %d activation rows of %d columns do not fit shared memory",
                        M, p.cols);
    const size_t smem = act + (size_t)warps * stages * kStage + (size_t)warps * stages * 8 + 64;
    int grid = (int)(((long long)p.rows + (long long)warps * R - 1) / ((long long)warps * R));
    if (grid < 1) grid = 1;
    if (grid > h->sm_count) grid = h->sm_count;
    auto kern = kquant_gemv_q8n_kernel<FMT, M, R, U>;
    static tpb_per_device_once smem_set;   // the size varies per call: opt in to the device maximum, once
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(grid), dim3(warps * 32), smem, st, p, stages));
    return TPB_OK;
}

// The ring kernel, where its stages fit at least three deep; 0 stages: does not fit.
template <int FMT, int U>
int ring_stages(tpb_handle_t h, const KGemvParams &p, int m, uint32_t *pitch_out) {
    const int n_units = p.cols / 64;
    const int cpr = (n_units + 32 * U - 1) / (32 * U);
    const uint32_t pitch = cpr == 1 ? (uint32_t)p.row_bytes : (uint32_t)(32 * U * Fmt<FMT>::kUnitBytes);
    const size_t limit = (size_t)h->smem_optin - 1024;
    const size_t act = (size_t)m * n_units * kActPairBytes + (size_t)m * p.nblk * 8;
    const size_t stage = (size_t)kRingRows * pitch;
    if (act + 256 >= limit) return 0;
    int stages = (int)((limit - act - 256) / (stage + 16));
    if (stages > 12) stages = 12;
    *pitch_out = pitch;
    return stages >= 3 ? stages : 0;
}

template <int FMT, int M, int U>
int launch_fmt_ring(tpb_handle_t h, cudaStream_t st, KGemvParams p, int stages, uint32_t pitch) {
    p.chunk_pitch = pitch;
    const size_t act = (size_t)M * (p.cols / 64) * kActPairBytes + (size_t)M * p.nblk * 8;
    const size_t smem = act + (size_t)stages * ((size_t)kRingRows * pitch + 16) + 64;
    int grid = (int)((p.rows + kRingRows - 1) / kRingRows);
    if (grid > h->sm_count) grid = h->sm_count;
    auto kern = kquant_gemv_ring_kernel<FMT, M, U>;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, h->smem_optin, smem_set));
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(grid), dim3(32 * (kRingRows + 1)), smem, st, p, stages));
    return TPB_OK;
}


template <int FMT, int M>
int launch_fmt_m(tpb_handle_t h, cudaStream_t st, const KGemvParams &p) {
    // three units per lane where that takes fewer chunks per row than two (K = 5120, M = 1: q4_k 17.0 -> 14.6 us,
    // q4_0 14.6 -> 12.1); with many activation rows the longer unrolled body costs more than it saves
    // (q5_k, M = 8: 38 -> 45 us), so only up to four
    const int n_units = p.cols / 64;
    bool u3 = false;
    if constexpr (M <= 4) u3 = (n_units + 95) / 96 < (n_units + 63) / 64;
    // The ring kernel for one or two activation rows where the per-warp rings serialise: rows of several chunks
    // (K = 17408, M = 1: q4_k 21.5 -> 14.4 us, q4_0 18.2 -> 12.7, q5_k 25.1 -> 18.2) and many rows per warp
    // (32000 x 4096: q4_k 28.9 -> 19.2 us).  With short rows and few of them per warp the two are within 5 %
    // either way, and from four activation rows on the dot products set the time in both.
    if constexpr (M <= 2) {
        const int force = k_kernel_override();
        const int cpr = (n_units + (u3 ? 96 : 64) - 1) / (u3 ? 96 : 64);
        const bool many_rows = p.rows > 10 * 16 * h->sm_count;
        if (force == 1 || (force == 0 && (cpr > 1 || many_rows))) {
            uint32_t pitch = 0;
            if (u3) {
                const int s = ring_stages<FMT, 3>(h, p, M, &pitch);
                if (s) return launch_fmt_ring<FMT, M, 3>(h, st, p, s, pitch);
            } else {
                const int s = ring_stages<FMT, 2>(h, p, M, &pitch);
                if (s) return launch_fmt_ring<FMT, M, 2>(h, st, p, s, pitch);
            }
        }
    }
    if constexpr (M <= 4)
        if (u3) return launch_fmt_mu<FMT, M, 3>(h, st, p);
    return launch_fmt_mu<FMT, M, 2>(h, st, p);
}

template <int FMT>
int launch_fmt(tpb_handle_t h, cudaStream_t st, const KGemvParams &p, int ng) {
    switch (ng) {
        case 1: return launch_fmt_m<FMT, 1>(h, st, p);
        case 2: return launch_fmt_m<FMT, 2>(h, st, p);
        case 3: return launch_fmt_m<FMT, 3>(h, st, p);
        case 4: return launch_fmt_m<FMT, 4>(h, st, p);
        case 5: return launch_fmt_m<FMT, 5>(h, st, p);
        case 6: return launch_fmt_m<FMT, 6>(h, st, p);
        case 7: return launch_fmt_m<FMT, 7>(h, st, p);
        case 8: return launch_fmt_m<FMT, 8>(h, st, p);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gguf_gemv: ng out of range");
}

// Whether ng activation rows of `cols` columns leave room for the smallest set of weight rings (four warps, two
// stages each) of the format's kernel.
bool kq_group_fits(tpb_handle_t h, int fmt, int ng, int64_t cols) {
    const size_t limit = (size_t)h->smem_optin - 1024;
    const size_t n_units = (size_t)(cols / 64), nblk = (size_t)(cols / 32);
    const size_t act = (size_t)ng * n_units * kActPairBytes + (size_t)ng * nblk * (fmt == TPB_GGUF_Q6_K ? 12 : 8);
    size_t stage;
    if (fmt == TPB_GGUF_Q6_K) {
        stage = 2 * (size_t)kQ6RowStage;
    } else {
        const bool u3 = ng <= 4 && (n_units + 95) / 96 < (n_units + 63) / 64;
        stage = 2 * (size_t)32 * (u3 ? 3 : 2) * (fmt == TPB_GGUF_Q5_K ? 44 : 36);
    }
    return act + 4 * 2 * stage + 4 * 2 * 8 + 64 <= limit;
}

}  // namespace

extern "C" {

size_t tpb_gguf_row_bytes(int fmt, int64_t cols) {
    switch (fmt) {
        case TPB_GGUF_Q8_0: return (size_t)(cols / 32) * 34;
        case TPB_GGUF_Q4_0:
        case TPB_GGUF_IQ4_NL: return (size_t)(cols / 32) * 18;
        case TPB_GGUF_Q4_K: return (size_t)(cols / 256) * 144;
        case TPB_GGUF_Q5_K: return (size_t)(cols / 256) * 176;
        case TPB_GGUF_Q6_K: return (size_t)(cols / 256) * 210;
    }
    return 0;
}

int tpb_gguf_gemv_q8n(tpb_handle_t h, tpb_stream_t stream, int fmt, float *y, const void *w, float scale,
                      int64_t rows, int64_t cols, const void *xq, int ng, int row_off, int n_total) {
    if (!h) return TPB_ERR_INVALID_ARG;
    if (fmt == TPB_GGUF_Q8_0)
        return tpb_q8_0_gemv_q8n(h, stream, y, w, scale, rows, cols, xq, ng, row_off, n_total);
    TPB_CHECK_ARG(h, fmt == TPB_GGUF_Q4_0 || fmt == TPB_GGUF_Q4_K || fmt == TPB_GGUF_Q5_K || fmt == TPB_GGUF_Q6_K ||
                         fmt == TPB_GGUF_IQ4_NL,
                  "gguf_gemv: unsupported format %d (q8_0, q4_0, q4_k, q5_k, q6_k, iq4_nl)", fmt);
    TPB_CHECK_ARG(h, y && w && xq, "gguf_gemv: null pointer");
    TPB_CHECK_ARG(h, rows >= 0 && rows < (1ll << 31) && cols > 0 && cols % 256 == 0 && cols < (1ll << 24),
                  "gguf_gemv: cols must be a multiple of 256 (cols=%lld)", (long long)cols);
    TPB_CHECK_ARG(h, ng >= 1 && ng <= 8 && row_off >= 0 && row_off + ng <= n_total,
                  "gguf_gemv: need 1 <= ng <= 8 and row_off + ng <= n_total");
    TPB_CHECK_ARG(h, tpb_aligned16(w) && tpb_aligned16(xq), "gguf_gemv: w and xq must be 16-byte aligned");
    if (rows == 0) return TPB_OK;
    if (ng > 1 && !kq_group_fits(h, fmt, ng, cols)) {
        // the group's activations would leave no room for the weight rings (eight rows of 17408 columns are
        // 209 KB): two launches with half the activation rows each -- a row's result does not depend on its group
        const int first = ng / 2;
        const int rc = tpb_gguf_gemv_q8n(h, stream, fmt, y, w, scale, rows, cols, xq, first, row_off, n_total);
        if (rc != TPB_OK) return rc;
        return tpb_gguf_gemv_q8n(h, stream, fmt, y + (size_t)first * (size_t)rows, w, scale, rows, cols, xq, ng - first,
                                 row_off + first, n_total);
    }
    KGemvParams p;
    const int nblk = (int)(cols / 32);
    p.y = y;
    p.w = reinterpret_cast<const uint8_t *>(w);
    p.xd = reinterpret_cast<const float *>(xq) + (size_t)row_off * nblk;
    p.xq = reinterpret_cast<const int8_t *>(xq) + (size_t)n_total * nblk * 4 + (size_t)row_off * cols;
    p.scale = scale;
    p.rows = (int)rows;
    p.cols = (int)cols;
    p.nblk = nblk;
    p.row_bytes = tpb_gguf_row_bytes(fmt, cols);
    p.status = h->d_status;
    cudaStream_t st = (cudaStream_t)stream;
    switch (fmt) {
        case TPB_GGUF_Q4_0: return launch_fmt<FMT_Q4_0>(h, st, p, ng);
        case TPB_GGUF_Q4_K: return launch_fmt<FMT_Q4_K>(h, st, p, ng);
        case TPB_GGUF_Q6_K: return launch_q6k(h, st, p, ng);
        case TPB_GGUF_IQ4_NL: return launch_fmt<FMT_IQ4_NL>(h, st, p, ng);
        default: return launch_fmt<FMT_Q5_K>(h, st, p, ng);
    }
}

}  // extern "C"
