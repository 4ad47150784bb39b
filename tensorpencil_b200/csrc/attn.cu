// Attention of the DiT block for sm_100a: per-head RMS norm of q and k + interleaved RoPE
// (one elementwise pass that also lays the operands out per head in bf16), then a
// flash-style softmax(q k^T * scale) v kernel on tcgen05 (kind::f16, bf16 operands, f32
// accumulators in TMEM).  Non-causal, no mask, grouped-query heads, head_dim 128: the shape
// of the Krea 2 transformer (src/models/dit_cuda.zig:479-489; CPU definitions
// src/ops/attention.zig:46-150, src/ops/rope.zig:68-90, src/ops/norm.zig:12-23).
//
// Kernel layout.  One CTA = TWO 128-row query tiles (A, B) of one head; it walks the kv sequence
// in tiles of 128.  Warp 0 loads tiles with TMA (Q once; K and V^T double-buffered), warp 1 issues
// the MMAs, warps 2-17 are the softmax (tile A / B x column half x row quarter).  Per tile x:
//   S_x  = Q_x K_j^T      M 128 x N 128 x K 128 (head_dim), both operands K-major from shared memory
//   P_x  = exp2(S_x * c - m), running reference point m and sum l per row (online softmax)
//   O_x += P_x V_j        M 128 x N 128 (head_dim) x K 128 (kv); V comes pre-transposed
//          ([head][d][kv], kv contiguous) so that it is K-major too
//   TMEM (512 columns): S_A +0, S_B +128, O_A +256, O_B +384.  P_x (bf16, two per 32-bit column)
//   is written over the first 64 columns of S_x with tcgen05.st and is the A operand of the second
//   product straight from tensor memory: no shared-memory round trip, no proxy fence.
// MMAs of one thread execute in issue order, which is what frees the buffers: S_x(j+1) is issued
// after P_x(j) V(j), so it overwrites S_x / P_x only after that product has read them, and its
// commit (s_full) also says that O_x holds the products up to tile j.  While the tensor pipe works
// for one query tile the other tile's softmax runs.  Every wait is bounded.
#include <cuda_bf16.h>

#include <climits>
#include <cstdint>
#include <type_traits>

#include "gemm_common.cuh"

using namespace tpb_gemm;

namespace {

constexpr int kHd = 128;          // head_dim
constexpr int kTile = 128;        // query rows per CTA and kv rows per step
constexpr int kAtomBytes = 16384; // [128 rows][64 bf16] in the 128-byte swizzle layout
constexpr int kAttnTmemCols = 512;  // S_A, S_B, O_A, O_B: 4 x 128 columns

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f2(uint64_t a, uint64_t b, uint64_t c) {   // two f32 FMAs in one instruction
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// kind::f16 instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, M 128, N 128.
__device__ __forceinline__ uint32_t make_idesc_bf16() {
    uint32_t d = 0;
    d |= 1u << 4;   // D: f32
    d |= 1u << 7;   // A: bf16
    d |= 1u << 10;  // B: bf16
    d |= (uint32_t)(128 >> 3) << 17;
    d |= (uint32_t)(128 >> 4) << 24;
    return d;
}

struct AttnParams {
    void *out;            // [seq_q][heads * 128], bf16 or f32
    int out_f32;
    int seq_q, seq_kv, heads, kv_heads;
    float scale_log2;     // scale * log2(e)
    uint32_t *status;
};

// ---- the attention kernel -------------------------------------------------------------------
constexpr int kAttnThreads = 576;                     // 2 + 16 warps
constexpr int kOffQ = 0;                               // Q_A, Q_B: 2 atoms each
constexpr int kOffK = 4 * kAtomBytes;                  // K stages 0, 1
constexpr int kOffV = kOffK + 4 * kAtomBytes;         // V^T stages 0, 1
constexpr int kOffBar = kOffV + 4 * kAtomBytes;
constexpr int kOffXch = kOffBar + 256;               // row-maximum exchange: 2 x 2 x 128 x 2 floats
constexpr int kAttnSmem = kOffXch + 4096 + 1024;

__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld_dep16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

__global__ void __launch_bounds__(kAttnThreads, 1)
flash_attn_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_vt, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem_base + kOffBar;
    const uint32_t q_full = bars;
    auto k_full = [&](int s) { return bars + 8u * (1 + s); };
    auto v_full = [&](int s) { return bars + 8u * (3 + s); };
    auto k_empty = [&](int s) { return bars + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bars + 8u * (7 + s); };
    auto s_full = [&](int x) { return bars + 8u * (9 + x); };     // x: query tile A = 0, B = 1
    auto p_full = [&](int x) { return bars + 8u * (11 + x); };
    const uint32_t o_done = bars + 8u * 13;
    auto p_half = [&](int x) { return bars + 8u * (14 + x); };    // the first 32 columns of both halves of P_x
    uint8_t *gen = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + kOffBar + 128);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + kOffBar + 136);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * 2 * kTile;
    const int head = blockIdx.y;
    const int hk = head / (p.heads / p.kv_heads);
    const int n_tiles = (p.seq_kv + kTile - 1) / kTile;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(k_full(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1);
            mbar_init(p_full(s), 8);
            mbar_init(p_half(s), 8);
        }
        mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32((const void *)tmem_slot)),
                     "r"(kAttnTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, 4 * kAtomBytes);
#pragma unroll
            for (int a = 0; a < 4; a++)
                tma_load_2d(smem_base + kOffQ + a * kAtomBytes, &tma_q, q_full, (a & 1) * 64,
                            head * p.seq_q + q0 + (a >> 1) * kTile);
            bool ok = true;
            for (int j = 0; ok && j < n_tiles; j++) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                ok = mbar_wait(k_empty(st), ph ^ 1u, abort_flag, p.status, (12u << 24) | 0x10u | st, true);
                if (!ok) break;
                mbar_arrive_expect_tx(k_full(st), 2 * kAtomBytes);
                const uint32_t kd = smem_base + kOffK + st * 2 * kAtomBytes;
                tma_load_2d(kd, &tma_k, k_full(st), 0, hk * p.seq_kv + j * kTile);
                tma_load_2d(kd + kAtomBytes, &tma_k, k_full(st), 64, hk * p.seq_kv + j * kTile);
                ok = mbar_wait(v_empty(st), ph ^ 1u, abort_flag, p.status, (12u << 24) | 0x20u | st, true);
                if (!ok) break;
                mbar_arrive_expect_tx(v_full(st), 2 * kAtomBytes);
                const uint32_t vd = smem_base + kOffV + st * 2 * kAtomBytes;
                tma_load_2d(vd, &tma_vt, v_full(st), j * kTile, hk * kHd);
                tma_load_2d(vd + kAtomBytes, &tma_vt, v_full(st), j * kTile + 64, hk * kHd);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16();
            // S_x = Q_x K_t^T: K dimension = head_dim = 2 atoms x 4 steps of 16 elements (32 bytes)
            auto issue_qk = [&](int x, int t) {
                const uint32_t ka = smem_base + kOffK + (t & 1) * 2 * kAtomBytes;
                const uint32_t qa = smem_base + kOffQ + x * 2 * kAtomBytes;
#pragma unroll
                for (int a = 0; a < 2; a++) {
                    const uint64_t qd = make_kmajor_sw128_desc(qa + a * kAtomBytes);
                    const uint64_t kd = make_kmajor_sw128_desc(ka + a * kAtomBytes);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
                        tc_mma_bf16(tmem_base + (uint32_t)(x * 128), qd + 2u * kk, kd + 2u * kk, idesc, (a | kk) ? 1u : 0u);
                }
                tc_commit(s_full(x));
            };
            // O_x += P_x V_t: P from tensor memory (8 columns = 16 bf16 per step), V^T from shared memory.  The
            // softmax hands P over in two parts -- kv columns 0..31 and 64..95 (the first chunk of each of a row's
            // two threads), then the rest -- so the product starts while the second chunk is still being computed.
            auto issue_pv = [&](int x, int t, int part) {
                const uint32_t va = smem_base + kOffV + (t & 1) * 2 * kAtomBytes;
#pragma unroll
                for (int a = 0; a < 2; a++) {
                    const uint64_t vd = make_kmajor_sw128_desc(va + a * kAtomBytes);
#pragma unroll
                    for (int k2 = 0; k2 < 2; k2++) {
                        const int kk = 2 * part + k2;
                        tc_mma_bf16_ts(tmem_base + 256u + (uint32_t)(x * 128), tmem_base + (uint32_t)(x * 128 + 8 * (4 * a + kk)),
                                       vd + 2u * kk, idesc, (t > 0 || part > 0 || a > 0 || k2 > 0) ? 1u : 0u);
                    }
                }
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, p.status, (13u << 24) | 1u);
            if (ok) ok = mbar_wait(k_full(0), 0, abort_flag, p.status, (13u << 24) | 2u);
            if (ok) {
                tc_fence_after();
                issue_qk(0, 0);
                issue_qk(1, 0);
                tc_commit(k_empty(0));
            }
            for (int j = 0; ok && j < n_tiles; j++) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)j & 1u;
                const bool more = j + 1 < n_tiles;
                ok = mbar_wait(v_full(st), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, (13u << 24) | 3u);
                if (!ok) break;
                ok = mbar_wait(p_half(0), ph, abort_flag, p.status, (13u << 24) | 4u);
                if (!ok) break;
                tc_fence_after();
                issue_pv(0, j, 0);
                ok = mbar_wait(p_full(0), ph, abort_flag, p.status, (13u << 24) | 7u);
                if (!ok) break;
                tc_fence_after();
                issue_pv(0, j, 1);
                if (more) {
                    ok = mbar_wait(k_full(st ^ 1), (uint32_t)((j + 1) >> 1) & 1u, abort_flag, p.status, (13u << 24) | 5u);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(0, j + 1);
                }
                ok = mbar_wait(p_half(1), ph, abort_flag, p.status, (13u << 24) | 6u);
                if (!ok) break;
                tc_fence_after();
                issue_pv(1, j, 0);
                ok = mbar_wait(p_full(1), ph, abort_flag, p.status, (13u << 24) | 8u);
                if (!ok) break;
                tc_fence_after();
                issue_pv(1, j, 1);
                tc_commit(v_empty(st));
                if (more) {
                    issue_qk(1, j + 1);
                    tc_commit(k_empty(st ^ 1));
                }
            }
            if (ok) tc_commit(o_done);
        }
    } else {
        // ---------------- softmax + output: two threads per query row of tile x ----------------
        // A thread owns 64 of the row's 128 kv columns (half hf), so each SM sub-partition runs four
        // softmax warps (tile A / B x half 0 / 1) and has other warps to issue from while one waits on a
        // dependent instruction.  The two threads of a row share the row maximum through shared memory
        // (one 64-thread named barrier per tile); their partial sums are added once, at the end.
        const int idx = (warp - 2) >> 2;                   // 0..3
        const int x = idx >> 1, hf = idx & 1;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                 // row within the tile = TMEM lane
        const uint32_t t_lane = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + t_lane + (uint32_t)(x * 128 + hf * 64);        // this half of S_x
        const uint32_t t_p = tmem_base + t_lane + (uint32_t)(x * 128 + hf * 32);        // this half of P_x (over S_x)
        const uint32_t t_o = tmem_base + t_lane + 256u + (uint32_t)(x * 128 + hf * 64); // this half of O_x
        float *xch = reinterpret_cast<float *>(gen + kOffXch);                         // [2 parity][2 x][128 rows][2 hf]
        const int bar_id = 1 + x * 4 + quarter;
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        auto do_tile = [&](auto masked_tag, const int j) -> bool {
            constexpr bool MASKED = decltype(masked_tag)::value;
            const bool good = mbar_wait(s_full(x), (uint32_t)j & 1u, abort_flag, p.status, (14u << 24) | 1u, true);
            if (!__all_sync(0xffffffffu, good)) return false;
            tc_fence_after();
            const int kv_left = p.seq_kv - j * kTile - hf * 64;     // this half's columns >= kv_left are past the end
            uint32_t v0[32], v1[32];
            tc_ld_32x32(t_s, v0);
            tc_ld_32x32(t_s + 32u, v1);
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            tc_wait_ld_dep(v0);
            tc_wait_ld_dep(v1);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                if (!MASKED || i < kv_left) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v0[i]));
                if (!MASKED || 32 + i < kv_left) m4[(i + 2) & 3] = fmaxf(m4[(i + 2) & 3], __uint_as_float(v1[i]));
            }
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            // Row maximum over both halves.  The barrier also orders the other thread's loads of S
            // before this thread's stores of P over the same columns.
            float *slot = xch + (((j & 1) * 2 + x) * kTile + r) * 2;
            slot[hf] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
            mx = fmaxf(mx, slot[hf ^ 1]);
            // lazy reference point: moves only when the maximum grew by more than 2^kLazy
            constexpr float kLazy = 8.0f;
            const float m_cand = mx * p.scale_log2;
            const float m_new = (m_cand > m_run + kLazy) ? m_cand : m_run;
            const float alpha = ex2(m_run - m_new);
            // O_x holds the products up to tile j - 1 (s_full of tile j was committed after them)
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    uint32_t o[16];
                    tc_ld_32x16(t_o + (uint32_t)(c * 16), o);
                    tc_wait_ld_dep16(o);
#pragma unroll
                    for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tc_st_32x16(t_o + (uint32_t)(c * 16), o);
                }
            }
            // P = exp2(S c - m) as bf16 pairs
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint64_t c2 = pack_f2(p.scale_log2, p.scale_log2), nm2 = pack_f2(-m_new, -m_new);
            auto exp_chunk = [&](const uint32_t (&cur)[32], const int c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    float a0, a1;
                    unpack_f2(fma_f2(pack_f2(__uint_as_float(cur[2 * i]), __uint_as_float(cur[2 * i + 1])), c2, nm2), a0, a1);
                    float e0 = ex2(a0), e1 = ex2(a1);
                    if (MASKED) {
                        if (c * 32 + 2 * i >= kv_left) e0 = 0.0f;
                        if (c * 32 + 2 * i + 1 >= kv_left) e1 = 0.0f;
                    }
                    sum4[(2 * i) & 3] += e0;
                    sum4[(2 * i + 1) & 3] += e1;
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
                    pk[i] = *reinterpret_cast<const uint32_t *>(&b2);
                }
                tc_st_32x16(t_p + (uint32_t)(c * 16), pk);
            };
            exp_chunk(v0, 0);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_half(x));
            exp_chunk(v1, 1);
            l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            m_run = m_new;
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(x));
            return true;
        };
        for (int j = 0; ok && j < n_tiles; j++)
            ok = (p.seq_kv - j * kTile < kTile) ? do_tile(std::true_type{}, j) : do_tile(std::false_type{}, j);
        if (ok) {
            ok = mbar_wait(o_done, 0, abort_flag, p.status, (14u << 24) | 3u, true);
            ok = __all_sync(0xffffffffu, ok);
        }
        // An aborted warp never reaches the named barrier below; its partner then waits in it.  The
        // partner shares every mbarrier wait with it (same tile, same barriers), so both abort together.
        if (ok) {
            tc_fence_after();
            // the row's sum = this half's + the other half's (both relative to the same reference point)
            float *slot = xch + ((n_tiles & 1) * 2 + x) * kTile * 2 + r * 2;
            slot[hf] = l_run;
            asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
            const float inv_l = 1.0f / (l_run + slot[hf ^ 1]);
            const int q = q0 + x * kTile + r;
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tc_ld_32x32(t_o + (uint32_t)(c * 32), v);
                tc_wait_ld_dep(v);
                if (q < p.seq_q) {
                    const size_t off = (size_t)q * p.heads * kHd + (size_t)head * kHd + hf * 64 + c * 32;
                    if (p.out_f32) {
                        float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.out) + off);
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            dst[i] = make_float4(__uint_as_float(v[4 * i]) * inv_l, __uint_as_float(v[4 * i + 1]) * inv_l,
                                                 __uint_as_float(v[4 * i + 2]) * inv_l, __uint_as_float(v[4 * i + 3]) * inv_l);
                    } else {
                        uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(p.out) + off);
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * e]) * inv_l,
                                                                                __uint_as_float(v[8 * i + 2 * e + 1]) * inv_l);
                                w[e] = *reinterpret_cast<const uint32_t *>(&b2);
                            }
                            dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAttnTmemCols)
                     : "memory");
    }
}

// ---- per-head RMS norm + RoPE + per-head bf16 layout ---------------------------------------
//
// Eight values of a row (f32 or bf16) as floats; the row pointer is 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load8(const T *src, float (&v)[8]) {
    if (sizeof(T) == 4) {
        const float4 a = __ldcg(reinterpret_cast<const float4 *>(src));
        const float4 b = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 t = __ldcg(reinterpret_cast<const uint4 *>(src));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}
__device__ __forceinline__ uint32_t bf16_pair(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&b);
}

// q [seq][heads*128] and k [seq][kv_heads*128] in one launch: a half-warp per (token, head) of q or
// of k, a lane holds 8 consecutive elements (four rotation pairs).
//   out [heads][seq][128] bf16 = rope(x * inv_rms(x) * w)
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const T *__restrict__ q, const T *__restrict__ k, const float *__restrict__ qw,
                    const float *__restrict__ kw, const float *__restrict__ cosv, const float *__restrict__ sinv,
                    float eps, int seq, int heads, int kv_heads, __nv_bfloat16 *__restrict__ qb,
                    __nv_bfloat16 *__restrict__ kb) {
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();
    const int slots = heads + kv_heads;
    const long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const int l = threadIdx.x & 15;
    // a whole half-warp leaves together: the shuffles below stay inside it
    const bool live = unit < (long long)seq * slots;
    const int p = live ? (int)(unit / slots) : 0;
    const int sl = live ? (int)(unit - (long long)p * slots) : 0;
    const bool is_q = sl < heads;
    const int h = is_q ? sl : sl - heads;
    const int nh = is_q ? heads : kv_heads;
    const T *src = (is_q ? q : k) + ((size_t)p * nh + h) * kHd + 8 * l;
    float v[8];
    load8(src, v);
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss += v[i] * v[i];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!live) return;
    const float inv = __frsqrt_rn(ss * (1.0f / kHd) + eps);
    const float *w = (is_q ? qw : kw) + 8 * l;
    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w)), w1 = __ldg(reinterpret_cast<const float4 *>(w) + 1);
    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    // rotation pairs 4l .. 4l+3 of this position's table
    const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cosv + (size_t)p * (kHd / 2)) + l);
    const float4 s4 = __ldg(reinterpret_cast<const float4 *>(sinv + (size_t)p * (kHd / 2)) + l);
    const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float a = v[2 * i] * inv * wv[2 * i], b = v[2 * i + 1] * inv * wv[2 * i + 1];
        o[i] = bf16_pair(a * cs[i] - b * sn[i], a * sn[i] + b * cs[i]);
    }
    __nv_bfloat16 *dst = (is_q ? qb : kb) + ((size_t)h * seq + p) * kHd + 8 * l;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
}

// v [seq][kv_heads*128] -> vt [kv_heads][128][seq_pad] bf16 (kv contiguous; columns seq..seq_pad-1 zero).
// A CTA transposes 64 tokens x 128 dims of one head through shared memory, 16 bytes per thread on
// both sides.  Shared tile: word [d][c] = tokens (2c', 2c'+1) of dim d, stored at column
// c = c' ^ (d >> 3): a half-warp (same token pair, 16 dim groups) then hits 16 different banks, and
// the second half-warp works 16 token pairs further on, in the other 16 banks.
template <typename T>
__global__ void __launch_bounds__(256)
v_transpose_kernel(const T *__restrict__ v, int seq, int seq_pad, int kv_heads, __nv_bfloat16 *__restrict__ vt) {
    __shared__ uint32_t tile[kHd][32];
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();
    const int p0 = blockIdx.x * 64, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane & 15;                                   // dim group: dims 8c .. 8c+7
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int pp = warp * 2 + it + 16 * (lane >> 4);        // token pair within the tile
        float a[8], b[8];
        const int t0 = p0 + 2 * pp;
        if (t0 < seq) load8(v + ((size_t)t0 * kv_heads + h) * kHd + 8 * c, a);
        else {
#pragma unroll
            for (int i = 0; i < 8; i++) a[i] = 0.0f;
        }
        if (t0 + 1 < seq) load8(v + ((size_t)(t0 + 1) * kv_heads + h) * kHd + 8 * c, b);
        else {
#pragma unroll
            for (int i = 0; i < 8; i++) b[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) tile[8 * c + i][pp ^ c] = bf16_pair(a[i], b[i]);
    }
    __syncthreads();
    const int s = threadIdx.x & 7;                              // 8 tokens = 4 words = 16 bytes of a row
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = (threadIdx.x >> 3) + 32 * i;
        const int cd = (d >> 3) & 15;
        // logical words 4s .. 4s+3 sit in the aligned group (4s ^ (cd & 12)), permuted by cd & 3
        const uint4 w = *reinterpret_cast<const uint4 *>(&tile[d][(4 * s) ^ (cd & 12)]);
        const uint32_t g[4] = {w.x, w.y, w.z, w.w};
        const int x = cd & 3;
        const int t0 = p0 + 8 * s;
        if (t0 < seq_pad)
            *reinterpret_cast<uint4 *>(vt + ((size_t)h * kHd + d) * seq_pad + t0) =
                make_uint4(g[0 ^ x], g[1 ^ x], g[2 ^ x], g[3 ^ x]);
    }
}

// 2-D bf16 tensor [rows][cols] (cols contiguous), box = 64 columns x 128 rows, 128-byte swizzle,
// out-of-range elements read as zero.
int make_bf16_map(tpb_handle_t h, CUtensorMap *map, const void *base, int64_t rows, int64_t cols, int64_t ld) {
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, 128u};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(h->encode_tiled)(
        map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), gdim, gstride, box, estride,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tpb_fail(h, TPB_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed (%d)", (int)r);
    return TPB_OK;
}

}  // namespace

extern "C" {

size_t tpb_attn_vt_elems(int64_t seq_kv, int kv_heads) {
    const int64_t seq_pad = (seq_kv + 7) / 8 * 8;
    return (size_t)kv_heads * kHd * (size_t)seq_pad;
}

int tpb_attn_prepare(tpb_handle_t h, tpb_stream_t stream, const void *q, const void *k, const void *v, int in_dtype,
                     const float *q_norm, const float *k_norm, float eps, const float *cosv, const float *sinv,
                     int64_t seq, int heads, int kv_heads, int head_dim, void *qb, void *kb, void *vt) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, q && k && v && q_norm && k_norm && cosv && sinv && qb && kb && vt, "attn_prepare: null pointer");
    TPB_CHECK_ARG(h, head_dim == kHd, "attn_prepare: head_dim must be 128 (got %d)", head_dim);
    TPB_CHECK_ARG(h, in_dtype == TPB_F32 || in_dtype == TPB_BF16, "attn_prepare: inputs must be f32 or bf16");
    TPB_CHECK_ARG(h, seq > 0 && seq < (1 << 24) && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && heads <= 65535 &&
                         (int64_t)(heads + kv_heads) * seq < INT32_MAX,
                  "attn_prepare: bad seq / heads / kv_heads");
    TPB_CHECK_ARG(h, tpb_aligned16(q) && tpb_aligned16(k) && tpb_aligned16(v) && tpb_aligned16(q_norm) &&
                         tpb_aligned16(k_norm) && tpb_aligned16(cosv) && tpb_aligned16(sinv) && tpb_aligned16(qb) &&
                         tpb_aligned16(kb) && tpb_aligned16(vt),
                  "attn_prepare: pointers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int seq_pad = (int)((seq + 7) / 8 * 8);
    const dim3 blk(256);
    const long long units = (long long)seq * (heads + kv_heads);     // half-warps
    const dim3 gqk((unsigned)((units + 15) / 16));
    const dim3 gv((unsigned)((seq_pad + 63) / 64), (unsigned)kv_heads);
    cudaError_t e;
    if (in_dtype == TPB_F32) {
        e = tpb_launch_pdl(qk_norm_rope_kernel<float>, gqk, blk, 0, st, (const float *)q, (const float *)k, q_norm, k_norm,
                           cosv, sinv, eps, (int)seq, heads, kv_heads, (__nv_bfloat16 *)qb, (__nv_bfloat16 *)kb);
        if (e == cudaSuccess) e = tpb_launch_pdl(v_transpose_kernel<float>, gv, blk, 0, st, (const float *)v, (int)seq, seq_pad, kv_heads, (__nv_bfloat16 *)vt);
    } else {
        e = tpb_launch_pdl(qk_norm_rope_kernel<__nv_bfloat16>, gqk, blk, 0, st, (const __nv_bfloat16 *)q,
                           (const __nv_bfloat16 *)k, q_norm, k_norm, cosv, sinv, eps, (int)seq, heads, kv_heads,
                           (__nv_bfloat16 *)qb, (__nv_bfloat16 *)kb);
        if (e == cudaSuccess) e = tpb_launch_pdl(v_transpose_kernel<__nv_bfloat16>, gv, blk, 0, st, (const __nv_bfloat16 *)v, (int)seq, seq_pad, kv_heads, (__nv_bfloat16 *)vt);
    }
    TPB_CUDA(h, e);
    return TPB_OK;
}

int tpb_attention(tpb_handle_t h, tpb_stream_t stream, void *out, int out_dtype, const void *qb, const void *kb,
                  const void *vt, int64_t seq_q, int64_t seq_kv, int heads, int kv_heads, int head_dim, float scale) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, out && qb && kb && vt, "attention: null pointer");
    TPB_CHECK_ARG(h, head_dim == kHd, "attention: head_dim must be 128 (got %d)", head_dim);
    TPB_CHECK_ARG(h, out_dtype == TPB_F32 || out_dtype == TPB_BF16, "attention: output must be f32 or bf16");
    TPB_CHECK_ARG(h, seq_q > 0 && seq_kv > 0 && seq_q < (1 << 24) && seq_kv < (1 << 24) && heads > 0 && kv_heads > 0 &&
                         heads % kv_heads == 0 && heads <= 65535,
                  "attention: bad seq / heads / kv_heads");
    // row coordinates of the tensor maps are 32-bit: (head, token) pairs must stay below 2^31, with a
    // tile of slack for the last query tile
    TPB_CHECK_ARG(h, (int64_t)heads * seq_q + 2 * kTile < INT32_MAX && (int64_t)kv_heads * seq_kv + kTile < INT32_MAX,
                  "attention: heads * seq exceeds the 32-bit row range");
    TPB_CHECK_ARG(h, tpb_aligned16(out) && tpb_aligned16(qb) && tpb_aligned16(kb) && tpb_aligned16(vt),
                  "attention: pointers must be 16-byte aligned");
    const int64_t seq_pad = (seq_kv + 7) / 8 * 8;
    CUtensorMap mq, mk, mv;
    int rc = make_bf16_map(h, &mq, qb, (int64_t)heads * seq_q, kHd, kHd);
    if (rc != TPB_OK) return rc;
    rc = make_bf16_map(h, &mk, kb, (int64_t)kv_heads * seq_kv, kHd, kHd);
    if (rc != TPB_OK) return rc;
    rc = make_bf16_map(h, &mv, vt, (int64_t)kv_heads * kHd, seq_pad, seq_pad);
    if (rc != TPB_OK) return rc;
    AttnParams p;
    p.out = out;
    p.out_f32 = out_dtype == TPB_F32;
    p.seq_q = (int)seq_q;
    p.seq_kv = (int)seq_kv;
    p.heads = heads;
    p.kv_heads = kv_heads;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = h->d_status;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, flash_attn_kernel, kAttnSmem, smem_set));
    const dim3 grid((unsigned)((seq_q + 2 * kTile - 1) / (2 * kTile)), (unsigned)heads);
    TPB_CUDA(h, tpb_launch_pdl(flash_attn_kernel, grid, dim3(kAttnThreads), (size_t)kAttnSmem, (cudaStream_t)stream, mq, mk, mv, p));
    return TPB_OK;
}

}  // extern "C"
