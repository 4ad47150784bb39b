// ConvRot int8 GEMM, two-CTA variant for sm_100a: a cluster of two CTAs (two SMs)
// computes one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Why: with one CTA per tile every SM stages a full 256-row weight tile per K
// block (48 KB written by TMA and read back by the tensor core per 512 MMA
// cycles), and shared-memory traffic, not the tensor pipe, sets the pace.  In
// the pair, each CTA stages its own 128 rows of q AND only its half (128 rows)
// of the weight tile; the hardware feeds both tensor cores from the two halves.
// Per SM and K block that is 32 KB instead of 48 KB.
//
// Roles per CTA (same warp layout in both CTAs of the pair):
//   warp 0  TMA producer for this CTA's A rows and B half; completion is counted
//           on the LEADER's (rank 0) "full" barrier.  No load uses multicast.
//   warp 1  TMEM allocation (collective over the pair); in the leader it also
//           issues every MMA and the tcgen05.commit arrivals, one to its own
//           barrier and one to the peer's (plain commits to a cluster address,
//           no multicast qualifier anywhere in this file).
//   warps 2..5  epilogue for this CTA's 128 rows, as in the one-CTA kernel (warps 2..9 in the gated-residual
//           mode at short K: see EW below).
// Every mbarrier wait is bounded; both CTAs always run the same collective
// steps (cluster barriers, TMEM alloc/dealloc) whatever happened in between.
#include "gemm_common.cuh"

namespace {

using namespace tpb_gemm;

constexpr int BN2 = 256;                       // tile width (UMMA N)
constexpr int kStageA = BM * BK;               // 16 KB: this CTA's 128 rows of q
constexpr int kStageB = (BN2 / 2) * BK;        // 16 KB: this CTA's half of the weight tile
constexpr int kStage2 = kStageA + kStageB;
// Epilogue warps per CTA (template parameter EW): four (one per 32-lane quarter of tensor memory, all 256 columns
// each, two 4 KB staging buffers per warp), or eight -- two warps per quarter, 128 columns each, one staging buffer
// per warp -- for the gated-residual mode, whose epilogue reads the residual tile it updates and sets the pace at
// short K (K = 3072: 56 -> 48 us; K = 12288: 134 -> 130 us).  The operand ring is the same either way.
constexpr int stages2(int) { return 6; }
constexpr int staging2(int) { return 4 * 2 * 4096; }   // two 4 KB buffers per warp (four warps) or one each (eight)
constexpr int smem2(int ew) { return stages2(ew) * kStage2 + staging2(ew) + 1024 + 256; }
constexpr int threads2(int ew) { return 64 + 32 * ew; }
constexpr int kTmemCols2 = 2 * BN2;

// Up to four weights of the same shape multiplied with the same activations in one launch (PAIR == 2): the
// tiles of weight g follow those of weight g - 1 in the persistent loop.  Weight 0 is described by the
// kernel's own tma_b / tma_y / p.w_scale, weights 1.. by this block.
struct GemmGroup {
    CUtensorMap b[3];
    CUtensorMap y[3];
    const float *w_scale[3];
    int count;   // weights in all, 1..4
};

// PAIR == 1: the weight tile's two halves come from two different weights (tma_b: the leader's 128 rows,
// tma_b2: the peer's), both for the same 128 output columns, and the epilogue combines the two
// projections into silu(first) * second (epilogue_pair).  PAIR == 2: several weights, see GemmGroup.
template <int OUT, int PEERS, int PAIR, int EW = 4>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads2(EW), 1)
convrot_gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const __grid_constant__ CUtensorMap tma_b2, const __grid_constant__ CUtensorMap tma_y,
                     const GemmParams p, const int b_unsigned, const __grid_constant__ GemmGroup grp) {
    constexpr bool MULTI = PAIR == 2;
    constexpr int S = stages2(EW);
    constexpr int kEpiWarps = EW;
    constexpr int kStaging2 = staging2(EW);
    constexpr int kEpiCols = BN2 * 4 / kEpiWarps;   // columns of a tile one epilogue warp handles
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t stg_base = smem_base + S * kStage2;
    const uint32_t bars = stg_base + kStaging2;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * S + 2 + a); };
    uint8_t *tail = smem_gen + S * kStage2 + kStaging2 + 8 * (2 * S + 4);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(tail);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tail + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;

    const int m_tiles = (p.m + 2 * BM - 1) / (2 * BM);  // 256-row tiles
    constexpr int kTileN = PAIR == 1 ? BN2 / 2 : BN2;   // output columns per tile
    const int n_tiles = (p.n + kTileN - 1) / kTileN;
    const int tiles_per_weight = m_tiles * n_tiles;
    const int num_tiles = MULTI ? tiles_per_weight * grp.count : tiles_per_weight;
    const int k_blocks = p.k / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 2 * kEpiWarps);  // the epilogue warps of both CTAs of the pair
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // collective over the pair: the same warp of both CTAs, same shared offset
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32((const void *)tmem_slot)),
                     "r"(kTmemCols2)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up above overlaps the previous kernel's tail; global memory only after this
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += n_pairs) {
                const int wg = MULTI ? tile / tiles_per_weight : 0;   // which weight
                const int wt = MULTI ? tile - wg * tiles_per_weight : tile;
                const int m0 = (wt % m_tiles) * (2 * BM) + (int)rank * BM;
                const int n0 = PAIR == 1 ? (wt / m_tiles) * kTileN : (wt / m_tiles) * BN2 + (int)rank * (BN2 / 2);
                const CUtensorMap *bmap = (PAIR == 1 && rank == 1) ? &tma_b2 : (MULTI && wg > 0) ? &grp.b[wg - 1] : &tma_b;
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, (1u << 24) | (rank << 8) | s, true);
                    if (!ok) break;
                    const uint32_t lead_full = mapa(full_bar(s), 0);
                    const bool load_a = !(p.ablate & 1), load_b = !(p.ablate & 2);
                    if (rank == 0)
                        mbar_arrive_expect_tx(full_bar(s), 2u * ((load_a ? kStageA : 0) + (load_b ? kStageB : 0)));
                    const uint32_t a_dst = smem_base + s * kStage2;
                    if (load_a) tma_load_2d_pair(a_dst, &tma_a, lead_full, kb * BK, m0);
                    if (load_b) tma_load_2d_pair(a_dst + kStageA, bmap, lead_full, kb * BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = make_idesc2_i8(b_unsigned != 0);
            uint32_t it = 0, t_it = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += n_pairs, t_it++) {
                const int acc = t_it & 1;
                const uint32_t acc_ph = (t_it >> 1) & 1u;
                ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, (2u << 24) | 0x100u | acc);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN2);
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, (2u << 24) | s);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * kStage2;
                    const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
                    const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + kStageA);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; kk++)
                        tc2_mma_i8(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    // the stage is free in BOTH CTAs once these MMAs have read it
                    tc2_commit(empty_bar(s));
                    tc2_commit(mapa(empty_bar(s), 1));
                }
                if (ok) {
                    tc2_commit(tfull_bar(acc));
                    tc2_commit(mapa(tfull_bar(acc), 1));
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, own 128 rows) ----------------
        const int quarter = warp & 3;
        const int chalf = (kEpiWarps == 8) ? (warp - 2) >> 2 : 0;   // which 128 columns of the tile (eight warps)
        const int c_off = chalf * kEpiCols;
        const uint32_t stg = stg_base + (uint32_t)(warp - 2) * (kEpiWarps == 8 ? 4096u : 8192u);
        const uint32_t my_row_off = (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);
        uint32_t n_store = 0;
        uint32_t t_it = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < num_tiles; tile += n_pairs, t_it++) {
            const int wg = MULTI ? tile / tiles_per_weight : 0;
            const int wt = MULTI ? tile - wg * tiles_per_weight : tile;
            const int m0 = (wt % m_tiles) * (2 * BM) + (int)rank * BM;
            const int n0 = (wt / m_tiles) * kTileN;
            const CUtensorMap *ymap = (MULTI && wg > 0) ? &grp.y[wg - 1] : &tma_y;
            const float *w_scale = (MULTI && wg > 0) ? grp.w_scale[wg - 1] : p.w_scale;
            const int acc = t_it & 1;
            const uint32_t acc_ph = (t_it >> 1) & 1u;
            if (PEERS == 3) {
                // gated residual: ask for this warp's 32 rows x 128 columns of the residual stream (a lane's row, four
                // lines) to be brought into L2 while the accumulators are still being produced.  Asking a whole
                // tile earlier was measured slower (m 4608, n 12288, k 3072: 202 us against 180 us).
                const int prow = m0 + quarter * 32 + lane;
                if (prow < p.m) {
                    const float *xp = static_cast<const float *>(p.y) + (size_t)prow * (size_t)p.ldy + n0 + c_off;
#pragma unroll
                    for (int i = 0; i < kEpiCols / 32; i++)
                        if (n0 + c_off + 32 * i < p.n) asm volatile("prefetch.global.L2 [%0];" ::"l"(xp + 32 * i));
                }
            }
            ok = mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, (3u << 24) | (rank << 8) | acc, true);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row0 = m0 + quarter * 32;
            const int row = row0 + lane;
            const bool row_ok = row < p.m;
            float as = 0.0f;
            int corr = 0;
            if (OUT != OUT_S32 && row_ok) as = __ldcg(p.act_scale + row);
            if (p.act_sum != nullptr && row_ok) corr = 8 * __ldcg(p.act_sum + row);
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN2 + c_off);
            if (PAIR == 1) {
                if constexpr (PAIR == 1 && (OUT == OUT_F32 || OUT == OUT_BF16))
                    epilogue_pair<OUT>(t_row, p, &tma_y, stg, my_row_off, sw, n_store, row0, n0, as, lane);
            } else if (!(p.ablate & 4)) {
                epilogue_tile<kEpiCols, OUT, PEERS, EW == 8 && PEERS == 3, EW == 8>(t_row, p, ymap, stg, my_row_off, sw, n_store, row0, n0 + c_off, as, corr, lane, w_scale);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    // ---------------- teardown (identical in both CTAs) ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync();  // nobody frees TMEM or leaves while the peer may still signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols2)
                     : "memory");
    }
}

}  // namespace

// ---- host side ------------------------------------------------------------------

namespace {

const GemmGroup kNoGroup = {};

// Weights w[0 .. count-1] of one shape times the same q, outputs y[0 .. count-1] (same dtype and ldy).
template <int OUT>
int launch_group(tpb_handle_t h, cudaStream_t st, const GemmParams &p0, const int8_t *q, int count, const void *const *w8,
                 const float *const *w_scale, void *const *y) {
    CUtensorMap ma, mb, my;
    GemmGroup grp = {};
    grp.count = count;
    int rc = make_kmajor_map(h, &ma, q, p0.m, p0.k, BM);
    if (rc != TPB_OK) return rc;
    GemmParams p = p0;
    for (int g = 0; g < count; g++) {
        p.y = y[g];
        rc = make_kmajor_map(h, g == 0 ? &mb : &grp.b[g - 1], w8[g], p.n, p.k, BN2 / 2);
        if (rc != TPB_OK) return rc;
        rc = make_out_map<OUT>(h, g == 0 ? &my : &grp.y[g - 1], p);
        if (rc != TPB_OK) return rc;
        if (g > 0) grp.w_scale[g - 1] = w_scale[g];
    }
    p.y = y[0];
    p.w_scale = w_scale[0];
    auto kern = convrot_gemm2_kernel<OUT, 0, 2>;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, smem2(4), smem_set));
    const int m_tiles = (p.m + 2 * BM - 1) / (2 * BM), n_tiles = (p.n + BN2 - 1) / BN2;
    const int tiles = m_tiles * n_tiles * count;
    const int max_pairs = h->sm_count / 2;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(2 * pairs), dim3(threads2(4)), smem2(4), st, ma, mb, mb, my, p, 0, grp));
    return TPB_OK;
}

template <int OUT, int PEERS, int EW = 4>
int launch_pair_p(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w8,
                bool b_unsigned) {
    CUtensorMap ma, mb, my;
    int rc = make_kmajor_map(h, &ma, q, p.m, p.k, BM);            // each CTA loads 128 rows of q
    if (rc != TPB_OK) return rc;
    rc = make_kmajor_map(h, &mb, w8, p.n, p.k, BN2 / 2);          // and 128 rows (half a tile) of w
    if (rc != TPB_OK) return rc;
    rc = make_out_map<OUT>(h, &my, p);
    if (rc != TPB_OK) return rc;
    auto kern = convrot_gemm2_kernel<OUT, PEERS, 0, EW>;
    static tpb_per_device_once smem_set;   // per instantiation
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, smem2(EW), smem_set));
    const int m_tiles = (p.m + 2 * BM - 1) / (2 * BM), n_tiles = (p.n + BN2 - 1) / BN2;
    const int tiles = m_tiles * n_tiles;
    const int max_pairs = h->sm_count / 2;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(2 * pairs), dim3(threads2(EW)), smem2(EW), st, ma, mb, mb, my, p, b_unsigned ? 1 : 0, kNoGroup));
    return TPB_OK;
}

template <int OUT>
int launch_silu_pair(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w_gate,
                     const void *w_up) {
    CUtensorMap ma, mb, mb2, my;
    int rc = make_kmajor_map(h, &ma, q, p.m, p.k, BM);
    if (rc != TPB_OK) return rc;
    rc = make_kmajor_map(h, &mb, w_gate, p.n, p.k, BN2 / 2);
    if (rc != TPB_OK) return rc;
    rc = make_kmajor_map(h, &mb2, w_up, p.n, p.k, BN2 / 2);
    if (rc != TPB_OK) return rc;
    rc = make_out_map<OUT>(h, &my, p);
    if (rc != TPB_OK) return rc;
    auto kern = convrot_gemm2_kernel<OUT, 0, 1>;
    static tpb_per_device_once smem_set;
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, smem2(4), smem_set));
    const int m_tiles = (p.m + 2 * BM - 1) / (2 * BM), n_tiles = (p.n + BN2 / 2 - 1) / (BN2 / 2);
    const int tiles = m_tiles * n_tiles;
    const int max_pairs = h->sm_count / 2;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(2 * pairs), dim3(threads2(4)), smem2(4), st, ma, mb, mb2, my, p, 0, kNoGroup));
    return TPB_OK;
}

template <int OUT>
int launch_pair(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w8,
                bool b_unsigned) {
    if (p.gate != nullptr) return launch_pair_p<OUT_F32, 3, 8>(h, st, p, q, w8, b_unsigned);
    if (p.mc_y != nullptr) return launch_pair_p<OUT, 2>(h, st, p, q, w8, b_unsigned);
    if (p.n_peers > 0) return launch_pair_p<OUT, 1>(h, st, p, q, w8, b_unsigned);
    // (eight epilogue warps in the plain modes: the epilogue alone gets faster -- n = 12288, k = 256: 77 -> 54 us --
    // but a GEMM bound by its main loop does not: k = 3072, n = 12288: 129 -> 134 us)
    return launch_pair_p<OUT, 0>(h, st, p, q, w8, b_unsigned);
}

}  // namespace

// True when the two-CTA kernel should take this problem: enough 256 x 256 tiles to
// occupy every SM pair.
bool tpb_gemm2_wants(tpb_handle_t h, int64_t m, int64_t n) {
    const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256);
    return tiles >= h->sm_count / 2;
}

int tpb_launch_gemm2_silu_pair(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype,
                               const int8_t *q, const void *w_gate, const void *w_up) {
    if (y_dtype == TPB_F32) return launch_silu_pair<OUT_F32>(h, st, p, q, w_gate, w_up);
    if (y_dtype == TPB_BF16) return launch_silu_pair<OUT_BF16>(h, st, p, q, w_gate, w_up);
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gemm_silu_pair: y_dtype must be f32 or bf16");
}

int tpb_launch_gemm2_group(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype, const int8_t *q,
                           int count, const void *const *w8, const float *const *w_scale, void *const *y) {
    if (y_dtype == TPB_F32) return launch_group<OUT_F32>(h, st, p, q, count, w8, w_scale, y);
    if (y_dtype == TPB_BF16) return launch_group<OUT_BF16>(h, st, p, q, count, w8, w_scale, y);
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gemm_group: y_dtype must be f32 or bf16");
}

int tpb_launch_gemm2(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype,
                     const int8_t *q, const void *w8, bool b_unsigned) {
    switch (y_dtype) {
        case TPB_F32: return launch_pair<OUT_F32>(h, st, p, q, w8, b_unsigned);
        case TPB_BF16: return launch_pair<OUT_BF16>(h, st, p, q, w8, b_unsigned);
        case TPB_S32: return launch_pair<OUT_S32>(h, st, p, q, w8, b_unsigned);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gemm: unsupported y_dtype %d", y_dtype);
}
