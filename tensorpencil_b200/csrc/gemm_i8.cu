// ConvRot int8 GEMM with fused dequant epilogue for sm_100a.
//
//   y[i][j] = (float(sum_k q[i][k] * w[j][k]) * act_scale[i]) * w_scale[j]
//
// Both operands are K-major (q is [m][k], w is [n][k]) so neither is transposed.
// One persistent CTA per SM walks output tiles of 128 x BN:
//   warp 0      : TMA producer -- 128-byte-swizzled tiles of q and w, K block of
//                 128 bytes per pipeline stage, completion on an mbarrier;
//   warp 1      : allocates TMEM and issues tcgen05.mma.kind::i8 (M=128, N=BN,
//                 K=32) from one thread; int32 accumulators live in TMEM, two
//                 buffers so the epilogue of tile t overlaps the main loop of t+1;
//   warps 2..5  : epilogue -- tcgen05.ld the accumulator rows (the load of the
//                 next 32 columns is in flight while the current ones are
//                 processed), apply the two scales, convert, stage the 32-row x
//                 128-byte piece in shared memory in the 128-byte swizzle
//                 pattern and hand it to a TMA store, so global memory sees
//                 whole 128-byte lines; two staging buffers per warp.
// Every wait on an mbarrier is bounded: on expiry the kernel records a status
// word, every role leaves its loop, TMEM is released and the kernel returns.
// No TMA load here uses cluster multicast.
#include <cstdlib>

#include "gemm_common.cuh"

bool tpb_gemm2_wants(tpb_handle_t h, int64_t m, int64_t n);
int tpb_launch_gemm2_group(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype, const int8_t *q,
                           int count, const void *const *w8, const float *const *w_scale, void *const *y);
int tpb_launch_gemm2_silu_pair(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype,
                               const int8_t *q, const void *w_gate, const void *w_up);
int tpb_launch_gemm2(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype,
                     const int8_t *q, const void *w8, bool b_unsigned);
int tpb_launch_gemm_w4(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype,
                        const int8_t *q, const void *w4);

namespace {

using namespace tpb_gemm;

// ---- the kernel ---------------------------------------------------------------

template <int BN, int OUT, int PEERS>
__global__ void __launch_bounds__(kThreads, 1)
convrot_gemm_kernel(const __grid_constant__ CUtensorMap tma_a,
                    const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_y, const GemmParams p,
                    const int b_unsigned) {
    using Cfg = TileCfg<BN>;
    constexpr int S = Cfg::kStages;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // layout: [S x (A tile | B tile)] [epilogue staging] [barriers] [tmem slot] [abort flag]
    const uint32_t stg_base = smem_base + S * Cfg::kStageBytes;
    const uint32_t bars = stg_base + Cfg::kStagingBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * S + 2 + a); };
    uint8_t *tail = smem_gen + S * Cfg::kStageBytes + Cfg::kStagingBytes + 8 * (2 * S + 4);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(tail);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tail + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int m_tiles = (p.m + BM - 1) / BM;
    const int n_tiles = (p.n + BN - 1) / BN;
    const int num_tiles = m_tiles * n_tiles;
    const int k_blocks = p.k / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32((const void *)tmem_slot)),
                     "r"(Cfg::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up above overlaps the previous kernel's tail; global memory only after this
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM;
                const int n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, (1u << 24) | s, true);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar(s), Cfg::kStageBytes);
                    const uint32_t a_dst = smem_base + s * Cfg::kStageBytes;
                    tma_load_2d(a_dst, &tma_a, full_bar(s), kb * BK, m0);
                    tma_load_2d(a_dst + Cfg::kStageBytesA, &tma_b, full_bar(s), kb * BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_i8<BN>(b_unsigned != 0);
            uint32_t it = 0, t_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, t_it++) {
                const int acc = t_it & 1;
                const uint32_t acc_ph = (t_it >> 1) & 1u;
                ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, (2u << 24) | 0x100u | acc);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, (2u << 24) | s);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
                    const uint64_t a_desc = make_kmajor_sw128_desc(a_addr);
                    const uint64_t b_desc = make_kmajor_sw128_desc(a_addr + Cfg::kStageBytesA);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; kk++) {
                        // advancing 32 bytes inside the 128-byte swizzle row = +2 in the
                        // (address >> 4) field of the descriptor
                        tc_mma_i8(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc,
                                  (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));  // stage reusable once these MMAs have read it
                }
                if (ok) tc_commit(tfull_bar(acc));  // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;  // TMEM lane quarter this warp may access
        // two 4 KB staging buffers per warp, each 32 rows x 128 bytes, 1024-byte aligned
        const uint32_t stg = stg_base + (uint32_t)(warp - 2) * 8192u;
        const uint32_t my_row_off = (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);  // 128-byte swizzle: 16-byte piece j of row r sits at j ^ (r & 7)
        uint32_t n_store = 0;                      // stores issued by this warp (selects the staging buffer)
        uint32_t t_it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, t_it++) {
            const int m0 = (tile % m_tiles) * BM;
            const int n0 = (tile / m_tiles) * BN;
            const int acc = t_it & 1;
            const uint32_t acc_ph = (t_it >> 1) & 1u;
            ok = mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, (3u << 24) | acc, true);
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
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);

            epilogue_tile<BN, OUT, PEERS>(t_row, p, &tma_y, stg, my_row_off, sw, n_store, row0, n0, as, corr, lane);
            // all of this warp's TMEM reads are complete: hand the buffer back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        // staging memory must outlive the stores that read it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // A role gave up.  Give copies and MMAs still in flight time to land
        // before shared memory and TMEM are released.
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(Cfg::kTmemCols)
                     : "memory");
    }
}

// ---- host side ------------------------------------------------------------------

template <int BN, int OUT, int PEERS>
int launch_cfg_p(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w8,
               bool b_unsigned) {
    using Cfg = TileCfg<BN>;
    CUtensorMap ma, mb, my;
    int rc = make_kmajor_map(h, &ma, q, p.m, p.k, BM);
    if (rc != TPB_OK) return rc;
    rc = make_kmajor_map(h, &mb, w8, p.n, p.k, BN);
    if (rc != TPB_OK) return rc;
    rc = make_out_map<OUT>(h, &my, p);
    if (rc != TPB_OK) return rc;
    auto kern = convrot_gemm_kernel<BN, OUT, PEERS>;
    static tpb_per_device_once smem_set;   // per instantiation
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, Cfg::kSmemBytes, smem_set));
    const int m_tiles = (p.m + BM - 1) / BM, n_tiles = (p.n + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const int grid = tiles < h->sm_count ? tiles : h->sm_count;
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, st, ma, mb, my, p, b_unsigned ? 1 : 0));
    return TPB_OK;
}

template <int BN, int OUT>
int launch_cfg(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w8,
               bool b_unsigned) {
    if (p.gate != nullptr) return launch_cfg_p<BN, OUT_F32, 3>(h, st, p, q, w8, b_unsigned);
    if (p.mc_y != nullptr) return launch_cfg_p<BN, OUT, 2>(h, st, p, q, w8, b_unsigned);
    return p.n_peers > 0 ? launch_cfg_p<BN, OUT, 1>(h, st, p, q, w8, b_unsigned)
                         : launch_cfg_p<BN, OUT, 0>(h, st, p, q, w8, b_unsigned);
}

template <int OUT>
int launch_out(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w8,
               bool b_unsigned) {
    // Widest tile that still gives every SM work; narrow tiles for small problems.
    const int m_tiles = (p.m + BM - 1) / BM;
    auto tiles = [&](int bn) { return m_tiles * ((p.n + bn - 1) / bn); };
    if (tiles(256) >= h->sm_count) return launch_cfg<256, OUT>(h, st, p, q, w8, b_unsigned);
    if (tiles(128) >= h->sm_count) return launch_cfg<128, OUT>(h, st, p, q, w8, b_unsigned);
    return launch_cfg<64, OUT>(h, st, p, q, w8, b_unsigned);
}

}  // namespace

int tpb_w4_scratch(tpb_handle_t h, int64_t n, int64_t k, int8_t **out) {
    const size_t need = (size_t)n * (size_t)k;
    if (h->w4_scratch_bytes < need)
        return tpb_fail(h, TPB_ERR_STATE,
                        "int4 weight of %lld x %lld needs %zu bytes of expansion scratch, %zu reserved: call "
                        "tpb_convrot_w4_reserve(h, n, k) once, outside the stream-ordered path",
                        (long long)n, (long long)k, need, h->w4_scratch_bytes);
    *out = h->w4_scratch;
    return TPB_OK;
}

int tpb_launch_gemm(tpb_handle_t h, cudaStream_t st, void *y, int y_dtype, int64_t ldy,
                    const int8_t *q, const float *act_scale, const int32_t *act_sum, const void *w,
                    int w_bits, const float *w_scale, int64_t m, int64_t n, int64_t k,
                    void *const *peer_y, int n_peers, void *mc_y, const float *gate) {
    GemmParams p;
    p.mc_y = mc_y;
    p.gate = gate;
    p.ablate = h->opt_gemm_ablate;
    p.n_peers = n_peers;
    for (int i = 0; i < kMaxPeers; i++) p.peer_y[i] = i < n_peers ? peer_y[i] : nullptr;
    p.y = y;
    p.ldy = ldy;
    p.act_scale = act_scale;
    p.w_scale = w_scale;
    p.act_sum = nullptr;
    p.m = (int)m;
    p.n = (int)n;
    p.k = (int)k;
    p.status = h->d_status;
    const void *w8 = w;
    const bool one_cta_only = h->opt_gemm_one_cta;
    if (w_bits == 4 && n_peers == 0 && mc_y == nullptr && gate == nullptr && h->opt_w4_fused &&
        ((m + 127) / 128) * ((n + 255) / 256) >= h->sm_count) {
        // opt-in: the packed weight is unpacked inside the GEMM (one-CTA kernel)
        p.act_sum = act_sum;
        return tpb_launch_gemm_w4(h, st, p, y_dtype, q, w);
    }
    if (w_bits == 4) {
        int8_t *buf = nullptr;
        int rc = tpb_w4_scratch(h, n, k, &buf);
        if (rc != TPB_OK) return rc;
        rc = tpb_launch_w4_expand(h, st, w, n, k, buf);
        if (rc != TPB_OK) return rc;
        w8 = buf;
    }
    // Large problems: two-CTA tiles (256 x 256 per SM pair).  TPB_GEMM_ONE_CTA=1 keeps
    // the one-CTA kernel for comparisons.
    if (!one_cta_only && tpb_gemm2_wants(h, m, n)) return tpb_launch_gemm2(h, st, p, y_dtype, q, w8, false);
    switch (y_dtype) {
        case TPB_F32: return launch_out<OUT_F32>(h, st, p, q, w8, false);
        case TPB_BF16: return launch_out<OUT_BF16>(h, st, p, q, w8, false);
        case TPB_S32: return launch_out<OUT_S32>(h, st, p, q, w8, false);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gemm: unsupported y_dtype %d", y_dtype);
}

// y = silu(gate projection) * (up projection): both weights multiplied in one launch of the two-CTA
// kernel (each CTA of a pair brings in one weight's half of the tile), combined in its epilogue.
int tpb_launch_gemm_silu_pair(tpb_handle_t h, cudaStream_t st, void *y, int y_dtype, int64_t ldy, const int8_t *q,
                              const float *act_scale, const void *w_gate, const float *w_gate_scale, const void *w_up,
                              const float *w_up_scale, int w_bits, int64_t m, int64_t n, int64_t k) {
    GemmParams p;
    p.mc_y = nullptr;
    p.gate = nullptr;
    p.ablate = 0;
    p.n_peers = 0;
    for (int i = 0; i < kMaxPeers; i++) p.peer_y[i] = nullptr;
    p.y = y;
    p.ldy = ldy;
    p.act_scale = act_scale;
    p.w_scale = w_gate_scale;
    p.w_scale2 = w_up_scale;
    p.act_sum = nullptr;
    p.m = (int)m;
    p.n = (int)n;
    p.k = (int)k;
    p.status = h->d_status;
    const void *g8 = w_gate, *u8 = w_up;
    if (w_bits == 4) {
        // both weights widened into the reserved scratch, one after the other
        int8_t *buf = nullptr;
        int rc = tpb_w4_scratch(h, 2 * n, k, &buf);
        if (rc != TPB_OK) return rc;
        rc = tpb_launch_w4_expand(h, st, w_gate, n, k, buf);
        if (rc != TPB_OK) return rc;
        rc = tpb_launch_w4_expand(h, st, w_up, n, k, buf + (size_t)n * (size_t)k);
        if (rc != TPB_OK) return rc;
        g8 = buf;
        u8 = buf + (size_t)n * (size_t)k;
    }
    return tpb_launch_gemm2_silu_pair(h, st, p, y_dtype, q, g8, u8);
}

// Up to four weights of one shape times the same activations in one launch of the two-CTA kernel (the q, k, v and
// gate projections of a DiT block): their tiles follow one another in its persistent loop, so the pipeline fills
// and drains once instead of once per weight.  Small problems, which the one-CTA kernel takes, run one by one.
int tpb_launch_gemm_group(tpb_handle_t h, cudaStream_t st, int count, void *const *y, int y_dtype, int64_t ldy,
                          const int8_t *q, const float *act_scale, const void *const *w, const float *const *w_scale,
                          int w_bits, int64_t m, int64_t n, int64_t k) {
    if (h->opt_gemm_one_cta || !tpb_gemm2_wants(h, m, n)) {
        for (int g = 0; g < count; g++) {
            const int rc = tpb_launch_gemm(h, st, y[g], y_dtype, ldy, q, act_scale, nullptr, w[g], w_bits, w_scale[g], m, n, k,
                                           nullptr, 0, nullptr, nullptr);
            if (rc != TPB_OK) return rc;
        }
        return TPB_OK;
    }
    GemmParams p;
    p.mc_y = nullptr;
    p.gate = nullptr;
    p.ablate = 0;
    p.n_peers = 0;
    for (int i = 0; i < kMaxPeers; i++) p.peer_y[i] = nullptr;
    p.y = y[0];
    p.ldy = ldy;
    p.act_scale = act_scale;
    p.w_scale = w_scale[0];
    p.act_sum = nullptr;
    p.m = (int)m;
    p.n = (int)n;
    p.k = (int)k;
    p.status = h->d_status;
    const void *w8[4] = {nullptr, nullptr, nullptr, nullptr};
    for (int g = 0; g < count; g++) w8[g] = w[g];
    if (w_bits == 4) {
        // every weight widened into the reserved scratch, one after the other
        int8_t *buf = nullptr;
        int rc = tpb_w4_scratch(h, (int64_t)count * n, k, &buf);
        if (rc != TPB_OK) return rc;
        for (int g = 0; g < count; g++) {
            int8_t *dst = buf + (size_t)g * (size_t)n * (size_t)k;
            rc = tpb_launch_w4_expand(h, st, w[g], n, k, dst);
            if (rc != TPB_OK) return rc;
            w8[g] = dst;
        }
    }
    return tpb_launch_gemm2_group(h, st, p, y_dtype, q, count, w8, w_scale, y);
}
