// ConvRot GEMM with INT4 weights for sm_100a: the packed weight tile is unpacked to
// int8 in shared memory ahead of the same tcgen05 kind::i8 pipe as the int8 kernel.
//
// tcgen05 has no int4 kind, so activations stay one int4-range value per int8 and the
// CTA widens the weight tile (256 rows x 64 packed bytes per K block) itself:
//   warp 0      TMA producer: 128 rows of q (128-byte swizzle) and the packed weight
//               tile (linear), on separate rings; packed loads run kLead K blocks
//               ahead of the q loads so a q tile is only resident for its own MMAs.
//               No load uses multicast.
//   warps 6..9  unpack: 16 packed bytes -> two 16-byte pieces of the swizzled
//               K-major int8 tile the MMA reads.  Nibbles are widened UNSIGNED
//               (n ^ 8 = value + 8: one LOP3 per four values instead of a sign
//               extension); the tensor core runs signed x unsigned and the epilogue
//               subtracts 8 * sum_k q[row][k] (act_sum from the prep kernel), which is
//               the same integer.
//   warp 1      TMEM allocation, all MMAs and commits.
//   warps 2..5  epilogue (shared with the int8 kernels).
// One CTA per tile on purpose: every producer/consumer hand-off here happens once
// per K block, and CTA-local mbarrier arrives are cheap where cluster-scope ones
// (measured in a two-CTA variant of this kernel) cost more than the K block itself.
// Every mbarrier wait is bounded.
//
// Measured at M=4608 N=12288 K=3072 this kernel is slower than expanding the weight
// to int8 in a separate pass and running the two-CTA int8 kernel (the unpack warps
// and the extra shared-memory traffic sit on the critical path), so the library
// only takes it when TPB_W4_FUSED=1 is set.
#include "gemm_common.cuh"

namespace {

using namespace tpb_gemm;

constexpr int kThreadsW4 = 320;                // 10 warps
constexpr int kA = BM * BK;                    // 16 KB  q rows of this CTA
constexpr int kBp = 256 * (BK / 2);            // 16 KB  packed weight tile (256 rows x 64 B)
constexpr int kBu = 256 * BK;                  // 32 KB  unpacked weight tile
// Three rings with different residency: a q tile lives from its TMA to the end of its
// MMAs; a packed half from its TMA (issued kLead K blocks earlier) to the end of its
// unpack; an unpacked half from the unpack to the end of its MMAs.
constexpr int kSA = 3;                         // q-tile ring
constexpr int kSP = 3;                         // packed-weight ring
constexpr int kU = 3;                          // unpacked-weight ring
constexpr int kLead = 2;                       // K blocks the packed loads run ahead of the q loads
constexpr int kStagingW4 = 4 * 2 * 4096;
constexpr int kNumBars = 2 * kSA + 2 * kSP + 2 * kU + 4;
constexpr int kSmemW4 = kSA * kA + kSP * kBp + kU * kBu + kStagingW4 + 1024 + 8 * kNumBars + 64;
constexpr int kTmemColsW4 = 512;


__device__ __forceinline__ void unpack16(const uint4 p, uint4 &lo, uint4 &hi) {
    const uint32_t in[4] = {p.x, p.y, p.z, p.w};
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        // even nibbles -> bytes (n0,n2,n4,n6), odd -> (n1,n3,n5,n7); ^8 makes them value+8
        const uint32_t e = (in[i] & 0x0f0f0f0fu) ^ 0x08080808u;
        const uint32_t o = ((in[i] >> 4) & 0x0f0f0f0fu) ^ 0x08080808u;
        out[2 * i] = __byte_perm(e, o, 0x5140);
        out[2 * i + 1] = __byte_perm(e, o, 0x7362);
    }
    lo = make_uint4(out[0], out[1], out[2], out[3]);
    hi = make_uint4(out[4], out[5], out[6], out[7]);
}

template <int OUT>
__global__ void __launch_bounds__(kThreadsW4, 1)
convrot_gemm_w4_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_bp,
                        const __grid_constant__ CUtensorMap tma_y, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // layout: [q ring][unpacked ring][packed ring][epilogue staging][barriers]
    const uint32_t bu_base = smem_base + kSA * kA;
    const uint32_t bp_base = bu_base + kU * kBu;
    const uint32_t stg_base = bp_base + kSP * kBp;
    const uint32_t bars = stg_base + kStagingW4;
    auto afull = [&](int s) { return bars + 8u * s; };                  // leader: q tiles of both CTAs landed
    auto aempty = [&](int s) { return bars + 8u * (kSA + s); };         // local: MMAs done with q tile
    auto pfull = [&](int s) { return bars + 8u * (2 * kSA + s); };      // local: packed half landed
    auto pempty = [&](int s) { return bars + 8u * (2 * kSA + kSP + s); };  // local: unpack done with packed half
    auto ufull = [&](int u) { return bars + 8u * (2 * kSA + 2 * kSP + u); };       // leader: both halves unpacked
    auto uempty = [&](int u) { return bars + 8u * (2 * kSA + 2 * kSP + kU + u); };  // local: MMAs done with unpacked half
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * kSA + 2 * kSP + 2 * kU + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * kSA + 2 * kSP + 2 * kU + 2 + a); };
    uint8_t *tail = smem_gen + (bars - smem_base) + 8 * kNumBars;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(tail);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tail + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x;     // this CTA walks tiles pair, pair + n_pairs, ...
    const int n_pairs = gridDim.x;
    const int m_tiles = (p.m + BM - 1) / BM;
    const int n_tiles = (p.n + 255) / 256;
    const int num_tiles = m_tiles * n_tiles;
    const int k_blocks = p.k / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSA; s++) {
            mbar_init(afull(s), 1);
            mbar_init(aempty(s), 1);
        }
        for (int s = 0; s < kSP; s++) {
            mbar_init(pfull(s), 1);
            mbar_init(pempty(s), 4);  // four unpack warps
        }
        for (int u = 0; u < kU; u++) {
            mbar_init(ufull(u), 4);   // four unpack warps
            mbar_init(uempty(u), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32((const void *)tmem_slot)),
                     "r"(kTmemColsW4)
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
            const int my_tiles = pair < num_tiles ? (num_tiles - pair + n_pairs - 1) / n_pairs : 0;
            const int total = my_tiles * k_blocks;
            bool ok = true;
            // packed weight half of flat iteration i (tile i / k_blocks, K block i % k_blocks)
            auto load_packed = [&](int i) {
                const int t = i / k_blocks, kb = i - t * k_blocks;
                const int tile = pair + t * n_pairs;
                const int n0 = (tile / m_tiles) * 256;
                const int s = i % kSP;
                if (!mbar_wait(pempty(s), ((i / kSP) & 1u) ^ 1u, abort_flag, p.status, (1u << 24) | 0x40u | s, true))
                    return false;
                mbar_arrive_expect_tx(pfull(s), kBp);
                tma_load_2d(bp_base + s * kBp, &tma_bp, pfull(s), kb * (BK / 2), n0);
                return true;
            };
            for (int i = 0; ok && i < kLead && i < total; i++) ok = load_packed(i);
            for (int i = 0; ok && i < total; i++) {
                if (i + kLead < total) ok = load_packed(i + kLead);
                if (!ok) break;
                const int t = i / k_blocks, kb = i - t * k_blocks;
                const int tile = pair + t * n_pairs;
                const int m0 = (tile % m_tiles) * BM;
                const int s = i % kSA;
                ok = mbar_wait(aempty(s), ((i / kSA) & 1u) ^ 1u, abort_flag, p.status, (1u << 24) | s, true);
                if (!ok) break;
                mbar_arrive_expect_tx(afull(s), kA);
                tma_load_2d(smem_base + s * kA, &tma_a, afull(s), kb * BK, m0);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_i8<256>(true);  // weights widened unsigned
            uint32_t it = 0, t_it = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < num_tiles; tile += n_pairs, t_it++) {
                const int acc = t_it & 1;
                const uint32_t acc_ph = (t_it >> 1) & 1u;
                ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, (2u << 24) | 0x100u | acc);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % kSA, u = it % kU;
                    ok = mbar_wait(afull(s), (it / kSA) & 1u, abort_flag, p.status, (2u << 24) | s) &&
                         mbar_wait(ufull(u), (it / kU) & 1u, abort_flag, p.status, (2u << 24) | 0x40u | u);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a_desc = make_kmajor_sw128_desc(smem_base + s * kA);
                    const uint64_t b_desc = make_kmajor_sw128_desc(bu_base + u * kBu);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; kk++)
                        tc_mma_i8(d_tmem, a_desc + 2u * kk, b_desc + 2u * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(aempty(s));
                    tc_commit(uempty(u));
                }
                if (ok) {
                    tc_commit(tfull_bar(acc));
                }
            }
        }
    } else if (warp >= 6) {
        // ---------------- unpack ----------------
        const int tid = threadIdx.x - 6 * 32;  // 0..127
        uint32_t it = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < num_tiles; tile += n_pairs) {
            for (int kb = 0; kb < k_blocks; kb++, it++) {
                const int s = it % kSP, u = it % kU;
                ok = mbar_wait(pfull(s), (it / kSP) & 1u, abort_flag, p.status, (5u << 24) | s) &&
                     mbar_wait(uempty(u), ((it / kU) & 1u) ^ 1u, abort_flag, p.status, (5u << 24) | 0x40u | u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t src = bp_base + s * kBp;
                const uint32_t dst = bu_base + u * kBu;
                // all eight 16-byte loads first (independent, so their latencies overlap),
                // then widen and store
                uint4 pk[8];
#pragma unroll
                for (int j = 0; j < 8; j++) pk[j] = ld_shared_v4(src + (uint32_t)(j * 128 + tid) * 16u);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int i = j * 128 + tid;       // packed 16-byte chunk: row i/4, chunk i%4
                    const int r = i >> 2, pc = i & 3;
                    uint4 lo, hi;
                    unpack16(pk[j], lo, hi);
                    const uint32_t row = dst + (uint32_t)r * 128u;
                    const uint32_t swz = (uint32_t)(r & 7);
                    st_shared_v4(row + ((((uint32_t)(2 * pc)) ^ swz) << 4), lo.x, lo.y, lo.z, lo.w);
                    st_shared_v4(row + ((((uint32_t)(2 * pc + 1)) ^ swz) << 4), hi.x, hi.y, hi.z, hi.w);
                }
                // generic-proxy writes -> visible to the tensor core's async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(ufull(u));
                    mbar_arrive(pempty(s));
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;
        const uint32_t stg = stg_base + (uint32_t)(warp - 2) * 8192u;
        const uint32_t my_row_off = (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);
        uint32_t n_store = 0, t_it = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < num_tiles; tile += n_pairs, t_it++) {
            const int m0 = (tile % m_tiles) * BM;
            const int n0 = (tile / m_tiles) * 256;
            const int acc = t_it & 1;
            ok = mbar_wait(tfull_bar(acc), (t_it >> 1) & 1u, abort_flag, p.status, (3u << 24) | acc, true);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row0 = m0 + quarter * 32;
            const int row = row0 + lane;
            const bool row_ok = row < p.m;
            float as = 0.0f;
            int corr = 0;
            if (OUT != OUT_S32 && row_ok) as = __ldcg(p.act_scale + row);
            if (row_ok) corr = 8 * __ldcg(p.act_sum + row);
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
            epilogue_tile<256, OUT>(t_row, p, &tma_y, stg, my_row_off, sw, n_store, row0, n0, as, corr, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsW4)
                     : "memory");
    }
}

}  // namespace

// ---- host side ------------------------------------------------------------------

namespace {

// packed weight [n][k/2] bytes, box = 64 bytes x 256 rows, no swizzle, zero fill
int make_packed_map(tpb_handle_t h, CUtensorMap *map, const void *base, int64_t n, int64_t k) {
    const cuuint64_t gdim[2] = {(cuuint64_t)(k / 2), (cuuint64_t)n};
    const cuuint64_t gstride[1] = {(cuuint64_t)(k / 2)};
    const cuuint32_t box[2] = {(cuuint32_t)(BK / 2), 256u};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(h->encode_tiled)(
        map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estride,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return tpb_fail(h, TPB_ERR_CUDA, "cuTensorMapEncodeTiled (packed weight) failed (%d)", (int)r);
    return TPB_OK;
}

template <int OUT>
int launch_w4(tpb_handle_t h, cudaStream_t st, const GemmParams &p, const int8_t *q, const void *w4) {
    CUtensorMap ma, mb, my;
    int rc = make_kmajor_map(h, &ma, q, p.m, p.k, BM);
    if (rc != TPB_OK) return rc;
    rc = make_packed_map(h, &mb, w4, p.n, p.k);
    if (rc != TPB_OK) return rc;
    rc = make_out_map<OUT>(h, &my, p);
    if (rc != TPB_OK) return rc;
    auto kern = convrot_gemm_w4_kernel<OUT>;
    static tpb_per_device_once smem_set;   // per instantiation
    TPB_CUDA(h, tpb_set_max_smem_once(h, kern, kSmemW4, smem_set));
    const int tiles = ((p.m + BM - 1) / BM) * ((p.n + 255) / 256);
    const int grid = tiles < h->sm_count ? tiles : h->sm_count;
    TPB_CUDA(h, tpb_launch_pdl(kern, dim3(grid), dim3(kThreadsW4), kSmemW4, st, ma, mb, my, p));
    return TPB_OK;
}

}  // namespace

// INT4 weights, unpacked inside the GEMM.  p.act_sum must be set.
int tpb_launch_gemm_w4(tpb_handle_t h, cudaStream_t st, const tpb_gemm::GemmParams &p, int y_dtype,
                        const int8_t *q, const void *w4) {
    switch (y_dtype) {
        case TPB_F32: return launch_w4<OUT_F32>(h, st, p, q, w4);
        case TPB_BF16: return launch_w4<OUT_BF16>(h, st, p, q, w4);
        case TPB_S32: return launch_w4<OUT_S32>(h, st, p, q, w4);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "gemm: unsupported y_dtype %d", y_dtype);
}
