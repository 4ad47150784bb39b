// Peer-mapped buffers and the cross-GPU barrier used by the GEMM whose epilogue also
// writes its output shard into the other GPUs' copies of y (tpb_convrot_gemm_allgather).
//
// One process per GPU.  A buffer is allocated with cudaMalloc on its owner, exported as
// a CUDA IPC handle (64 opaque bytes the host exchanges through any channel it likes),
// and opened by the peers; NVLink peer access is enabled by the open.  Nothing here has
// a reference counterpart: the reference runs on one GPU (src/gpu/cuda/context.zig:111).
//
// The barrier is a flag exchange: rank r owns flags[r][0..world), rank s announces epoch
// e by storing e into flags[r][s] on every r (release, system scope) and then waits until
// its own row holds e everywhere (acquire, system scope).  Epochs only grow, so no reset
// is needed.  The wait is bounded: after timeout_ms it records TPB_ERR_TIMEOUT in the
// handle's status word and returns, leaving the context usable.
#include "tpb_internal.h"

#include <cstring>

namespace {

constexpr uint32_t kStatusBarrierTimeout = 0xBA000000u;

struct FlagPtrs {
    uint32_t *p[8];
};

__device__ __forceinline__ void st_release_sys(uint32_t *addr, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *addr) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void peer_barrier_kernel(const FlagPtrs flags, const int world, const int rank, const uint32_t epoch,
                                    const unsigned long long timeout_ns, uint32_t *status) {
    const int t = threadIdx.x;
    if (t >= world) return;
    // Everything this GPU wrote before the barrier (earlier kernels in the stream, peer
    // stores included) becomes visible to rank t before it can see the flag.
    __threadfence_system();
    st_release_sys(flags.p[t] + rank, epoch);
    const uint32_t *mine = flags.p[rank] + t;
    const unsigned long long t0 = globaltimer_ns();
    // Iteration cap as a second bound, in case the timer misbehaves: ~1 us per poll.
    const unsigned long long max_polls = timeout_ns / 500ull + 1024ull;
    for (unsigned long long it = 0;; ++it) {
        if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) return;
        __nanosleep(it < 64 ? 100 : 1000);
        if (it >= max_polls || ((it & 15ull) == 15ull && globaltimer_ns() - t0 > timeout_ns)) {
            atomicCAS(status, 0u, kStatusBarrierTimeout | (uint32_t)t);
            return;
        }
    }
}

}  // namespace

int tpb_launch_peer_barrier(tpb_handle_t h, cudaStream_t st, uint32_t *const *flags, int world, int rank,
                            uint32_t epoch, int timeout_ms) {
    FlagPtrs fp;
    for (int i = 0; i < 8; i++) fp.p[i] = i < world ? flags[i] : nullptr;
    peer_barrier_kernel<<<1, 32, 0, st>>>(fp, world, rank, epoch, (unsigned long long)timeout_ms * 1000000ull,
                                          h->d_status);
    TPB_CUDA(h, cudaGetLastError());
    return TPB_OK;
}

extern "C" {

int tpb_peer_alloc(tpb_handle_t h, size_t bytes, void **ptr, void *ipc_handle) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, ptr && ipc_handle && bytes > 0, "peer_alloc: null pointer or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == TPB_PEER_HANDLE_BYTES, "IPC handle size");
    TPB_CUDA(h, cudaSetDevice(h->device));
    void *p = nullptr;
    const cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        return tpb_fail(h, TPB_ERR_OOM, "peer_alloc: out of device memory (%zu bytes)", bytes);
    }
    TPB_CUDA(h, e);
    cudaError_t e2 = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t hd;
    if (e2 == cudaSuccess) e2 = cudaIpcGetMemHandle(&hd, p);
    if (e2 != cudaSuccess) {
        cudaFree(p);
        TPB_CUDA(h, e2);
    }
    memcpy(ipc_handle, &hd, sizeof(hd));
    *ptr = p;
    return TPB_OK;
}

int tpb_peer_open(tpb_handle_t h, const void *ipc_handle, void **ptr) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, ptr && ipc_handle, "peer_open: null pointer");
    TPB_CUDA(h, cudaSetDevice(h->device));
    cudaIpcMemHandle_t hd;
    memcpy(&hd, ipc_handle, sizeof(hd));
    void *p = nullptr;
    TPB_CUDA(h, cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return TPB_OK;
}

int tpb_peer_close(tpb_handle_t h, void *ptr) {
    if (!h) return TPB_ERR_INVALID_ARG;
    if (!ptr) return TPB_OK;
    TPB_CUDA(h, cudaIpcCloseMemHandle(ptr));
    return TPB_OK;
}

int tpb_peer_free(tpb_handle_t h, void *ptr) {
    if (!h) return TPB_ERR_INVALID_ARG;
    if (!ptr) return TPB_OK;
    TPB_CUDA(h, cudaFree(ptr));
    return TPB_OK;
}

int tpb_peer_barrier(tpb_handle_t h, tpb_stream_t stream, uint32_t *const *flags, int world, int rank,
                     uint32_t epoch, int timeout_ms) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, flags && world >= 1 && world <= 8 && rank >= 0 && rank < world,
                  "peer_barrier: need 1 <= world <= 8 and 0 <= rank < world");
    TPB_CHECK_ARG(h, timeout_ms > 0 && timeout_ms <= 60000, "peer_barrier: timeout_ms must be in 1..60000");
    for (int i = 0; i < world; i++)
        TPB_CHECK_ARG(h, flags[i] && (reinterpret_cast<uintptr_t>(flags[i]) & 3u) == 0,
                      "peer_barrier: flags[%d] is null or misaligned", i);
    return tpb_launch_peer_barrier(h, (cudaStream_t)stream, flags, world, rank, epoch, timeout_ms);
}

int tpb_convrot_gemm_allgather(tpb_handle_t h, tpb_stream_t stream, void *const *y_all, int world, int rank,
                               int y_dtype, int64_t ldy, const int8_t *q, const float *act_scale,
                               const int32_t *act_sum, const void *w_shard, int w_bits,
                               const float *w_scale_shard, int64_t m, int64_t n_shard, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y_all && world >= 1 && world <= 8 && rank >= 0 && rank < world,
                  "gemm_allgather: need 1 <= world <= 8 and 0 <= rank < world");
    TPB_CHECK_ARG(h, y_dtype == TPB_F32 || y_dtype == TPB_BF16 || y_dtype == TPB_S32,
                  "gemm_allgather: y_dtype must be f32, bf16 or s32");
    TPB_CHECK_ARG(h, n_shard > 0 && ldy >= n_shard * world, "gemm_allgather: ldy must be >= world * n_shard");
    const size_t esz = y_dtype == TPB_BF16 ? 2 : 4;
    void *peers[7];
    int n_peers = 0;
    for (int r = 0; r < world; r++) {
        TPB_CHECK_ARG(h, y_all[r] && tpb_aligned16(y_all[r]), "gemm_allgather: y_all[%d] is null or misaligned", r);
        if (r != rank) peers[n_peers++] = static_cast<char *>(y_all[r]) + (size_t)rank * (size_t)n_shard * esz;
    }
    void *y_local = static_cast<char *>(y_all[rank]) + (size_t)rank * (size_t)n_shard * esz;
    // The remaining argument checks are those of the plain GEMM on the local shard.
    TPB_CHECK_ARG(h, q && w_shard, "gemm_allgather: null pointer");
    TPB_CHECK_ARG(h, y_dtype == TPB_S32 || (act_scale && w_scale_shard), "gemm_allgather: scales are required");
    TPB_CHECK_ARG(h, w_bits == 8 || w_bits == 4, "gemm_allgather: w_bits must be 8 or 4 (got %d)", w_bits);
    TPB_CHECK_ARG(h, w_bits == 8 || act_sum, "gemm_allgather: act_sum is required when w_bits = 4");
    TPB_CHECK_ARG(h, m >= 0 && k > 0 && k % 256 == 0 && n_shard % 16 == 0,
                  "gemm_allgather: need k %% 256 == 0 and n_shard %% 16 == 0");
    TPB_CHECK_ARG(h, m < (1ll << 31) && n_shard * world < (1ll << 31) && k < (1ll << 31),
                  "gemm_allgather: dims exceed 2^31");
    const int64_t ld_mult = y_dtype == TPB_BF16 ? 8 : 4;
    TPB_CHECK_ARG(h, ldy % ld_mult == 0, "gemm_allgather: ldy must be a multiple of %lld", (long long)ld_mult);
    TPB_CHECK_ARG(h, tpb_aligned16(q) && tpb_aligned16(w_shard) && tpb_aligned16(w_scale_shard),
                  "gemm_allgather: q, w and w_scale must be 16-byte aligned");
    if (m == 0) return TPB_OK;
    return tpb_launch_gemm(h, (cudaStream_t)stream, y_local, y_dtype, ldy, q, act_scale, act_sum, w_shard, w_bits,
                           w_scale_shard, m, n_shard, k, peers, n_peers);
}

int tpb_convrot_gemm_multi(tpb_handle_t h, tpb_stream_t stream, void *y_local, void *const *y_peers, int n_peers,
                           int y_dtype, int64_t ldy, const int8_t *q, const float *act_scale,
                           const int32_t *act_sum, const void *w, int w_bits, const float *w_scale, int64_t m,
                           int64_t n, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, n_peers >= 0 && n_peers <= 7 && (n_peers == 0 || y_peers), "gemm_multi: need 0 <= n_peers <= 7");
    for (int i = 0; i < n_peers; i++)
        TPB_CHECK_ARG(h, y_peers[i] && tpb_aligned16(y_peers[i]), "gemm_multi: y_peers[%d] is null or misaligned", i);
    // every other check is the plain GEMM's
    const int rc = tpb_convrot_gemm(h, nullptr, y_local, y_dtype, ldy, q, act_scale, act_sum, w, w_bits, w_scale, 0, n, k);
    if (rc != TPB_OK) return rc;
    TPB_CHECK_ARG(h, m >= 0 && m < (1ll << 31), "gemm_multi: bad m");
    if (m == 0) return TPB_OK;
    return tpb_launch_gemm(h, (cudaStream_t)stream, y_local, y_dtype, ldy, q, act_scale, act_sum, w, w_bits, w_scale,
                           m, n, k, y_peers, n_peers);
}

int tpb_convrot_gemm_allgather_mc(tpb_handle_t h, tpb_stream_t stream, void *y_mc, void *y_local, int world,
                                  int rank, int y_dtype, int64_t ldy, const int8_t *q, const float *act_scale,
                                  const int32_t *act_sum, const void *w_shard, int w_bits,
                                  const float *w_scale_shard, int64_t m, int64_t n_shard, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y_mc && y_local && tpb_aligned16(y_mc) && tpb_aligned16(y_local),
                  "gemm_allgather_mc: y_mc / y_local null or misaligned");
    TPB_CHECK_ARG(h, world >= 1 && world <= 8 && rank >= 0 && rank < world,
                  "gemm_allgather_mc: need 1 <= world <= 8 and 0 <= rank < world");
    TPB_CHECK_ARG(h, y_dtype == TPB_F32 || y_dtype == TPB_BF16 || y_dtype == TPB_S32,
                  "gemm_allgather_mc: y_dtype must be f32, bf16 or s32");
    TPB_CHECK_ARG(h, n_shard > 0 && ldy >= n_shard * world, "gemm_allgather_mc: ldy must be >= world * n_shard");
    TPB_CHECK_ARG(h, q && w_shard, "gemm_allgather_mc: null pointer");
    TPB_CHECK_ARG(h, y_dtype == TPB_S32 || (act_scale && w_scale_shard), "gemm_allgather_mc: scales are required");
    TPB_CHECK_ARG(h, w_bits == 8 || w_bits == 4, "gemm_allgather_mc: w_bits must be 8 or 4 (got %d)", w_bits);
    TPB_CHECK_ARG(h, w_bits == 8 || act_sum, "gemm_allgather_mc: act_sum is required when w_bits = 4");
    TPB_CHECK_ARG(h, m >= 0 && k > 0 && k % 256 == 0 && n_shard % 16 == 0,
                  "gemm_allgather_mc: need k %% 256 == 0 and n_shard %% 16 == 0");
    TPB_CHECK_ARG(h, m < (1ll << 31) && n_shard * world < (1ll << 31) && k < (1ll << 31),
                  "gemm_allgather_mc: dims exceed 2^31");
    const int64_t ld_mult = y_dtype == TPB_BF16 ? 8 : 4;
    TPB_CHECK_ARG(h, ldy % ld_mult == 0, "gemm_allgather_mc: ldy must be a multiple of %lld", (long long)ld_mult);
    TPB_CHECK_ARG(h, tpb_aligned16(q) && tpb_aligned16(w_shard) && tpb_aligned16(w_scale_shard),
                  "gemm_allgather_mc: q, w and w_scale must be 16-byte aligned");
    if (m == 0) return TPB_OK;
    const size_t esz = y_dtype == TPB_BF16 ? 2 : 4;
    const size_t col_off = (size_t)rank * (size_t)n_shard * esz;
    return tpb_launch_gemm(h, (cudaStream_t)stream, static_cast<char *>(y_local) + col_off, y_dtype, ldy, q, act_scale,
                           act_sum, w_shard, w_bits, w_scale_shard, m, n_shard, k, nullptr, 0,
                           static_cast<char *>(y_mc) + col_off);
}

}  // extern "C"
