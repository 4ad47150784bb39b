// Internal declarations shared by the translation units of libtpb200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdlib>
#include <cstdio>
#include <string>

#include "tpb200.h"

#define TPB_VERSION 100

struct tpb_handle_s {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    uint32_t *d_status = nullptr;   // device status word written by bounded waits
    // cuTensorMapEncodeTiled, resolved through the runtime so the library has no
    // link-time dependency on libcuda (it must load on a host without a driver).
    void *encode_tiled = nullptr;
    // int8 expansion of the int4 weight of the call in flight (grown on demand, freed with the
    // handle).  Calls on one handle are ordered by the caller's stream, so one buffer is enough;
    // two handles never share it.
    int8_t *w4_scratch = nullptr;
    size_t w4_scratch_bytes = 0;
    // switches read from the environment once, at tpb_create
    bool opt_w4_fused = false;      // TPB_W4_FUSED=1: unpack int4 weights inside the GEMM
    bool opt_gemm_one_cta = false;  // TPB_GEMM_ONE_CTA=1: keep large GEMMs on the one-CTA kernel
    char err[512] = {0};
};

int tpb_fail(tpb_handle_t h, int code, const char *fmt, ...);

#define TPB_CHECK_ARG(h, cond, ...)                                   \
    do {                                                              \
        if (!(cond)) return tpb_fail((h), TPB_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

#define TPB_CUDA(h, expr)                                                          \
    do {                                                                           \
        cudaError_t e__ = (expr);                                                  \
        if (e__ != cudaSuccess)                                                    \
            return tpb_fail((h), e__ == cudaErrorMemoryAllocation ? TPB_ERR_OOM : TPB_ERR_CUDA, \
                            "%s failed: %s", #expr, cudaGetErrorString(e__));      \
    } while (0)

// Launch with programmatic stream serialisation: the grid may start while the previous
// kernel in the stream is still draining.  Every kernel launched this way executes
// griddepcontrol.wait before it reads or writes global memory, which also keeps the
// ordering transitive along the stream.  Data that another kernel of the stream may have written
// (activations, scales, modulation vectors, residuals) is loaded with __ldcg, never __ldg: a load
// through the read-only path counts as invariant for the compiler, which may move it above
// griddepcontrol.wait, where it reads what the previous kernel has not written yet.  __ldg is for
// weights and tables that no kernel writes.
template <typename... KArgs, typename... Args>
static inline cudaError_t tpb_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    static const bool no_pdl = getenv("TPB_NO_PDL") != nullptr;
    attr[0].val.programmaticStreamSerializationAllowed = no_pdl ? 0 : 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void tpb_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void tpb_grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

static inline bool tpb_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Kernel launchers (one per .cu file).  All return a tpb_status.
int tpb_launch_prep(tpb_handle_t h, cudaStream_t st, const void *x, int x_dtype, int64_t m,
                    int64_t k, int bits, int8_t *q, float *act_scale, int32_t *act_sum);
int tpb_launch_w4_expand(tpb_handle_t h, cudaStream_t st, const void *w4, int64_t n, int64_t k,
                         int8_t *w8);
int tpb_launch_gemm(tpb_handle_t h, cudaStream_t st, void *y, int y_dtype, int64_t ldy,
                    const int8_t *q, const float *act_scale, const int32_t *act_sum,
                    const void *w, int w_bits, const float *w_scale, int64_t m, int64_t n,
                    int64_t k, void *const *peer_y = nullptr, int n_peers = 0, void *mc_y = nullptr,
                    const float *gate = nullptr);
// The int8 expansion scratch of an [n][k] int4 weight on the handle's device (grown on demand).
int tpb_w4_scratch(tpb_handle_t h, int64_t n, int64_t k, int8_t **out);
int tpb_launch_peer_barrier(tpb_handle_t h, cudaStream_t st, uint32_t *const *flags, int world,
                            int rank, uint32_t epoch, int timeout_ms);
int tpb_launch_q8_1_quantize(tpb_handle_t h, cudaStream_t st, const float *x, int64_t n_elems,
                             void *xq);
int tpb_launch_q8_0_gemv_q8n(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale,
                             int64_t rows, int64_t cols, const void *xq, int ng, int row_off,
                             int n_total);
int tpb_launch_q8_0_gemv_f32(tpb_handle_t h, cudaStream_t st, float *y, const float *x,
                             const void *w, float scale, int64_t rows, int64_t cols);
