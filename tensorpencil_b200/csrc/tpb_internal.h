// Internal declarations shared by the translation units of libtpb200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdlib>
#include <cstdio>
#include <string>

#include "tpb200.h"

#define TPB_VERSION 101
#define TPB_MAX_DEVICES 64   // per-device tables below are indexed by the device ordinal; tpb_create refuses more

// One slot of the per-handle tensor-map cache (see tpb_tensor_map_cached in gemm_common.cuh): a
// tensor map depends only on (base, dims, stride, box, type), and a model calls the same linears with
// the same buffers step after step, so the driver's encode call is made once per distinct operand.
struct tpb_map_slot {
    uint64_t key[5] = {0, 0, 0, 0, 0};
    bool valid = false;
    alignas(64) unsigned char map[128];
};
constexpr int TPB_MAP_CACHE_SLOTS = 128;

struct tpb_handle_s {
    tpb_map_slot map_cache[TPB_MAP_CACHE_SLOTS];
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    uint32_t *d_status = nullptr;   // device status word written by bounded waits
    // cuTensorMapEncodeTiled, resolved through the runtime so the library has no
    // link-time dependency on libcuda (it must load on a host without a driver).
    void *encode_tiled = nullptr;
    // int8 expansion of the int4 weight of the call in flight (sized by tpb_convrot_w4_reserve, freed
    // with the handle).  Calls on one handle are ordered by the caller's stream, so one buffer is
    // enough; two handles never share it.
    int8_t *w4_scratch = nullptr;
    size_t w4_scratch_bytes = 0;
    // switches read from the environment once, at tpb_create
    bool opt_w4_fused = false;      // TPB_W4_FUSED=1: unpack int4 weights inside the GEMM
    bool opt_gemm_one_cta = false;  // TPB_GEMM_ONE_CTA=1: keep large GEMMs on the one-CTA kernel
    int opt_gemm_ablate = 0;        // TPB_GEMM_ABLATE=<bits>: timing diagnosis of the two-CTA GEMM (see GemmParams)
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
// weights and tables that no kernel writes.  For the same reason a kernel parameter that may alias
// another (the in-place elementwise ops: out == first input) or that another kernel of the stream
// writes is never declared `const __restrict__`: that qualifier lets the compiler pick the
// read-only path by itself.
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

// Makes `device` current for the lifetime of the object (allocations and symbol look-ups go to the
// current device, which need not be the handle's when a host drives several handles).
struct tpb_device_guard {
    int prev = -1;
    bool switched = false;
    cudaError_t err = cudaSuccess;
    explicit tpb_device_guard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
            switched = err == cudaSuccess;
        }
    }
    ~tpb_device_guard() {
        if (switched) cudaSetDevice(prev);
    }
};

// "Done once per device" flags for settings that belong to a kernel, not to a handle
// (cudaFuncSetAttribute).  Racing threads at worst both apply the same setting.
struct tpb_per_device_once {
    std::atomic<unsigned char> done[TPB_MAX_DEVICES];
    bool test(int device) const { return done[device & (TPB_MAX_DEVICES - 1)].load(std::memory_order_acquire) != 0; }
    void set(int device) { done[device & (TPB_MAX_DEVICES - 1)].store(1, std::memory_order_release); }
};
// Opts `kern` in to `bytes` of dynamic shared memory, once per device.
template <typename Kern>
static inline cudaError_t tpb_set_max_smem_once(tpb_handle_t h, Kern kern, int bytes, tpb_per_device_once &once) {
    if (once.test(h->device)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) once.set(h->device);
    return e;
}

static inline bool tpb_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Kernel launchers (one per .cu file).  All return a tpb_status.
int tpb_launch_prep(tpb_handle_t h, cudaStream_t st, const void *x, int x_dtype, int64_t m,
                    int64_t k, int bits, int8_t *q, float *act_scale, int32_t *act_sum);
int tpb_launch_w4_expand(tpb_handle_t h, cudaStream_t st, const void *w4, int64_t n, int64_t k,
                         int8_t *w8);
int tpb_launch_gemm_silu_pair(tpb_handle_t h, cudaStream_t st, void *y, int y_dtype, int64_t ldy, const int8_t *q,
                              const float *act_scale, const void *w_gate, const float *w_gate_scale, const void *w_up,
                              const float *w_up_scale, int w_bits, int64_t m, int64_t n, int64_t k);
int tpb_launch_gemm_group(tpb_handle_t h, cudaStream_t st, int count, void *const *y, int y_dtype, int64_t ldy,
                          const int8_t *q, const float *act_scale, const void *const *w, const float *const *w_scale,
                          int w_bits, int64_t m, int64_t n, int64_t k);
int tpb_launch_gemm(tpb_handle_t h, cudaStream_t st, void *y, int y_dtype, int64_t ldy,
                    const int8_t *q, const float *act_scale, const int32_t *act_sum,
                    const void *w, int w_bits, const float *w_scale, int64_t m, int64_t n,
                    int64_t k, void *const *peer_y = nullptr, int n_peers = 0, void *mc_y = nullptr,
                    const float *gate = nullptr);
// The int8 expansion scratch of an [n][k] int4 weight (tpb_convrot_w4_reserve sized it; TPB_ERR_STATE
// when it is too small: no compute entry allocates).
int tpb_w4_scratch(tpb_handle_t h, int64_t n, int64_t k, int8_t **out);
int tpb_launch_peer_barrier(tpb_handle_t h, cudaStream_t st, uint32_t *const *flags, int world,
                            int rank, uint32_t epoch, int timeout_ms);
int tpb_launch_q8_1_quantize(tpb_handle_t h, cudaStream_t st, const float *x, int64_t n_elems,
                             void *xq);
int tpb_launch_q8_0_gemv_q8n(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale,
                             int64_t rows, int64_t cols, const void *xq, int ng, int row_off,
                             int n_total);
int tpb_q8_0_gemv_mma_fits(tpb_handle_t h, int64_t rows, int64_t cols, int *npass, int *np_waste_pct);   // 0 = no; else CTAs K is split over
int tpb_launch_q8_0_gemv_mma(tpb_handle_t h, cudaStream_t st, float *y, const void *w, float scale, int64_t rows,
                             int64_t cols, const void *xq, int ng, int row_off, int n_total);
int tpb_launch_q8_0_gemv_f32(tpb_handle_t h, cudaStream_t st, float *y, const float *x,
                             const void *w, float scale, int64_t rows, int64_t cols);
