// C-ABI entry points of libtpb200.so: handle lifetime, argument validation and
// dispatch to the kernel launchers.  See include/tpb200.h for the contract and
// for the TensorPencil interface each entry point replaces.
#include <cstring>
#include <new>

#include "tpb_internal.h"

#include <cstdlib>

int tpb_fail(tpb_handle_t h, int code, const char *fmt, ...) {
    if (h) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(h->err, sizeof h->err, fmt, ap);
        va_end(ap);
    }
    return code;
}

extern "C" {

int tpb_version(void) { return TPB_VERSION; }

const char *tpb_status_string(int status) {
    switch (status) {
        case TPB_OK: return "ok";
        case TPB_ERR_INVALID_ARG: return "invalid argument";
        case TPB_ERR_CUDA: return "CUDA error";
        case TPB_ERR_OOM: return "out of memory";
        case TPB_ERR_TIMEOUT: return "device-side wait timed out";
        case TPB_ERR_STATE: return "call order violated";
        case TPB_ERR_NO_DEVICE: return "no usable sm_100 device";
        default: return "unknown status";
    }
}

int tpb_create(tpb_handle_t *out, int device_ordinal) {
    if (!out) return TPB_ERR_INVALID_ARG;
    *out = nullptr;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev <= 0) {
        cudaGetLastError();
        return TPB_ERR_NO_DEVICE;
    }
    if (device_ordinal < 0 || device_ordinal >= n_dev || device_ordinal >= TPB_MAX_DEVICES) return TPB_ERR_INVALID_ARG;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return TPB_ERR_CUDA;
    // The kernels are built for sm_100a only: refuse anything else instead of
    // failing at the first launch.
    if (prop.major != 10) return TPB_ERR_NO_DEVICE;
    tpb_handle_s *h = new (std::nothrow) tpb_handle_s();
    if (!h) return TPB_ERR_OOM;
    h->device = device_ordinal;
    h->sm_count = prop.multiProcessorCount;
    h->smem_optin = (int)prop.sharedMemPerBlockOptin;
    const char *e1 = getenv("TPB_W4_FUSED"), *e2 = getenv("TPB_GEMM_ONE_CTA");
    h->opt_w4_fused = e1 != nullptr && e1[0] == '1';
    h->opt_gemm_one_cta = e2 != nullptr && e2[0] == '1';
    if (const char *e3 = getenv("TPB_GEMM_ABLATE")) h->opt_gemm_ablate = atoi(e3) & 31;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e = cudaSetDevice(device_ordinal);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_status, 256);
    if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, 256);
    if (e == cudaSuccess) {
        cudaDriverEntryPointQueryResult qres;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &h->encode_tiled, cudaEnableDefault,
                                    &qres);
        if (e == cudaSuccess && (qres != cudaDriverEntryPointSuccess || !h->encode_tiled))
            e = cudaErrorUnknown;
    }
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
        if (h->d_status) cudaFree(h->d_status);
        delete h;
        return e == cudaErrorMemoryAllocation ? TPB_ERR_OOM : TPB_ERR_CUDA;
    }
    *out = h;
    return TPB_OK;
}

int tpb_destroy(tpb_handle_t h) {
    if (!h) return TPB_ERR_INVALID_ARG;
    if (h->w4_scratch) cudaFree(h->w4_scratch);
    if (h->d_status) cudaFree(h->d_status);
    delete h;
    return TPB_OK;
}

const char *tpb_last_error(tpb_handle_t h) { return h ? h->err : "null handle"; }

int tpb_device_sm_count(tpb_handle_t h) { return h ? h->sm_count : TPB_ERR_INVALID_ARG; }

int tpb_status_poll(tpb_handle_t h, tpb_stream_t stream, uint32_t *detail) {
    if (!h) return TPB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t word = 0;
    TPB_CUDA(h, cudaStreamSynchronize(st));
    TPB_CUDA(h, cudaMemcpyAsync(&word, h->d_status, 4, cudaMemcpyDeviceToHost, st));
    TPB_CUDA(h, cudaStreamSynchronize(st));
    if (detail) *detail = word;
    if (word != 0) {
        TPB_CUDA(h, cudaMemsetAsync(h->d_status, 0, 4, st));
        return tpb_fail(h, TPB_ERR_TIMEOUT, "bounded wait expired on the device (status 0x%08x)",
                        word);
    }
    return TPB_OK;
}

int tpb_convrot_prep(tpb_handle_t h, tpb_stream_t stream, const void *x, int x_dtype, int64_t m,
                     int64_t k, int bits, int8_t *q, float *act_scale, int32_t *act_sum) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, x && q && act_scale, "prep: null pointer");
    TPB_CHECK_ARG(h, bits == 8 || bits == 4, "prep: bits must be 8 or 4 (got %d)", bits);
    TPB_CHECK_ARG(h, x_dtype == TPB_F32 || x_dtype == TPB_F16 || x_dtype == TPB_BF16,
                  "prep: x_dtype must be f32, f16 or bf16");
    TPB_CHECK_ARG(h, m >= 0 && k > 0 && k % 256 == 0 && k <= 32768,
                  "prep: k must be a multiple of 256 in [256, 32768] (m=%lld k=%lld)",
                  (long long)m, (long long)k);
    TPB_CHECK_ARG(h, bits == 8 || act_sum, "prep: act_sum is required when bits = 4");
    TPB_CHECK_ARG(h, tpb_aligned16(x) && tpb_aligned16(q), "prep: x and q must be 16-byte aligned");
    if (m == 0) return TPB_OK;
    return tpb_launch_prep(h, (cudaStream_t)stream, x, x_dtype, m, k, bits, q, act_scale, act_sum);
}

int tpb_convrot_w4_reserve(tpb_handle_t h, int64_t n, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, n > 0 && k > 0 && n < (1ll << 31) && k < (1ll << 31), "w4_reserve: bad shape");
    const size_t need = (size_t)n * (size_t)k;
    if (h->w4_scratch_bytes >= need) return TPB_OK;
    tpb_device_guard guard(h->device);
    TPB_CUDA(h, guard.err);
    // cudaFree waits for the work that may still read the old buffer
    if (h->w4_scratch) TPB_CUDA(h, cudaFree(h->w4_scratch));
    h->w4_scratch = nullptr;
    h->w4_scratch_bytes = 0;
    TPB_CUDA(h, cudaMalloc(&h->w4_scratch, need));
    h->w4_scratch_bytes = need;
    return TPB_OK;
}

size_t tpb_convrot_w4_expanded_bytes(int64_t n, int64_t k) {
    return (n > 0 && k > 0) ? (size_t)n * (size_t)k : 0;
}

int tpb_convrot_w4_expand(tpb_handle_t h, tpb_stream_t stream, const void *w4, int64_t n,
                          int64_t k, int8_t *w8) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, w4 && w8, "w4_expand: null pointer");
    TPB_CHECK_ARG(h, n >= 0 && k > 0 && k % 32 == 0, "w4_expand: k must be a multiple of 32");
    TPB_CHECK_ARG(h, tpb_aligned16(w4) && tpb_aligned16(w8), "w4_expand: pointers must be 16-byte aligned");
    if (n == 0) return TPB_OK;
    return tpb_launch_w4_expand(h, (cudaStream_t)stream, w4, n, k, w8);
}

int tpb_convrot_gemm(tpb_handle_t h, tpb_stream_t stream, void *y, int y_dtype, int64_t ldy,
                     const int8_t *q, const float *act_scale, const int32_t *act_sum,
                     const void *w, int w_bits, const float *w_scale, int64_t m, int64_t n,
                     int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y && q && w, "gemm: null pointer");
    TPB_CHECK_ARG(h, y_dtype == TPB_F32 || y_dtype == TPB_BF16 || y_dtype == TPB_S32,
                  "gemm: y_dtype must be f32, bf16 or s32");
    TPB_CHECK_ARG(h, y_dtype == TPB_S32 || (act_scale && w_scale), "gemm: scales are required");
    TPB_CHECK_ARG(h, w_bits == 8 || w_bits == 4, "gemm: w_bits must be 8 or 4 (got %d)", w_bits);
    TPB_CHECK_ARG(h, w_bits == 8 || act_sum, "gemm: act_sum is required when w_bits = 4");
    TPB_CHECK_ARG(h, m >= 0 && n > 0 && k > 0 && k % 256 == 0 && n % 16 == 0,
                  "gemm: need k %% 256 == 0 and n %% 16 == 0 (m=%lld n=%lld k=%lld)", (long long)m,
                  (long long)n, (long long)k);
    TPB_CHECK_ARG(h, m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "gemm: dims exceed 2^31");
    const int64_t ld_mult = y_dtype == TPB_BF16 ? 8 : 4;
    TPB_CHECK_ARG(h, ldy >= n && ldy % ld_mult == 0, "gemm: ldy must be >= n and a multiple of %lld",
                  (long long)ld_mult);
    TPB_CHECK_ARG(h, tpb_aligned16(y) && tpb_aligned16(q) && tpb_aligned16(w) &&
                         tpb_aligned16(w_scale) && ((reinterpret_cast<uintptr_t>(act_scale) & 3u) == 0),
                  "gemm: y, q, w and w_scale must be 16-byte aligned");
    if (m == 0) return TPB_OK;
    return tpb_launch_gemm(h, (cudaStream_t)stream, y, y_dtype, ldy, q, act_scale, act_sum, w,
                           w_bits, w_scale, m, n, k);
}

int tpb_convrot_linear(tpb_handle_t h, tpb_stream_t stream, void *y, int y_dtype, int64_t ldy, const void *x,
                       int x_dtype, int8_t *q, float *act_scale, int32_t *act_sum, const void *w, int w_bits,
                       const float *w_scale, int64_t m, int64_t n, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // Validate everything before anything is enqueued (m = 0 runs the checks only).
    int rc = tpb_convrot_prep(h, nullptr, x, x_dtype, 0, k, w_bits, q, act_scale, act_sum);
    if (rc != TPB_OK) return rc;
    rc = tpb_convrot_gemm(h, nullptr, y, y_dtype, ldy, q, act_scale, act_sum, w, w_bits, w_scale, 0, n, k);
    if (rc != TPB_OK) return rc;
    TPB_CHECK_ARG(h, m >= 0 && m < (1ll << 31), "linear: bad m");
    if (m == 0) return TPB_OK;
    if (w_bits != 4 || h->opt_w4_fused) {
        rc = tpb_launch_prep(h, st, x, x_dtype, m, k, w_bits, q, act_scale, act_sum);
        if (rc != TPB_OK) return rc;
        return tpb_launch_gemm(h, st, y, y_dtype, ldy, q, act_scale, act_sum, w, w_bits, w_scale, m, n, k);
    }
    // INT4: widen the weight, prepare the activations, multiply.  (Running the widening beside
    // the prep -- on a second stream, or as extra CTAs mixed into the prep's grid -- was measured
    // and gains nothing: both passes already run at the same ~4.2 TB/s.)
    int8_t *w8 = nullptr;
    rc = tpb_w4_scratch(h, n, k, &w8);
    if (rc != TPB_OK) return rc;
    rc = tpb_launch_w4_expand(h, st, w, n, k, w8);
    if (rc != TPB_OK) return rc;
    rc = tpb_launch_prep(h, st, x, x_dtype, m, k, 4, q, act_scale, act_sum);
    if (rc != TPB_OK) return rc;
    return tpb_launch_gemm(h, st, y, y_dtype, ldy, q, act_scale, nullptr, w8, 8, w_scale, m, n, k);
}

int tpb_convrot_gemm_gated_add(tpb_handle_t h, tpb_stream_t stream, float *x, int64_t ldx, const float *gate,
                               const int8_t *q, const float *act_scale, const int32_t *act_sum, const void *w,
                               int w_bits, const float *w_scale, int64_t m, int64_t n, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, gate && tpb_aligned16(gate), "gemm_gated_add: gate is null or misaligned");
    // everything else is checked as for the plain GEMM with an f32 output
    const int rc = tpb_convrot_gemm(h, nullptr, x, TPB_F32, ldx, q, act_scale, act_sum, w, w_bits, w_scale, 0, n, k);
    if (rc != TPB_OK) return rc;
    TPB_CHECK_ARG(h, m >= 0 && m < (1ll << 31), "gemm_gated_add: bad m");
    if (m == 0) return TPB_OK;
    return tpb_launch_gemm(h, (cudaStream_t)stream, x, TPB_F32, ldx, q, act_scale, act_sum, w, w_bits, w_scale, m, n,
                           k, nullptr, 0, nullptr, gate);
}

int tpb_convrot_gemm_silu_pair(tpb_handle_t h, tpb_stream_t stream, void *y, int y_dtype, int64_t ldy, const int8_t *q,
                               const float *act_scale, const int32_t *act_sum, const void *w_gate,
                               const float *w_gate_scale, const void *w_up, const float *w_up_scale, int w_bits,
                               int64_t m, int64_t n, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y_dtype == TPB_F32 || y_dtype == TPB_BF16, "gemm_silu_pair: y_dtype must be f32 or bf16");
    // each weight is checked as for the plain GEMM
    int rc = tpb_convrot_gemm(h, nullptr, y, y_dtype, ldy, q, act_scale, act_sum, w_gate, w_bits, w_gate_scale, 0, n, k);
    if (rc != TPB_OK) return rc;
    rc = tpb_convrot_gemm(h, nullptr, y, y_dtype, ldy, q, act_scale, act_sum, w_up, w_bits, w_up_scale, 0, n, k);
    if (rc != TPB_OK) return rc;
    TPB_CHECK_ARG(h, m >= 0 && m < (1ll << 31), "gemm_silu_pair: bad m");
    if (m == 0) return TPB_OK;
    return tpb_launch_gemm_silu_pair(h, (cudaStream_t)stream, y, y_dtype, ldy, q, act_scale, w_gate, w_gate_scale, w_up,
                                     w_up_scale, w_bits, m, n, k);
}

int tpb_convrot_gemm_group(tpb_handle_t h, tpb_stream_t stream, int count, void *const *y, int y_dtype, int64_t ldy,
                           const int8_t *q, const float *act_scale, const int32_t *act_sum, const void *const *w,
                           const float *const *w_scale, int w_bits, int64_t m, int64_t n, int64_t k) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, count >= 1 && count <= 4, "gemm_group: 1 to 4 weights per call (got %d)", count);
    TPB_CHECK_ARG(h, y && w && w_scale, "gemm_group: null pointer");
    TPB_CHECK_ARG(h, y_dtype == TPB_F32 || y_dtype == TPB_BF16, "gemm_group: y_dtype must be f32 or bf16");
    // each weight and output is checked as for the plain GEMM
    for (int g = 0; g < count; g++) {
        const int rc = tpb_convrot_gemm(h, nullptr, y[g], y_dtype, ldy, q, act_scale, act_sum, w[g], w_bits, w_scale[g], 0, n, k);
        if (rc != TPB_OK) return rc;
    }
    TPB_CHECK_ARG(h, m >= 0 && m < (1ll << 31), "gemm_group: bad m");
    if (m == 0) return TPB_OK;
    return tpb_launch_gemm_group(h, (cudaStream_t)stream, count, y, y_dtype, ldy, q, act_scale, w, w_scale, w_bits, m, n, k);
}

int tpb_q8_1_quantize(tpb_handle_t h, tpb_stream_t stream, const float *x, int64_t n_elems,
                      void *xq) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, x && xq, "q8_1_quantize: null pointer");
    TPB_CHECK_ARG(h, n_elems >= 0 && n_elems % 32 == 0, "q8_1_quantize: n_elems must be a multiple of 32");
    TPB_CHECK_ARG(h, tpb_aligned16(x) && tpb_aligned16(xq), "q8_1_quantize: pointers must be 16-byte aligned");
    if (n_elems == 0) return TPB_OK;
    return tpb_launch_q8_1_quantize(h, (cudaStream_t)stream, x, n_elems, xq);
}

int tpb_q8_0_gemv_q8n(tpb_handle_t h, tpb_stream_t stream, float *y, const void *w, float scale,
                      int64_t rows, int64_t cols, const void *xq, int ng, int row_off,
                      int n_total) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y && w && xq, "q8_0_gemv_q8n: null pointer");
    TPB_CHECK_ARG(h, rows >= 0 && rows < (1ll << 26) && cols > 0 && cols % 32 == 0 && cols < (1ll << 24),
                  "q8_0_gemv_q8n: cols must be a multiple of 32 (below 2^24) and rows below 2^26");
    TPB_CHECK_ARG(h, ng >= 1 && ng <= 8 && row_off >= 0 && row_off + ng <= n_total,
                  "q8_0_gemv_q8n: need 1 <= ng <= 8 and row_off + ng <= n_total");
    TPB_CHECK_ARG(h, tpb_aligned16(w) && tpb_aligned16(xq), "q8_0_gemv_q8n: w and xq must be 16-byte aligned");
    if (rows == 0) return TPB_OK;
    return tpb_launch_q8_0_gemv_q8n(h, (cudaStream_t)stream, y, w, scale, rows, cols, xq, ng,
                                    row_off, n_total);
}

int tpb_q8_0_gemv_f32(tpb_handle_t h, tpb_stream_t stream, float *y, const float *x, const void *w,
                      float scale, int64_t rows, int64_t cols) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, y && x && w, "q8_0_gemv_f32: null pointer");
    TPB_CHECK_ARG(h, rows >= 0 && rows < (1ll << 31) && cols > 0 && cols % 32 == 0,
                  "q8_0_gemv_f32: cols must be a multiple of 32 and rows below 2^31");
    TPB_CHECK_ARG(h, tpb_aligned16(w) && tpb_aligned16(x), "q8_0_gemv_f32: w and x must be 16-byte aligned");
    if (rows == 0) return TPB_OK;
    return tpb_launch_q8_0_gemv_f32(h, (cudaStream_t)stream, y, x, w, scale, rows, cols);
}

int tpb_host_alloc(tpb_handle_t h, size_t bytes, void **out) {
    if (!h || !out) return TPB_ERR_INVALID_ARG;
    *out = nullptr;
    cudaError_t e = cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocPortable);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tpb_fail(h, TPB_ERR_OOM, "pinned host allocation of %zu bytes failed: %s", bytes,
                        cudaGetErrorString(e));
    }
    return TPB_OK;
}

int tpb_host_free(tpb_handle_t h, void *p) {
    if (!h) return TPB_ERR_INVALID_ARG;
    if (p) TPB_CUDA(h, cudaFreeHost(p));
    return TPB_OK;
}

}  // extern "C"
