// tpb200.hpp -- C++ mirror of TensorPencil's cuda.Backend operator interface for the
// quantized-linear path, header-only, on top of the C ABI in tpb200.h.
//
// Same method names, argument meaning and error behaviour as the reference's Zig
// Backend (src/gpu/cuda/backend.zig; line numbers at each method), so that host code and
// tests written against the reference read the same here: device tensors are opaque
// DeviceBuffers, weights arrive as HOST byte slices and are cached on the device by
// host address (cachedWeight, backend.zig:1376-1445), the prepped activation lives in
// backend-owned scratch (i8_x / i8_scale) between op{I8,I4}Prep and the GEMMs that follow,
// and every failure throws tpb::Error carrying the tpb_status (the reference returns
// error.CudaError / error.DeviceOutOfMemory).
//
// Needs the CUDA runtime headers for allocation and copies; link with libtpb200.so and
// libcudart.  One Backend per host thread (thread-compatible, like the reference's).
#ifndef TPB200_HPP
#define TPB200_HPP

#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "tpb200.h"
#include "tpb200_cache.hpp"

namespace tpb {

struct Error : std::runtime_error {
    int status;
    Error(int st, const std::string &what) : std::runtime_error(what), status(st) {}
};

// The reference's DType values this path uses (src/core/dtype.zig).
enum class DType { f32, f16, bf16, i8, i4, q8_0, q4_0, q4_k, q5_k, q6_k, iq4_nl };

struct DeviceBuffer {  // src/gpu/cuda/context.zig DeviceBuffer: an address and a size
    void *p = nullptr;
    size_t size = 0;
    void *ptr() const { return p; }
};

class Backend {
  public:
    // Backend.init (backend.zig:459): binds to `device`, creates the compute stream.
    explicit Backend(int device = 0) : device_(device) {
        int rc = tpb_create(&h_, device);
        if (rc != TPB_OK) throw Error(rc, std::string("tpb_create: ") + tpb_status_string(rc));
        cuda(cudaSetDevice(device), "cudaSetDevice");
        cuda(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    }
    // Backend.deinit (backend.zig:514)
    ~Backend() {
        if (stream_) cudaStreamSynchronize(stream_);
        dropWeights();
        release(i8_x_);
        release(attn_q_);
        release(attn_k_);
        release(attn_vt_);
        release(i8_scale_);
        release(i8_sum_);
        release(q8_);
        if (stream_) cudaStreamDestroy(stream_);
        if (h_) tpb_destroy(h_);
    }
    Backend(const Backend &) = delete;
    Backend &operator=(const Backend &) = delete;

    cudaStream_t stream() const { return stream_; }

    // ---- tensors (backend.zig:740, :1172, :1257, :1262) ----
    DeviceBuffer tensorCreate(uint64_t size) {
        DeviceBuffer db;
        const cudaError_t e = cudaMalloc(&db.p, size ? size : 1);
        if (e == cudaErrorMemoryAllocation) {
            (void)cudaGetLastError();
            throw Error(TPB_ERR_OOM, "tensorCreate: DeviceOutOfMemory");
        }
        cuda(e, "cudaMalloc");
        db.size = size;
        return db;
    }
    void tensorDestroy(DeviceBuffer &db) { release(db); }
    void tensorUpload(DeviceBuffer db, const void *bytes, size_t n) {
        if (n > db.size) throw Error(TPB_ERR_INVALID_ARG, "tensorUpload: source larger than the tensor");
        cuda(cudaMemcpyAsync(db.p, bytes, n, cudaMemcpyHostToDevice, stream_), "tensorUpload");
    }
    // Synchronises, as the reference's download does: the bytes are valid on return.
    void tensorDownload(DeviceBuffer db, void *out, size_t n) {
        if (n > db.size) throw Error(TPB_ERR_INVALID_ARG, "tensorDownload: destination larger than the tensor");
        cuda(cudaMemcpyAsync(out, db.p, n, cudaMemcpyDeviceToHost, stream_), "tensorDownload");
        sync();
    }
    // Waits for the stream and surfaces a bounded device-side wait that gave up.
    void sync() { check(tpb_status_poll(h_, stream_, nullptr)); }

    // ---- weight cache keyed by host address (backend.zig:1376-1445) ----
    // As in the reference, a cached weight is identified by its host address and size only:
    // keep weight memory alive and unchanged while cached, or call dropWeights() first.
    const void *cachedWeight(const void *host, size_t bytes, bool pin = false) {
        try {
            return weights_.get(host, bytes, pin).p;
        } catch (const CacheFull &e) {
            throw Error(TPB_ERR_OOM, e.what());
        }
    }
    // --vram-budget for the weights (backend.zig:222-252): least-recently-used weights that are not
    // pinned are freed to make room; 0 = no limit.  Freeing synchronises the device (cudaFree), so a
    // weight is never released under a kernel that still reads it.
    void setWeightBudget(size_t bytes) { weights_.setBudget(bytes); }
    void unpinWeight(const void *host) { weights_.unpin(host); }
    size_t weightBytes() const { return weights_.bytes(); }
    size_t weightEvictions() const { return weights_.evictions; }
    void dropWeights() {
        if (stream_) cudaStreamSynchronize(stream_);
        weights_.dropAll();
    }

    // ---- ConvRot linears ----
    // opI8Prep (backend.zig:2454-2480): rotate + per-row int8 quantise x[m][cols] (f32, or f16
    // when in_f16) into the backend's prepped activation.
    void opI8Prep(DeviceBuffer x, size_t m, size_t cols, bool in_f16 = false) {
        prep(x, in_f16 ? TPB_F16 : TPB_F32, m, cols, 8);
    }
    // opI4Prep (backend.zig:2532-2553)
    void opI4Prep(DeviceBuffer x, size_t m, size_t cols) { prep(x, TPB_F32, m, cols, 4); }
    // bf16 activations (no reference counterpart: its 16-bit chain is f16)
    void opPrepBf16(DeviceBuffer x, size_t m, size_t cols, int bits) { prep(x, TPB_BF16, m, cols, bits); }

    // opI8Gemm (backend.zig:2484-2501): y[m][rows] = prepped @ W^T * act_scale[row] * weight_scale[col].
    // c_h16 selects a 16-bit output (bf16 here, f16 in the reference's .libs mode).
    void opI8Gemm(DeviceBuffer y, const void *w_bytes, const float *weight_scale, size_t rows, bool c_h16 = false) {
        gemm(y, w_bytes, rows * cols_, weight_scale, rows, 8, c_h16 ? TPB_BF16 : TPB_F32);
    }
    // opI4Gemm (backend.zig:2558-2573): w_bytes is the packed weight [rows][cols/2]
    void opI4Gemm(DeviceBuffer y, const void *w_bytes, const float *weight_scale, size_t rows) {
        gemm(y, w_bytes, rows * cols_ / 2, weight_scale, rows, 4, TPB_F32);
    }

    // ---- elementwise neighbours (backend.zig:2738, :3294, :3310, :3342) ----
    void rmsMod(DeviceBuffer x, DeviceBuffer out, DeviceBuffer mod, size_t rows, size_t dim, size_t premul_off,
                size_t shift_off, float eps) {
        const float *m = static_cast<const float *>(mod.p);
        check(tpb_rms_mod(h_, stream_, x.p, TPB_F32, static_cast<float *>(out.p), m + premul_off, m + shift_off, eps,
                          (int64_t)rows, (int64_t)dim));
    }
    void siluMul(DeviceBuffer a, DeviceBuffer b, size_t total) {
        check(tpb_silu_mul(h_, stream_, a.p, b.p, TPB_F32, static_cast<float *>(a.p), (int64_t)total));
    }
    void sigmoidMul(DeviceBuffer a, DeviceBuffer b, size_t total) {
        check(tpb_sigmoid_mul(h_, stream_, a.p, b.p, TPB_F32, static_cast<float *>(a.p), (int64_t)total));
    }
    void gatedAdd(DeviceBuffer a, DeviceBuffer b, DeviceBuffer mod, size_t total, size_t dim, size_t gate_off) {
        check(tpb_gated_add(h_, stream_, static_cast<float *>(a.p), b.p, TPB_F32,
                            static_cast<const float *>(mod.p) + gate_off, (int64_t)(total / dim), (int64_t)dim));
    }

    // ---- the same ops folded into the prep and the GEMM epilogue (no reference counterpart: it runs
    // op, then prep; GEMM, then gatedAdd).  q / scales are bit-identical to the two-call sequences. ----
    // rmsMod + opI{8,4}Prep (dit_cuda.zig:473-474, :499-500)
    void prepRmsMod(DeviceBuffer x, DeviceBuffer mod, size_t rows, size_t dim, size_t premul_off, size_t shift_off, float eps,
                    int bits = 8) {
        const float *m = static_cast<const float *>(mod.p);
        prepFused(TPB_OP_RMS_MOD, x.p, nullptr, m + premul_off, m + shift_off, eps, rows, dim, bits);
    }
    // siluMul + prep (dit_cuda.zig:513-514) and sigmoidMul + prep (:490-491)
    void prepSiluMul(DeviceBuffer gate, DeviceBuffer up, size_t m, size_t cols, int bits = 8) {
        prepFused(TPB_OP_SILU_MUL, gate.p, up.p, nullptr, nullptr, 0.0f, m, cols, bits);
    }
    void prepSigmoidMul(DeviceBuffer a, DeviceBuffer gate, size_t m, size_t cols, int bits = 8) {
        prepFused(TPB_OP_SIGMOID_MUL, a.p, gate.p, nullptr, nullptr, 0.0f, m, cols, bits);
    }
    // opI{8,4}Gemm + gatedAdd (dit_cuda.zig:492-493, :515-516): x[m][rows] += mod[gate_off + c] * linear
    void gemmGatedAdd(DeviceBuffer x, const void *w_bytes, const float *weight_scale, size_t rows, DeviceBuffer mod,
                      size_t gate_off, int bits = 8) {
        if (bits_ != bits) throw Error(TPB_ERR_STATE, "gemmGatedAdd must follow the matching prep");
        const size_t w_size = bits == 4 ? rows * cols_ / 2 : rows * cols_;
        const void *w = cachedWeight(w_bytes, w_size, true);
        const float *ws = nullptr;
        try {
            ws = static_cast<const float *>(cachedWeight(weight_scale, rows * 4));
        } catch (...) {
            unpinWeight(w_bytes);
            throw;
        }
        unpinWeight(w_bytes);
        if (bits == 4) reserveW4(rows, cols_);
        check(tpb_convrot_gemm_gated_add(h_, stream_, static_cast<float *>(x.p), (int64_t)rows,
                                         static_cast<const float *>(mod.p) + gate_off, static_cast<const int8_t *>(i8_x_.p),
                                         static_cast<const float *>(i8_scale_.p),
                                         bits == 4 ? static_cast<const int32_t *>(i8_sum_.p) : nullptr, w, bits, ws,
                                         (int64_t)m_, (int64_t)rows, (int64_t)cols_));
    }

    // mlp.gate GEMM + mlp.up GEMM + siluMul in one launch (dit_cuda.zig:508-513):
    // y[m][rows] = silu(linear_gate(prepped)) * linear_up(prepped), f32
    void gemmSiluPair(DeviceBuffer y, const void *gate_bytes, const float *gate_scale, const void *up_bytes,
                      const float *up_scale, size_t rows, int bits = 8) {
        if (bits_ != bits) throw Error(TPB_ERR_STATE, "gemmSiluPair must follow the matching prep");
        const size_t w_size = bits == 4 ? rows * cols_ / 2 : rows * cols_;
        // all four arrays must be resident at once: pin each until the call is enqueued
        const void *hosts[4] = {gate_bytes, gate_scale, up_bytes, up_scale};
        const size_t sizes[4] = {w_size, rows * 4, w_size, rows * 4};
        const void *dev[4] = {nullptr, nullptr, nullptr, nullptr};
        int pinned = 0;
        try {
            for (; pinned < 4; pinned++) dev[pinned] = cachedWeight(hosts[pinned], sizes[pinned], true);
        } catch (...) {
            for (int i = 0; i < pinned; i++) unpinWeight(hosts[i]);
            throw;
        }
        for (int i = 0; i < 4; i++) unpinWeight(hosts[i]);
        if (bits == 4) reserveW4(2 * rows, cols_);
        check(tpb_convrot_gemm_silu_pair(h_, stream_, y.p, TPB_F32, (int64_t)rows, static_cast<const int8_t *>(i8_x_.p),
                                         static_cast<const float *>(i8_scale_.p),
                                         bits == 4 ? static_cast<const int32_t *>(i8_sum_.p) : nullptr, dev[0],
                                         static_cast<const float *>(dev[1]), dev[2], static_cast<const float *>(dev[3]),
                                         bits, (int64_t)m_, (int64_t)rows, (int64_t)cols_));
    }

    // Up to four op{I8,I4}Gemm calls on the same prepped activations in one launch (q, k, v and gate of a block,
    // dit_cuda.zig:473-478): ys[g][m][rows] = linear_g(prepped), f32, bit-identical to the separate calls.
    void gemmGroup(int count, const DeviceBuffer *ys, const void *const *w_bytes, const float *const *w_scales, size_t rows,
                   int bits = 8) {
        if (bits_ != bits) throw Error(TPB_ERR_STATE, "gemmGroup must follow the matching prep");
        if (count < 1 || count > 4) throw Error(TPB_ERR_INVALID_ARG, "gemmGroup takes 1 to 4 weights");
        const size_t w_size = bits == 4 ? rows * cols_ / 2 : rows * cols_;
        // every array must be resident at once: pin each until the call is enqueued
        const void *hosts[8];
        size_t sizes[8];
        for (int g = 0; g < count; g++) {
            hosts[2 * g] = w_bytes[g];
            sizes[2 * g] = w_size;
            hosts[2 * g + 1] = w_scales[g];
            sizes[2 * g + 1] = rows * 4;
        }
        const void *dev[8];
        int pinned = 0;
        try {
            for (; pinned < 2 * count; pinned++) dev[pinned] = cachedWeight(hosts[pinned], sizes[pinned], true);
        } catch (...) {
            for (int i = 0; i < pinned; i++) unpinWeight(hosts[i]);
            throw;
        }
        for (int i = 0; i < 2 * count; i++) unpinWeight(hosts[i]);
        if (bits == 4) reserveW4((size_t)count * rows, cols_);
        void *y[4];
        const void *w[4];
        const float *sc[4];
        for (int g = 0; g < count; g++) {
            y[g] = ys[g].p;
            w[g] = dev[2 * g];
            sc[g] = static_cast<const float *>(dev[2 * g + 1]);
        }
        check(tpb_convrot_gemm_group(h_, stream_, count, y, TPB_F32, (int64_t)rows, static_cast<const int8_t *>(i8_x_.p),
                                     static_cast<const float *>(i8_scale_.p),
                                     bits == 4 ? static_cast<const int32_t *>(i8_sum_.p) : nullptr, w, sc, bits, (int64_t)m_,
                                     (int64_t)rows, (int64_t)cols_));
    }

    // ---- attention of the DiT block (dit_cuda.zig:479-489: qkNorm, rope, attn / opAttnTC) ----
    // q [seq][heads*hd], k / v [seq][kv_heads*hd] (f32), freqs = cos table [seq][hd/2] then, sin_off floats
    // later, the sin table; out [seq][heads*hd] f32.  head_dim 128, non-causal.  Unlike the reference's
    // in-place qkNorm / rope, q and k are left untouched (the rotated bf16 copies live in scratch).
    void attention(DeviceBuffer q, DeviceBuffer k, DeviceBuffer v, DeviceBuffer out, DeviceBuffer q_norm,
                   DeviceBuffer k_norm, DeviceBuffer freqs, size_t sin_off, size_t seq, size_t heads, size_t kv_heads,
                   size_t hd, float eps, float scale) {
        ensure(attn_q_, heads * seq * hd * 2);
        ensure(attn_k_, kv_heads * seq * hd * 2);
        ensure(attn_vt_, tpb_attn_vt_elems((int64_t)seq, (int)kv_heads) * 2);
        const float *f = static_cast<const float *>(freqs.p);
        check(tpb_attn_prepare(h_, stream_, q.p, k.p, v.p, TPB_F32, static_cast<const float *>(q_norm.p),
                               static_cast<const float *>(k_norm.p), eps, f, f + sin_off, (int64_t)seq, (int)heads,
                               (int)kv_heads, (int)hd, attn_q_.p, attn_k_.p, attn_vt_.p));
        check(tpb_attention(h_, stream_, out.p, TPB_F32, attn_q_.p, attn_k_.p, attn_vt_.p, (int64_t)seq, (int64_t)seq,
                            (int)heads, (int)kv_heads, (int)hd, scale));
    }

    // ---- GGUF decode GEMV ----
    // opGemvQuantizeX (backend.zig:1687-1695): cols = total element count, a multiple of 32
    void opGemvQuantizeX(DeviceBuffer x, size_t cols) {
        ensure(q8_, cols / 32 * 4 + cols);
        check(tpb_q8_1_quantize(h_, stream_, static_cast<const float *>(x.p), (int64_t)cols, q8_.p));
        q8_total_ = cols;
    }
    // opGemvQuantQ8N (backend.zig:1719-1735)
    void opGemvQuantQ8N(DType dt, DeviceBuffer y, const void *w_bytes, float scale, size_t rows, size_t cols, size_t ng,
                        size_t row_off, size_t n_total) {
        if (q8_total_ != n_total * cols) throw Error(TPB_ERR_STATE, "opGemvQuantQ8N: activations were not staged for this shape");
        const int fmt = ggufFormat(dt);
        const void *w = cachedWeight(w_bytes, rows * tpb_gguf_row_bytes(fmt, (int64_t)cols));
        check(tpb_gguf_gemv_q8n(h_, stream_, fmt, static_cast<float *>(y.p), w, scale, (int64_t)rows, (int64_t)cols, q8_.p,
                                (int)ng, (int)row_off, (int)n_total));
    }
    // opGemvQuant (backend.zig:1660-1681): one activation row, quantised on the way
    void opGemvQuant(DType dt, DeviceBuffer y, DeviceBuffer x, const void *w_bytes, float scale, size_t rows, size_t cols) {
        opGemvQuantizeX(x, cols);
        opGemvQuantQ8N(dt, y, w_bytes, scale, rows, cols, 1, 0, 1);
    }

  private:
    static int ggufFormat(DType dt) {
        switch (dt) {
            case DType::q8_0: return TPB_GGUF_Q8_0;
            case DType::q4_0: return TPB_GGUF_Q4_0;
            case DType::q4_k: return TPB_GGUF_Q4_K;
            case DType::q5_k: return TPB_GGUF_Q5_K;
            case DType::q6_k: return TPB_GGUF_Q6_K;
            case DType::iq4_nl: return TPB_GGUF_IQ4_NL;
            default: throw Error(TPB_ERR_INVALID_ARG, "unsupported GEMV weight format");
        }
    }
    void prep(DeviceBuffer x, int x_dtype, size_t m, size_t cols, int bits) {
        ensure(i8_x_, m * cols);
        ensure(i8_scale_, m * 4);
        ensure(i8_sum_, m * 4);
        check(tpb_convrot_prep(h_, stream_, x.p, x_dtype, (int64_t)m, (int64_t)cols, bits, static_cast<int8_t *>(i8_x_.p),
                               static_cast<float *>(i8_scale_.p), static_cast<int32_t *>(i8_sum_.p)));
        m_ = m;
        cols_ = cols;
        bits_ = bits;
    }
    void prepFused(int op, const void *a, const void *b, const float *premul, const float *shift, float eps, size_t m,
                   size_t cols, int bits) {
        ensure(i8_x_, m * cols);
        ensure(i8_scale_, m * 4);
        ensure(i8_sum_, m * 4);
        check(tpb_convrot_prep_fused(h_, stream_, op, a, b, premul, shift, eps, TPB_F32, (int64_t)m, (int64_t)cols, bits,
                                     static_cast<int8_t *>(i8_x_.p), static_cast<float *>(i8_scale_.p),
                                     static_cast<int32_t *>(i8_sum_.p)));
        m_ = m;
        cols_ = cols;
        bits_ = bits;
    }
    void gemm(DeviceBuffer y, const void *w_host, size_t w_bytes, const float *ws_host, size_t rows, int bits, int y_dtype) {
        if (bits_ != bits) throw Error(TPB_ERR_STATE, "op{I8,I4}Gemm must follow the matching prep");
        // the weight stays pinned while its scales are fetched: under a tight budget the second
        // lookup must not evict the first
        const void *w = cachedWeight(w_host, w_bytes, true);
        const float *ws = nullptr;
        try {
            ws = static_cast<const float *>(cachedWeight(ws_host, rows * 4));
        } catch (...) {
            unpinWeight(w_host);
            throw;
        }
        unpinWeight(w_host);
        if (bits == 4) reserveW4(rows, cols_);
        check(tpb_convrot_gemm(h_, stream_, y.p, y_dtype, (int64_t)rows, static_cast<const int8_t *>(i8_x_.p),
                               static_cast<const float *>(i8_scale_.p),
                               bits == 4 ? static_cast<const int32_t *>(i8_sum_.p) : nullptr, w, bits, ws, (int64_t)m_,
                               (int64_t)rows, (int64_t)cols_));
    }
    // int4 weights are widened into a scratch the library owns; it is sized here, on the set-up
    // side, so that the GEMM entry points never allocate (tpb_convrot_w4_reserve)
    void reserveW4(size_t rows, size_t cols) {
        if (rows * cols <= w4_reserved_) return;
        check(tpb_convrot_w4_reserve(h_, (int64_t)rows, (int64_t)cols));
        w4_reserved_ = rows * cols;
    }
    void ensure(DeviceBuffer &db, size_t bytes) {
        if (db.size >= bytes && db.p) return;
        if (db.p) {
            cuda(cudaStreamSynchronize(stream_), "sync before regrowing scratch");
            release(db);
        }
        db = tensorCreate(bytes);
    }
    static void release(DeviceBuffer &db) {
        if (db.p) cudaFree(db.p);
        db.p = nullptr;
        db.size = 0;
    }
    void check(int rc) {
        if (rc != TPB_OK) throw Error(rc, tpb_last_error(h_));
    }
    static void cuda(cudaError_t e, const char *what) {
        if (e != cudaSuccess) throw Error(TPB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    }

    tpb_handle_t h_ = nullptr;
    int device_ = 0;
    cudaStream_t stream_ = nullptr;
    DeviceBuffer i8_x_, i8_scale_, i8_sum_, q8_, attn_q_, attn_k_, attn_vt_;
    size_t m_ = 0, cols_ = 0, q8_total_ = 0;
    int bits_ = 0;
    size_t w4_reserved_ = 0;
    WeightCache<DeviceBuffer> weights_{
        [this](const void *host, size_t bytes) {
            DeviceBuffer db = tensorCreate(bytes);
            cuda(cudaMemcpyAsync(db.p, host, bytes, cudaMemcpyHostToDevice, stream_), "cachedWeight upload");
            return db;
        },
        [](DeviceBuffer &db) { release(db); }};
};

}  // namespace tpb

#endif  // TPB200_HPP
