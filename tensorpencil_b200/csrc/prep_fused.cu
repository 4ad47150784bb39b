// The elementwise neighbours of the quantized linears in the DiT block, and the
// activation prep with those producers fused in (kernel in prep_common.cuh).
//
//   silu_mul     a = silu(a) * b          before mlp.down   src/gpu/cuda/backend.zig:3310-3315, src/ops/act.zig:61-70
//   sigmoid_mul  a = a * sigmoid(b)       before attn.wo    src/gpu/cuda/backend.zig:3294-3299, src/ops/act.zig:141-149
//   rms_mod      out = x*inv*premul+shift before q/k/v/gate and mlp.gate/up
//                                                           src/gpu/cuda/backend.zig:2738-2760, src/gpu/cuda/elt.zig:9-66
//   gated_add    x += gate[c] * delta     after wo / mlp.down
//                                                           src/gpu/cuda/backend.zig:3342-3347, src/models/dit.zig:584-590
//
// All of them are HBM-bound.  Stand-alone they move 12 bytes per element (two reads and a
// write, f32); fused into the prep the producer's output is never written, which at the
// mlp.down shape (2048..4608 x 12288) saves a 226 MB write and a 226 MB read per call.
#include "prep_common.cuh"

using namespace tpb_prep;

namespace {

template <typename T, int OP>
__global__ void __launch_bounds__(256) gate_mul_kernel(const T *a, const T *b, float *out, size_t n4) {
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n4; c += (size_t)gridDim.x * blockDim.x) {
        float va[4], vb[4];
        load4<T>(a + 4 * c, va);
        load4<T>(b + 4 * c, vb);
        float4 r;
        if (OP == OP_SILU_MUL) {
            r.x = (va[0] * sigmoid_fast(va[0])) * vb[0];
            r.y = (va[1] * sigmoid_fast(va[1])) * vb[1];
            r.z = (va[2] * sigmoid_fast(va[2])) * vb[2];
            r.w = (va[3] * sigmoid_fast(va[3])) * vb[3];
        } else {
            r.x = va[0] * sigmoid_fast(vb[0]);
            r.y = va[1] * sigmoid_fast(vb[1]);
            r.z = va[2] * sigmoid_fast(vb[2]);
            r.w = va[3] * sigmoid_fast(vb[3]);
        }
        reinterpret_cast<float4 *>(out)[c] = r;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) gated_add_kernel(float *x, const T *delta, const float *gate, size_t n4,
                                                         int dim4) {
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n4; c += (size_t)gridDim.x * blockDim.x) {
        float d[4];
        load4<T>(delta + 4 * c, d);
        const float4 g = __ldcg(reinterpret_cast<const float4 *>(gate) + (c % (size_t)dim4));
        float4 v = reinterpret_cast<float4 *>(x)[c];
        v.x = __fmaf_rn(g.x, d[0], v.x);
        v.y = __fmaf_rn(g.y, d[1], v.y);
        v.z = __fmaf_rn(g.z, d[2], v.z);
        v.w = __fmaf_rn(g.w, d[3], v.w);
        reinterpret_cast<float4 *>(x)[c] = v;
    }
}

unsigned elementwise_grid(tpb_handle_t h, size_t n4) {
    const size_t want = (n4 + 255) / 256;
    const size_t cap = (size_t)h->sm_count * 16;
    return (unsigned)(want < cap ? (want ? want : 1) : cap);
}

template <typename T>
int launch_fused_t(tpb_handle_t h, cudaStream_t st, int op, const PrepParams &P, int64_t m, int64_t k, int bits,
                   bool act_only) {
    switch (op) {
        case OP_SILU_MUL: return launch_prep_op<T, OP_SILU_MUL, false>(h, st, P, m, k, bits);
        case OP_SIGMOID_MUL: return launch_prep_op<T, OP_SIGMOID_MUL, false>(h, st, P, m, k, bits);
        case OP_RMS_MOD:
            return act_only ? launch_prep_op<T, OP_RMS_MOD, true>(h, st, P, m, k, bits)
                            : launch_prep_op<T, OP_RMS_MOD, false>(h, st, P, m, k, bits);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "prep_fused: unknown op %d", op);
}

int launch_fused(tpb_handle_t h, cudaStream_t st, int op, int dtype, const PrepParams &P, int64_t m, int64_t k,
                 int bits, bool act_only) {
    switch (dtype) {
        case TPB_F32: return launch_fused_t<float>(h, st, op, P, m, k, bits, act_only);
        case TPB_BF16: return launch_fused_t<__nv_bfloat16>(h, st, op, P, m, k, bits, act_only);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "prep_fused: inputs must be f32 or bf16 (got dtype %d)", dtype);
}

}  // namespace

extern "C" {

int tpb_convrot_prep_fused(tpb_handle_t h, tpb_stream_t stream, int op, const void *a, const void *b,
                           const float *premul, const float *shift, float eps, int in_dtype, int64_t m,
                           int64_t k, int bits, int8_t *q, float *act_scale, int32_t *act_sum) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, op == OP_SILU_MUL || op == OP_SIGMOID_MUL || op == OP_RMS_MOD,
                  "prep_fused: op must be 1 (silu_mul), 2 (sigmoid_mul) or 3 (rms_mod)");
    TPB_CHECK_ARG(h, a && q && act_scale, "prep_fused: null pointer");
    TPB_CHECK_ARG(h, op == OP_RMS_MOD ? (premul && shift) : (b != nullptr),
                  "prep_fused: op %d is missing its second input", op);
    TPB_CHECK_ARG(h, bits == 8 || bits == 4, "prep_fused: bits must be 8 or 4 (got %d)", bits);
    TPB_CHECK_ARG(h, bits == 8 || act_sum, "prep_fused: act_sum is required when bits = 4");
    TPB_CHECK_ARG(h, m >= 0 && k > 0 && k % 256 == 0 && k <= 32768,
                  "prep_fused: k must be a multiple of 256, at most 32768 (k=%lld)", (long long)k);
    TPB_CHECK_ARG(h, tpb_aligned16(a) && tpb_aligned16(b) && tpb_aligned16(q) && tpb_aligned16(premul) &&
                         tpb_aligned16(shift),
                  "prep_fused: pointers must be 16-byte aligned");
    if (m == 0) return TPB_OK;
    PrepParams P = {};
    P.a = a;
    P.b = b;
    P.premul = premul;
    P.shift = shift;
    P.eps = eps;
    P.q = q;
    P.act_scale = act_scale;
    P.act_sum = act_sum;
    return launch_fused(h, (cudaStream_t)stream, op, in_dtype, P, m, k, bits, false);
}

int tpb_rms_mod(tpb_handle_t h, tpb_stream_t stream, const void *x, int x_dtype, float *out, const float *premul,
                const float *shift, float eps, int64_t rows, int64_t dim) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, x && out && premul && shift, "rms_mod: null pointer");
    TPB_CHECK_ARG(h, rows >= 0 && dim > 0 && dim % 256 == 0 && dim <= 32768,
                  "rms_mod: dim must be a multiple of 256, at most 32768 (dim=%lld)", (long long)dim);
    TPB_CHECK_ARG(h, tpb_aligned16(x) && tpb_aligned16(out) && tpb_aligned16(premul) && tpb_aligned16(shift),
                  "rms_mod: pointers must be 16-byte aligned");
    if (rows == 0) return TPB_OK;
    PrepParams P = {};
    P.a = x;
    P.premul = premul;
    P.shift = shift;
    P.eps = eps;
    P.act_out = out;
    return launch_fused(h, (cudaStream_t)stream, OP_RMS_MOD, x_dtype, P, rows, dim, 8, true);
}

static int gate_mul(tpb_handle_t h, tpb_stream_t stream, int op, const void *a, const void *b, int dtype,
                    float *out, int64_t n, const char *name) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, a && b && out, "%s: null pointer", name);
    TPB_CHECK_ARG(h, n >= 0 && n % 4 == 0, "%s: n must be a multiple of 4", name);
    TPB_CHECK_ARG(h, tpb_aligned16(a) && tpb_aligned16(b) && tpb_aligned16(out), "%s: pointers must be 16-byte aligned",
                  name);
    TPB_CHECK_ARG(h, dtype == TPB_F32 || dtype == TPB_BF16, "%s: inputs must be f32 or bf16", name);
    if (n == 0) return TPB_OK;
    const size_t n4 = (size_t)n / 4;
    const dim3 grid(elementwise_grid(h, n4)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == TPB_F32) {
        e = op == OP_SILU_MUL
                ? tpb_launch_pdl(gate_mul_kernel<float, OP_SILU_MUL>, grid, block, 0, st, (const float *)a, (const float *)b, out, n4)
                : tpb_launch_pdl(gate_mul_kernel<float, OP_SIGMOID_MUL>, grid, block, 0, st, (const float *)a, (const float *)b, out, n4);
    } else {
        e = op == OP_SILU_MUL
                ? tpb_launch_pdl(gate_mul_kernel<__nv_bfloat16, OP_SILU_MUL>, grid, block, 0, st, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, out, n4)
                : tpb_launch_pdl(gate_mul_kernel<__nv_bfloat16, OP_SIGMOID_MUL>, grid, block, 0, st, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, out, n4);
    }
    TPB_CUDA(h, e);
    return TPB_OK;
}

int tpb_silu_mul(tpb_handle_t h, tpb_stream_t stream, const void *gate, const void *up, int in_dtype, float *out,
                 int64_t n) {
    return gate_mul(h, stream, OP_SILU_MUL, gate, up, in_dtype, out, n, "silu_mul");
}

int tpb_sigmoid_mul(tpb_handle_t h, tpb_stream_t stream, const void *a, const void *gate, int in_dtype, float *out,
                    int64_t n) {
    return gate_mul(h, stream, OP_SIGMOID_MUL, a, gate, in_dtype, out, n, "sigmoid_mul");
}

int tpb_gated_add(tpb_handle_t h, tpb_stream_t stream, float *x, const void *delta, int delta_dtype,
                  const float *gate, int64_t rows, int64_t dim) {
    if (!h) return TPB_ERR_INVALID_ARG;
    TPB_CHECK_ARG(h, x && delta && gate, "gated_add: null pointer");
    TPB_CHECK_ARG(h, rows >= 0 && dim > 0 && dim % 4 == 0, "gated_add: dim must be a multiple of 4");
    TPB_CHECK_ARG(h, tpb_aligned16(x) && tpb_aligned16(delta) && tpb_aligned16(gate),
                  "gated_add: pointers must be 16-byte aligned");
    TPB_CHECK_ARG(h, delta_dtype == TPB_F32 || delta_dtype == TPB_BF16, "gated_add: delta must be f32 or bf16");
    if (rows == 0) return TPB_OK;
    const size_t n4 = (size_t)rows * (size_t)dim / 4;
    const dim3 grid(elementwise_grid(h, n4)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    const cudaError_t e =
        delta_dtype == TPB_F32
            ? tpb_launch_pdl(gated_add_kernel<float>, grid, block, 0, st, x, (const float *)delta, gate, n4, (int)(dim / 4))
            : tpb_launch_pdl(gated_add_kernel<__nv_bfloat16>, grid, block, 0, st, x, (const __nv_bfloat16 *)delta, gate, n4, (int)(dim / 4));
    TPB_CUDA(h, e);
    return TPB_OK;
}

}  // extern "C"
