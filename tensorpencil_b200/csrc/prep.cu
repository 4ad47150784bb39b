// Plain ConvRot activation prep (x already in memory) and the int4 -> int8 weight
// expansion.  The kernel itself is in prep_common.cuh.
#include "prep_common.cuh"

using namespace tpb_prep;

namespace {

// int4 -> int8 expansion of a packed weight: 16 packed bytes in, 32 bytes out.
__global__ void __launch_bounds__(256)
w4_expand_kernel(const uint4 *__restrict__ w4, uint4 *__restrict__ w8, size_t n_chunks) {
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks;
         c += (size_t)gridDim.x * blockDim.x)
        w4_expand_chunk(w4, w8, c);
}

template <typename T>
int launch_prep_t(tpb_handle_t h, cudaStream_t st, const T *x, int64_t m, int64_t k, int bits,
                  int8_t *q, float *act_scale, int32_t *act_sum) {
    PrepParams P = {};
    P.a = x;
    P.q = q;
    P.act_scale = act_scale;
    P.act_sum = act_sum;
    return launch_prep_op<T, OP_PLAIN, false>(h, st, P, m, k, bits);
}

}  // namespace

int tpb_launch_prep(tpb_handle_t h, cudaStream_t st, const void *x, int x_dtype, int64_t m,
                    int64_t k, int bits, int8_t *q, float *act_scale, int32_t *act_sum) {
    switch (x_dtype) {
        case TPB_F32:
            return launch_prep_t<float>(h, st, (const float *)x, m, k, bits, q, act_scale, act_sum);
        case TPB_F16:
            return launch_prep_t<__half>(h, st, (const __half *)x, m, k, bits, q, act_scale, act_sum);
        case TPB_BF16:
            return launch_prep_t<__nv_bfloat16>(h, st, (const __nv_bfloat16 *)x, m, k, bits, q,
                                                act_scale, act_sum);
    }
    return tpb_fail(h, TPB_ERR_INVALID_ARG, "prep: unsupported x_dtype %d", x_dtype);
}

int tpb_launch_w4_expand(tpb_handle_t h, cudaStream_t st, const void *w4, int64_t n, int64_t k,
                         int8_t *w8) {
    const size_t n_chunks = (size_t)n * (size_t)k / 32;  // 16 packed bytes each
    const int block = 256;
    size_t want = (n_chunks + block - 1) / block;
    const size_t cap = (size_t)h->sm_count * 16;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    TPB_CUDA(h, tpb_launch_pdl(w4_expand_kernel, dim3(grid), dim3(block), 0, st, (const uint4 *)w4, (uint4 *)w8, n_chunks));
    return TPB_OK;
}
