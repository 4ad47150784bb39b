// ConvRot activation prep for sm_100a: block Hadamard rotation + per-token
// absmax quantisation in one pass over the activations (HBM-bound: reads
// sizeof(x)*m*k, writes m*k + 8*m bytes).
//
// Arithmetic contract (bit-exact with the CPU replica the reference's own GPU
// tests compare against, src/gpu/cuda/kernels.zig:2638-2653 and :2487-2502):
//   rotation  : radix-4 FWHT per 256-group, passes at strides 1,4,16,64 in
//               that order, each output ((a+b)+c)-d, ((a+b)-c)+d, ((a-b)+c)+d,
//               ((-a+b)+c)+d, then /16            (src/ops/convrot.zig:56-78)
//   scale     : s = max(absmax / maxq, 1e-12)     IEEE division
//   quantise  : q = round-half-away(v / s)        IEEE division
//
// Work split: one CTA per token row; a half-warp owns one 256-group, a lane
// holds 16 of its elements.  Writing the element index as bits e7..e0, a radix-4
// pass over base-4 digit d needs both bits of d inside one lane's registers:
//   layout A  registers {e0,e1,e6,e7}, lane {e2..e5}: four coalesced 16-byte
//             global loads; passes d0 (stride 1) and d3 (stride 64) are local;
//   layout B  registers {e2,e3,e4,e5}, lane {e0,e1,e6,e7}: passes d1 (stride 4)
//             and d2 (stride 16) are local.
// The pass order 1,4,16,64 therefore runs A -> B -> A, and the two layout changes
// go through a warp-private shared-memory tile (272 words per group: 4 pad words
// after every 64 so that both layouts are bank-conflict free); only __syncwarp is
// needed.  Back in layout A the int8 results leave as 32-bit stores of four
// consecutive elements.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tpb_internal.h"

namespace {

constexpr int kMaxWarps = 8;

// One 4-point regular-Hadamard butterfly with the reference's association.
// (-a + b) is computed as -(a - b), which is the same float.
__device__ __forceinline__ void hadamard4(float &a, float &b, float &c, float &d) {
    const float s = a + b;
    const float t = a - b;
    const float o0 = (s + c) - d;
    const float o1 = (s - c) + d;
    const float o2 = (t + c) + d;
    const float o3 = (c - t) + d;
    a = o0;
    b = o1;
    c = o2;
    d = o3;
}

constexpr int kGroupWords = 272;  // 256 data words + 4 pad words per 64

__device__ __forceinline__ void lds128(float (&v)[4], const float *p) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void sts128(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}

// Un-normalised H*v of one 256-group spread over a half-warp.  `tile` is this
// half-warp's 272-word shared tile; element e lives at word e + 4*(e >> 6).
__device__ __forceinline__ void rotate_group(float (&v)[4][4], float *tile, int l16) {
#pragma unroll
    for (int i = 0; i < 4; i++) hadamard4(v[i][0], v[i][1], v[i][2], v[i][3]);  // stride 1
    // layout A -> shared: chunk c = l16 + 16 i (4 elements) at word 4c + 4i
    float *a_ptr = tile + 4 * l16;
#pragma unroll
    for (int i = 0; i < 4; i++) sts128(a_ptr + 68 * i, v[i]);
    __syncwarp();
    // layout B: element (l16 & 3) + 4 r + 64 (l16 >> 2), r = 0..15
    float *b_ptr = tile + (l16 & 3) + 68 * (l16 >> 2);
    float u[16];
#pragma unroll
    for (int r = 0; r < 16; r++) u[r] = b_ptr[4 * r];
#pragma unroll
    for (int hi = 0; hi < 4; hi++) hadamard4(u[4 * hi], u[4 * hi + 1], u[4 * hi + 2], u[4 * hi + 3]);  // stride 4
#pragma unroll
    for (int lo = 0; lo < 4; lo++) hadamard4(u[lo], u[lo + 4], u[lo + 8], u[lo + 12]);  // stride 16
#pragma unroll
    for (int r = 0; r < 16; r++) b_ptr[4 * r] = u[r];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; i++) lds128(v[i], a_ptr + 68 * i);
    __syncwarp();  // the tile is reused by this half-warp's next group
#pragma unroll
    for (int j = 0; j < 4; j++) hadamard4(v[0][j], v[1][j], v[2][j], v[3][j]);  // stride 64
}

template <typename T>
__device__ __forceinline__ void load4(const T *p, float (&out)[4]);

template <>
__device__ __forceinline__ void load4<float>(const float *p, float (&out)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__half>(const __half *p, float (&out)[4]) {
    const uint2 t = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&t.y));
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16 *p, float (&out)[4]) {
    const uint2 t = __ldg(reinterpret_cast<const uint2 *>(p));
    out[0] = __uint_as_float(t.x << 16);
    out[1] = __uint_as_float(t.x & 0xffff0000u);
    out[2] = __uint_as_float(t.y << 16);
    out[3] = __uint_as_float(t.y & 0xffff0000u);
}

constexpr float kRoundMagic = 12582912.0f;  // 1.5 * 2^23: adding it leaves rint(x) in the low mantissa bits

// PPW = group pairs per warp (compile time, sizes the register file use).
template <typename T, int PPW>
__global__ void __launch_bounds__(kMaxWarps * 32)
convrot_prep_kernel(const T *__restrict__ x, int8_t *__restrict__ q, float *__restrict__ act_scale,
                    int32_t *__restrict__ act_sum, int k, int n_groups, float maxq) {
    __shared__ float s_max[kMaxWarps];
    __shared__ int s_sum[kMaxWarps];
    __shared__ __align__(16) float s_tile[kMaxWarps][2][kGroupWords];

    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5;
    const int n_warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int hw = lane >> 4;
    const int l16 = lane & 15;
    const T *xrow = x + (size_t)row * k;
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();

    float v[PPW][4][4];
    float amax = 0.0f;
#pragma unroll
    for (int p = 0; p < PPW; p++) {
        const int g = 2 * (warp + p * n_warps) + hw;
        const bool live = g < n_groups;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (live) {
                load4<T>(xrow + g * 256 + 4 * (l16 + 16 * i), v[p][i]);
            } else {
                v[p][i][0] = v[p][i][1] = v[p][i][2] = v[p][i][3] = 0.0f;
            }
        }
    }
#pragma unroll
    for (int p = 0; p < PPW; p++) {
        rotate_group(v[p], s_tile[warp][hw], l16);
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) amax = fmaxf(amax, fabsf(v[p][i][j]));
    }

    // Row absmax: warp butterfly, then across the CTA's warps.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) s_max[warp] = amax;
    __syncthreads();
    amax = s_max[0];
    for (int w = 1; w < n_warps; w++) amax = fmaxf(amax, s_max[w]);

    // The values above are 16x the rotated ones; /16 is exact, so the absmax of
    // the rotated row is amax/16 and v/16/s == v/(16 s) as correctly rounded floats.
    const float s = fmaxf(__fdiv_rn(amax * 0.0625f, maxq), 1e-12f);
    const float s16 = s * 16.0f;
    const float rcp = __frcp_rn(s16);
    if (threadIdx.x == 0) act_scale[row] = s;

    int isum = 0;
#pragma unroll
    for (int p = 0; p < PPW; p++) {
        const int g = 2 * (warp + p * n_warps) + hw;
        const bool live = g < n_groups;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t yb[4];
            // Fast path: v*rcp is within 2e-5 of the IEEE quotient for |q| <= 128, so
            // unless it sits within 1e-4 of a half-integer, rounding it to nearest gives
            // round-half-away(v / s) exactly.  y = rint(v*rcp) + magic in one FMA; the
            // distance of v*rcp from that integer in a second one.
            float y[4];
            bool near_tie = false;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                y[j] = __fmaf_rn(v[p][i][j], rcp, kRoundMagic);
                const float diff = __fmaf_rn(v[p][i][j], rcp, -(y[j] - kRoundMagic));
                near_tie |= fabsf(diff) > 0.4999f;
            }
            if (near_tie) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float t = __fdiv_rn(v[p][i][j] * 0.0625f, s);
                    y[j] = roundf(t) + kRoundMagic;  // half away from zero, exact
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) yb[j] = __float_as_uint(y[j]);
            const uint32_t lo = __byte_perm(yb[0], yb[1], 0x0040);
            const uint32_t hi = __byte_perm(yb[2], yb[3], 0x0040);
            const uint32_t word = __byte_perm(lo, hi, 0x5410);
            isum = __dp4a((int)word, 0x01010101, isum);
            if (live) {
                const int chunk = l16 + 16 * i;
                *reinterpret_cast<uint32_t *>(q + (size_t)row * k + g * 256 + 4 * chunk) = word;
            }
        }
    }
    if (act_sum != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
        if (lane == 0) s_sum[warp] = isum;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < n_warps; w++) t += s_sum[w];
            act_sum[row] = t;
        }
    }
}

// int4 -> int8 expansion of a packed weight: 16 packed bytes in, 32 bytes out.
__global__ void __launch_bounds__(256)
w4_expand_kernel(const uint4 *__restrict__ w4, uint4 *__restrict__ w8, size_t n_chunks) {
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks;
         c += (size_t)gridDim.x * blockDim.x) {
        const uint4 p = __ldg(w4 + c);
        const uint32_t in[4] = {p.x, p.y, p.z, p.w};
        uint32_t out[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // even nibbles -> bytes (n0,n2,n4,n6), odd -> (n1,n3,n5,n7); sign-extend
            // each nibble inside its byte: x | ((x & 8) * 30) sets bits 4..7.
            uint32_t e = in[i] & 0x0f0f0f0fu;
            uint32_t o = (in[i] >> 4) & 0x0f0f0f0fu;
            e |= (e & 0x08080808u) * 30u;
            o |= (o & 0x08080808u) * 30u;
            out[2 * i] = __byte_perm(e, o, 0x5140);      // n0 n1 n2 n3
            out[2 * i + 1] = __byte_perm(e, o, 0x7362);  // n4 n5 n6 n7
        }
        w8[2 * c] = make_uint4(out[0], out[1], out[2], out[3]);
        w8[2 * c + 1] = make_uint4(out[4], out[5], out[6], out[7]);
    }
}

template <typename T>
int launch_prep_t(tpb_handle_t h, cudaStream_t st, const T *x, int64_t m, int64_t k, int bits,
                  int8_t *q, float *act_scale, int32_t *act_sum) {
    const int n_groups = (int)(k / 256);
    const int n_pairs = (n_groups + 1) / 2;
    int ppw = (n_pairs + kMaxWarps - 1) / kMaxWarps;
    // round PPW up to an instantiated value
    static const int kPpw[] = {1, 2, 3, 4, 6, 8};
    int ppw_inst = 8;
    for (int c : kPpw)
        if (c >= ppw) {
            ppw_inst = c;
            break;
        }
    const int warps = (n_pairs + ppw_inst - 1) / ppw_inst;
    const dim3 grid((unsigned)m), block(warps * 32);
    const float maxq = bits == 4 ? 7.0f : 127.0f;
    cudaError_t err = cudaSuccess;
#define TPB_PREP_CASE(P)                                                                          \
    case P:                                                                                       \
        err = tpb_launch_pdl(convrot_prep_kernel<T, P>, grid, block, 0, st, x, q, act_scale, act_sum, (int)k, n_groups, maxq); \
        break;
    switch (ppw_inst) {
        TPB_PREP_CASE(1)
        TPB_PREP_CASE(2)
        TPB_PREP_CASE(3)
        TPB_PREP_CASE(4)
        TPB_PREP_CASE(6)
        TPB_PREP_CASE(8)
    }
#undef TPB_PREP_CASE
    TPB_CUDA(h, err);
    return TPB_OK;
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
