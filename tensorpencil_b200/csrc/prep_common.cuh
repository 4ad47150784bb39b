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
// Work split: one CTA per token row; a half-warp owns a PAIR of adjacent 256-groups
// and a lane holds 16 elements of each, element e of the first group packed with
// element e of the second in one 64-bit register pair.  All rotation and quantiser
// arithmetic then runs on Blackwell's two-wide f32 instructions (add/sub/fma.rn.f32x2:
// IEEE results per half, so nothing changes numerically) -- the kernel is bound by
// instruction issue, not by HBM, and this halves its floating-point instruction count.
// Writing the element index as bits e7..e0, a radix-4 pass over base-4 digit d needs
// both bits of d inside one lane's registers:
//   layout A  registers {e0,e1,e6,e7}, lane {e2..e5}: four coalesced 16-byte
//             global loads per group; passes d0 (stride 1) and d3 (stride 64) are local;
//   layout B  registers {e2,e3,e4,e5}, lane {e0,e1,e6,e7}: passes d1 (stride 4)
//             and d2 (stride 16) are local.
// The pass order 1,4,16,64 therefore runs A -> B -> A, and the two layout changes
// go through a half-warp-private shared-memory tile of packed pairs: slot
// lane_A + 18 * lane_B (8 bytes each), so layout A moves 64-bit words that are
// contiguous across lanes and layout B moves 128-bit words at a 144-byte lane pitch,
// both bank-conflict free; only __syncwarp is needed.  Back in layout A the int8
// results leave as 32-bit stores of four consecutive elements.
//
// Producers.  The reference computes the prep's input with a separate elementwise
// kernel (silu(gate)*up before mlp.down, attn*sigmoid(gate) before wo, RMS norm +
// AdaLN modulation before q/k/v/gate and mlp.gate/up; src/models/dit_cuda.zig:473-514)
// and writes it to memory first.  The kernel below takes the producer as a template
// parameter and applies it to the values as they are loaded, so the f32 activation
// never makes the round trip through HBM.  ACT_ONLY stops after the producer and
// stores its f32 result: the stand-alone form of the same op, bit-identical to what
// the fused form feeds the rotation (same instructions, same reduction order).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tpb_internal.h"

namespace tpb_prep {

enum PrepOp { OP_PLAIN = 0, OP_SILU_MUL = 1, OP_SIGMOID_MUL = 2, OP_RMS_MOD = 3 };

struct PrepParams {
    const void *a;        // x | gate (silu_mul) | attention output (sigmoid_mul) | residual stream (rms_mod)
    const void *b;        // - | up              | gate                           | -
    const float *premul;  // rms_mod: per-column multiplier ((1 + scale) * norm weight)
    const float *shift;   // rms_mod: per-column shift
    float eps;            // rms_mod
    float *act_out;       // ACT_ONLY: f32 [m][k] result of the producer
    int8_t *q;
    float *act_scale;
    int32_t *act_sum;
    int m, k, n_groups;
    float maxq;
};

// 16 packed int4 bytes -> 32 int8 bytes (element 2j in the low nibble, src/core/dtype.zig:146-149)
__device__ __forceinline__ void w4_expand_chunk(const uint4 *__restrict__ w4, uint4 *__restrict__ w8, size_t c) {
    const uint4 p = __ldcg(w4 + c);
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


constexpr int kMaxWarps = 8;
constexpr int kMaxWarpsWide = 16;
#ifndef TPB_F32_LOAD_FIRST
#define TPB_F32_LOAD_FIRST 1
#endif
constexpr bool kF32LoadFirst = TPB_F32_LOAD_FIRST != 0;   // rows of the gated preps: one unit per half-warp, more warps per row
constexpr int kTilePairs = 16 * 18;  // 64-bit slots of one half-warp's tile (2304 bytes)

// Two packed f32 values; every operation rounds each half like the scalar instruction.
typedef unsigned long long f2;
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
    f2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 sub2(f2 a, f2 b) {
    f2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f2 pack2(float lo, float hi) {
    f2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack2(f2 v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// One 4-point regular-Hadamard butterfly with the reference's association, on two
// independent groups at once.  (-a + b) is computed as -(a - b), which is the same float.
__device__ __forceinline__ void hadamard4(f2 &a, f2 &b, f2 &c, f2 &d) {
    const f2 s = add2(a, b);
    const f2 t = sub2(a, b);
    const f2 o0 = sub2(add2(s, c), d);
    const f2 o1 = add2(sub2(s, c), d);
    const f2 o2 = add2(add2(t, c), d);
    const f2 o3 = add2(sub2(c, t), d);
    a = o0;
    b = o1;
    c = o2;
    d = o3;
}

// Un-normalised H*v of a pair of 256-groups spread over a half-warp.  `tile` is this
// half-warp's shared tile; element e = 4*(lane_A + 16 i) + j lives in slot
// lane_A + 18*(j + 4 i).
__device__ __forceinline__ void rotate_unit(f2 (&v)[4][4], f2 *tile, int l16) {
#pragma unroll
    for (int i = 0; i < 4; i++) hadamard4(v[i][0], v[i][1], v[i][2], v[i][3]);  // stride 1
    f2 *a_ptr = tile + l16;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) a_ptr[18 * (j + 4 * i)] = v[i][j];
    __syncwarp();
    // layout B: this lane is (j, i) = (l16 & 3, l16 >> 2) and reads lane_A = 0..15
    ulonglong2 *b_ptr = reinterpret_cast<ulonglong2 *>(tile + 18 * l16);
    f2 u[16];
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const ulonglong2 t = b_ptr[r];
        u[2 * r] = t.x;
        u[2 * r + 1] = t.y;
    }
#pragma unroll
    for (int hi = 0; hi < 4; hi++) hadamard4(u[4 * hi], u[4 * hi + 1], u[4 * hi + 2], u[4 * hi + 3]);  // stride 4
#pragma unroll
    for (int lo = 0; lo < 4; lo++) hadamard4(u[lo], u[lo + 4], u[lo + 8], u[lo + 12]);  // stride 16
#pragma unroll
    for (int r = 0; r < 8; r++) b_ptr[r] = make_ulonglong2(u[2 * r], u[2 * r + 1]);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) v[i][j] = a_ptr[18 * (j + 4 * i)];
    __syncwarp();  // the tile is reused by this half-warp's next unit
#pragma unroll
    for (int j = 0; j < 4; j++) hadamard4(v[0][j], v[1][j], v[2][j], v[3][j]);  // stride 64
}

template <typename T>
__device__ __forceinline__ void load4(const T *p, float (&out)[4]);

template <>
__device__ __forceinline__ void load4<float>(const float *p, float (&out)[4]) {
    const float4 t = __ldcg(reinterpret_cast<const float4 *>(p));
    out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__half>(const __half *p, float (&out)[4]) {
    const uint2 t = __ldcg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&t.y));
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16 *p, float (&out)[4]) {
    const uint2 t = __ldcg(reinterpret_cast<const uint2 *>(p));
    out[0] = __uint_as_float(t.x << 16);
    out[1] = __uint_as_float(t.x & 0xffff0000u);
    out[2] = __uint_as_float(t.y << 16);
    out[3] = __uint_as_float(t.y & 0xffff0000u);
}


// The same four values kept as loaded (8 or 16 bytes), converted later: lets a thread put all the
// loads of a unit in flight before the first value is used.
template <typename T>
struct Raw4 {
    uint2 r;
};
template <>
struct Raw4<float> {
    float4 r;
};
template <typename T>
__device__ __forceinline__ Raw4<T> load_raw(const T *p) {
    Raw4<T> v;
    v.r = __ldcg(reinterpret_cast<const uint2 *>(p));
    return v;
}
template <>
__device__ __forceinline__ Raw4<float> load_raw<float>(const float *p) {
    Raw4<float> v;
    v.r = __ldcg(reinterpret_cast<const float4 *>(p));
    return v;
}
__device__ __forceinline__ void raw_to_f4(const Raw4<float> &v, float (&out)[4]) {
    out[0] = v.r.x; out[1] = v.r.y; out[2] = v.r.z; out[3] = v.r.w;
}
__device__ __forceinline__ void raw_to_f4(const Raw4<__half> &v, float (&out)[4]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v.r.y));
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
__device__ __forceinline__ void raw_to_f4(const Raw4<__nv_bfloat16> &v, float (&out)[4]) {
    out[0] = __uint_as_float(v.r.x << 16);
    out[1] = __uint_as_float(v.r.x & 0xffff0000u);
    out[2] = __uint_as_float(v.r.y << 16);
    out[3] = __uint_as_float(v.r.y & 0xffff0000u);
}

// sigmoid(x) = 1 / (1 + exp(-x)) with the fast exponential and reciprocal (the reference's
// GPU kernels use ex2.approx + rcp.approx for it too, src/gpu/cuda/elt.zig:4-7).
__device__ __forceinline__ float sigmoid_fast(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}

constexpr float kRoundMagic = 12582912.0f;  // 1.5 * 2^23: adding it leaves rint(x) in the low mantissa bits

// UPW = units (pairs of groups) per half-warp (compile time, sizes the register file use).
// ONE_WARP: the row fits one warp (k <= 1024): every warp of the CTA takes its own row and
// no CTA-wide barrier or shared reduction is needed; otherwise one row per CTA.
template <typename T, int UPW, int OP, bool ACT_ONLY, bool ONE_WARP>
__global__ void __launch_bounds__((UPW == 1 ? kMaxWarpsWide : kMaxWarps) * 32)
convrot_prep_kernel(const PrepParams P) {
    __shared__ float s_max[kMaxWarpsWide];
    __shared__ int s_sum[kMaxWarpsWide];
    extern __shared__ __align__(16) unsigned char s_dyn[];

    const int cta_warp = threadIdx.x >> 5;
    const int row = ONE_WARP ? blockIdx.x * (blockDim.x >> 5) + cta_warp : blockIdx.x;
    const int warp = ONE_WARP ? 0 : cta_warp;                 // this warp's index within its row
    const int n_warps = ONE_WARP ? 1 : (blockDim.x >> 5);     // warps sharing the row
    const int lane = threadIdx.x & 31;
    const int hw = lane >> 4;
    const int l16 = lane & 15;
    const int k = P.k, n_groups = P.n_groups;
    f2 *tile = reinterpret_cast<f2 *>(s_dyn) + (size_t)(2 * cta_warp + hw) * kTilePairs;
    if (ONE_WARP && row >= P.m) return;
    const T *arow = static_cast<const T *>(P.a) + (size_t)row * k;
    const T *brow = static_cast<const T *>(P.b) + (size_t)row * k;
    tpb_grid_dep_launch();
    tpb_grid_dep_wait();

    f2 v[UPW][4][4];
    float sumsq = 0.0f;
#pragma unroll
    for (int p = 0; p < UPW; p++) {
        const int g0 = 2 * ((2 * warp + hw) + p * 2 * n_warps);
        if ((OP == OP_SILU_MUL || OP == OP_SIGMOID_MUL) && sizeof(T) == 2) {
            // two operands per element and a sigmoid between load and use: with 16-bit inputs all sixteen
            // loads of the unit go out first, the arithmetic follows (same operations, same order per
            // element); with f32 inputs the raw values would double the live registers and the
            // interleaved order below measured faster
            Raw4<T> ra[4][2], rb[4][2];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int h = 0; h < 2; h++)
                    if (g0 + h < n_groups) {
                        const int off = (g0 + h) * 256 + 4 * (l16 + 16 * i);
                        ra[i][h] = load_raw<T>(arow + off);
                        rb[i][h] = load_raw<T>(brow + off);
                    }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float x[2][4];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (g0 + h < n_groups) {
                        float u[4];
                        raw_to_f4(ra[i][h], x[h]);
                        raw_to_f4(rb[i][h], u);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            x[h][j] = OP == OP_SILU_MUL ? (x[h][j] * sigmoid_fast(x[h][j])) * u[j] : x[h][j] * sigmoid_fast(u[j]);
                    } else {
                        x[h][0] = x[h][1] = x[h][2] = x[h][3] = 0.0f;
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) v[p][i][j] = pack2(x[0][j], x[1][j]);
            }
            continue;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float x[2][4];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (g0 + h < n_groups) {
                    const int off = (g0 + h) * 256 + 4 * (l16 + 16 * i);
                    load4<T>(arow + off, x[h]);
                    if (OP == OP_SILU_MUL) {
                        float u[4];
                        load4<T>(brow + off, u);
#pragma unroll
                        for (int j = 0; j < 4; j++) x[h][j] = (x[h][j] * sigmoid_fast(x[h][j])) * u[j];
                    } else if (OP == OP_SIGMOID_MUL) {
                        float u[4];
                        load4<T>(brow + off, u);
#pragma unroll
                        for (int j = 0; j < 4; j++) x[h][j] = x[h][j] * sigmoid_fast(u[j]);
                    } else if (OP == OP_RMS_MOD) {
#pragma unroll
                        for (int j = 0; j < 4; j++) sumsq = __fmaf_rn(x[h][j], x[h][j], sumsq);
                    }
                } else {
                    x[h][0] = x[h][1] = x[h][2] = x[h][3] = 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) v[p][i][j] = pack2(x[0][j], x[1][j]);
        }
    }
    if (OP == OP_RMS_MOD) {
        // Row sum of squares: lane chains above, warp butterfly, then the warps in order.
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
        float tot = sumsq;
        if (!ONE_WARP) {
            if (lane == 0) s_max[warp] = sumsq;
            __syncthreads();
            tot = s_max[0];
            for (int w = 1; w < n_warps; w++) tot += s_max[w];
            __syncthreads();  // s_max is reused for the absmax below
        }
        const float inv = __frsqrt_rn(__fdiv_rn(tot, (float)k) + P.eps);
#pragma unroll
        for (int p = 0; p < UPW; p++) {
            const int g0 = 2 * ((2 * warp + hw) + p * 2 * n_warps);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float x[2][4];
#pragma unroll
                for (int j = 0; j < 4; j++) unpack2(v[p][i][j], x[0][j], x[1][j]);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (g0 + h < n_groups) {
                        const int off = (g0 + h) * 256 + 4 * (l16 + 16 * i);
                        // Plain loads: every row of the launch reads the same two vectors, so they are served
                        // from L1 after an SM's first row (past L1 they were 24 KB per row from L2, four times
                        // the bf16 row itself).  Coherent, and issued after griddepcontrol.wait: a kernel of the
                        // stream may have written them.
                        const float4 pm = *reinterpret_cast<const float4 *>(P.premul + off);
                        const float4 sh = *reinterpret_cast<const float4 *>(P.shift + off);
                        x[h][0] = __fmaf_rn(x[h][0] * inv, pm.x, sh.x);
                        x[h][1] = __fmaf_rn(x[h][1] * inv, pm.y, sh.y);
                        x[h][2] = __fmaf_rn(x[h][2] * inv, pm.z, sh.z);
                        x[h][3] = __fmaf_rn(x[h][3] * inv, pm.w, sh.w);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) v[p][i][j] = pack2(x[0][j], x[1][j]);
            }
        }
    }
    if (ACT_ONLY) {
#pragma unroll
        for (int p = 0; p < UPW; p++) {
            const int g0 = 2 * ((2 * warp + hw) + p * 2 * n_warps);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float x[2][4];
#pragma unroll
                for (int j = 0; j < 4; j++) unpack2(v[p][i][j], x[0][j], x[1][j]);
#pragma unroll
                for (int h = 0; h < 2; h++)
                    if (g0 + h < n_groups)
                        *reinterpret_cast<float4 *>(P.act_out + (size_t)row * k + (g0 + h) * 256 + 4 * (l16 + 16 * i)) =
                            make_float4(x[h][0], x[h][1], x[h][2], x[h][3]);
            }
        }
        return;
    }

    float amax = 0.0f;
#pragma unroll
    for (int p = 0; p < UPW; p++) {
        rotate_unit(v[p], tile, l16);
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float lo, hi;
                unpack2(v[p][i][j], lo, hi);
                amax = fmaxf(amax, fmaxf(fabsf(lo), fabsf(hi)));
            }
    }

    // Row absmax: warp butterfly, then across the CTA's warps.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!ONE_WARP) {
        if (lane == 0) s_max[warp] = amax;
        __syncthreads();
        amax = s_max[0];
        for (int w = 1; w < n_warps; w++) amax = fmaxf(amax, s_max[w]);
    }

    // The values above are 16x the rotated ones; /16 is exact, so the absmax of
    // the rotated row is amax/16 and v/16/s == v/(16 s) as correctly rounded floats.
    const float s = fmaxf(__fdiv_rn(amax * 0.0625f, P.maxq), 1e-12f);
    const float s16 = s * 16.0f;
    const float rcp = __frcp_rn(s16);
    if (warp == 0 && lane == 0) P.act_scale[row] = s;
    const f2 rcp2 = pack2(rcp, rcp);
    const f2 magic2 = pack2(kRoundMagic, kRoundMagic);

    int isum = 0;
#pragma unroll
    for (int p = 0; p < UPW; p++) {
        const int g0 = 2 * ((2 * warp + hw) + p * 2 * n_warps);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // Fast path: v*rcp is within 2e-5 of the IEEE quotient for |q| <= 128, so
            // unless it sits within 1e-4 of a half-integer, rounding it to nearest gives
            // round-half-away(v / s) exactly.  y = rint(v*rcp) + magic in one FMA; the
            // distance of v*rcp from that integer in a second one.
            f2 y[4];
            float tie = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                y[j] = fma2(v[p][i][j], rcp2, magic2);
                const f2 neg_int = sub2(magic2, y[j]);  // -(rint(v*rcp)), exact
                float dl, dh;
                unpack2(fma2(v[p][i][j], rcp2, neg_int), dl, dh);
                tie = fmaxf(tie, fmaxf(fabsf(dl), fabsf(dh)));
            }
            uint32_t yb[2][4];
            if (tie > 0.4999f) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float lo, hi;
                    unpack2(v[p][i][j], lo, hi);
                    // half away from zero, exact
                    yb[0][j] = __float_as_uint(roundf(__fdiv_rn(lo * 0.0625f, s)) + kRoundMagic);
                    yb[1][j] = __float_as_uint(roundf(__fdiv_rn(hi * 0.0625f, s)) + kRoundMagic);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    yb[0][j] = (uint32_t)y[j];
                    yb[1][j] = (uint32_t)(y[j] >> 32);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t lo = __byte_perm(yb[h][0], yb[h][1], 0x0040);
                const uint32_t hi = __byte_perm(yb[h][2], yb[h][3], 0x0040);
                const uint32_t word = __byte_perm(lo, hi, 0x5410);
                isum = __dp4a((int)word, 0x01010101, isum);
                if (g0 + h < n_groups) {
                    const int chunk = l16 + 16 * i;
                    *reinterpret_cast<uint32_t *>(P.q + (size_t)row * k + (g0 + h) * 256 + 4 * chunk) = word;
                }
            }
        }
    }
    if (P.act_sum != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
        if (ONE_WARP) {
            if (lane == 0) P.act_sum[row] = isum;
        } else {
            if (lane == 0) s_sum[warp] = isum;
            __syncthreads();
            if (threadIdx.x == 0) {
                int t = 0;
                for (int w = 0; w < n_warps; w++) t += s_sum[w];
                P.act_sum[row] = t;
            }
        }
    }
}

// Narrow rows (k <= 1024: one warp's worth) run four rows per CTA, one warp each.  Wider
// rows take one CTA per row with as many warps as possible (up to 8) and 1..4 group pairs
// per half-warp: many warps with few pairs each beat few warps with many (measured at
// k = 3072 and 12288, also against a persistent grid that prefetches the next row into
// registers) -- occupancy hides more latency than the per-thread bookkeeping costs.
constexpr int kRowsPerCta = 4;

template <typename T, int OP, bool ACT_ONLY>
int launch_prep_op(tpb_handle_t h, cudaStream_t st, const PrepParams &P0, int64_t m, int64_t k, int bits) {
    PrepParams P = P0;
    const int n_groups = (int)(k / 256);
    const int n_units = (n_groups + 1) / 2;
    P.m = (int)m;
    P.k = (int)k;
    P.n_groups = n_groups;
    P.maxq = bits == 4 ? 7.0f : 127.0f;
    cudaError_t err = cudaSuccess;
    if (n_units <= 2) {
        const dim3 grid((unsigned)((m + kRowsPerCta - 1) / kRowsPerCta)), block(kRowsPerCta * 32);
        const size_t smem = ACT_ONLY ? 0 : (size_t)kRowsPerCta * 2 * kTilePairs * sizeof(f2);
        err = tpb_launch_pdl(convrot_prep_kernel<T, 1, OP, ACT_ONLY, true>, grid, block, smem, st, P);
    } else {
        // The gated preps do more arithmetic per element and gain from more warps per row (one unit per
        // half-warp, up to 16 warps) while the row still fits that way; the plain prep does not.
        const bool wide = (OP == OP_SILU_MUL || OP == OP_SIGMOID_MUL) && n_units <= 2 * kMaxWarpsWide;
        const int max_warps = wide ? kMaxWarpsWide : kMaxWarps;
        const int upw = (n_units + 2 * max_warps - 1) / (2 * max_warps);  // 1..4 for k <= 32768
        const int warps = (n_units + 2 * upw - 1) / (2 * upw);
        const dim3 grid((unsigned)m), block(warps * 32);
        const size_t smem = ACT_ONLY ? 0 : (size_t)warps * 2 * kTilePairs * sizeof(f2);
#define TPB_PREP_CASE(UU)                                                                               \
    case UU: {                                                                                          \
        auto kern = convrot_prep_kernel<T, UU, OP, ACT_ONLY, false>;                                    \
        if (smem > 48 * 1024) err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (err == cudaSuccess) err = tpb_launch_pdl(kern, grid, block, smem, st, P);                   \
        break;                                                                                          \
    }
        switch (upw) {
            TPB_PREP_CASE(1)
            TPB_PREP_CASE(2)
            TPB_PREP_CASE(3)
            TPB_PREP_CASE(4)
            default: return tpb_fail(h, TPB_ERR_INVALID_ARG, "prep: k = %lld is too wide", (long long)k);
        }
#undef TPB_PREP_CASE
    }
    TPB_CUDA(h, err);
    return TPB_OK;
}

}  // namespace tpb_prep
