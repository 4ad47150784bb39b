/*
 * tpb_oracle.c -- CPU restatement of TensorPencil's quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY (see tpb_oracle.h).  Compile with
 * -ffp-contract=off: the reference's Zig code fuses a multiply-add only where
 * it says @mulAdd, and this file does the same with explicit FMA intrinsics.
 */
#include "tpb_oracle.h"

#include <immintrin.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int tpo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* ConvRot rotation -- src/ops/convrot.zig                                   */
/* ------------------------------------------------------------------------ */

/* 4x4 regular-Hadamard block, convrot.zig:19-25. */
static const float H4[4][4] = {
    {1, 1, 1, -1},
    {1, 1, -1, 1},
    {1, -1, 1, 1},
    {-1, 1, 1, 1},
};

void tpo_hadamard256(float *out) {
    /* convrot.zig:30-47: product over the four base-4 digits, then /16. */
    for (int i = 0; i < TPO_GROUP; i++) {
        for (int j = 0; j < TPO_GROUP; j++) {
            float p = 1.0f;
            int ii = i, jj = j;
            for (int d = 0; d < 4; d++) {
                p *= H4[ii % 4][jj % 4];
                ii /= 4;
                jj /= 4;
            }
            out[i * TPO_GROUP + j] = p / 16.0f;
        }
    }
}

/* convrot.zig:56-78.  The add order is the reference's, left to right:
 * ((a+b)+c)-d, ((a+b)-c)+d, ((a-b)+c)+d, ((-a+b)+c)+d. */
static void rotate_group(float *v) {
    static const size_t strides[4] = {1, 4, 16, 64};
    for (int si = 0; si < 4; si++) {
        const size_t s = strides[si];
        for (size_t base = 0; base < TPO_GROUP; base += s * 4) {
            for (size_t o = 0; o < s; o++) {
                const size_t p = base + o;
                const float a = v[p];
                const float b = v[p + s];
                const float c = v[p + 2 * s];
                const float d = v[p + 3 * s];
                v[p] = a + b + c - d;
                v[p + s] = a + b - c + d;
                v[p + 2 * s] = a - b + c + d;
                v[p + 3 * s] = -a + b + c + d;
            }
        }
    }
    for (size_t i = 0; i < TPO_GROUP; i++) v[i] /= 16.0f;
}

void tpo_convrot_rotate(float *data, size_t n) {
    for (size_t off = 0; off + TPO_GROUP <= n; off += TPO_GROUP)
        rotate_group(data + off);
}

/* ------------------------------------------------------------------------ */
/* Storage layouts -- src/core/dtype.zig                                     */
/* ------------------------------------------------------------------------ */

int8_t tpo_nibble_i4(uint8_t byte, int idx) {
    /* dtype.zig:146-149: take the nibble, reinterpret as a signed 4-bit value. */
    const uint8_t nib = (uint8_t)((byte >> (idx ? 4 : 0)) & 0xF);
    return (int8_t)((nib & 0x8) ? (int)nib - 16 : (int)nib);
}

void tpo_unpack_i4(const uint8_t *packed, size_t n_elems, int8_t *out) {
    for (size_t e = 0; e < n_elems; e++)
        out[e] = tpo_nibble_i4(packed[e / 2], (int)(e & 1));
}

void tpo_pack_i4(const int8_t *vals, size_t n_elems, uint8_t *packed) {
    for (size_t i = 0; i < n_elems / 2; i++)
        packed[i] = (uint8_t)(((uint8_t)vals[2 * i] & 0xF) |
                              (((uint8_t)vals[2 * i + 1] & 0xF) << 4));
}

void tpo_i4_convrot_dequant(const uint8_t *packed, const float *row_scale,
                            size_t rows, size_t cols, float *out) {
    for (size_t r = 0; r < rows; r++) {
        const uint8_t *rb = packed + r * cols / 2;
        float *row = out + r * cols;
        for (size_t k = 0; k < cols; k++)
            row[k] = (float)tpo_nibble_i4(rb[k / 2], (int)(k & 1)) * row_scale[r];
        tpo_convrot_rotate(row, cols);
    }
}

/* ------------------------------------------------------------------------ */
/* Integer-domain replica -- src/gpu/cuda/kernels.zig:2638-2677, :2487-2523  */
/* ------------------------------------------------------------------------ */

void tpo_convrot_prep(const float *x, size_t m, size_t k, int bits, int8_t *q,
                      float *act_scale, float *xr_out) {
    const float maxq = bits == 4 ? 7.0f : 127.0f;
    const int lo = bits == 4 ? -8 : -127;
    const int hi = bits == 4 ? 7 : 127;
#pragma omp parallel
    {
        float *tmp = (float *)malloc(k * sizeof(float));
#pragma omp for schedule(static)
        for (long long i = 0; i < (long long)m; i++) {
            float *xr = xr_out ? xr_out + (size_t)i * k : tmp;
            memcpy(xr, x + (size_t)i * k, k * sizeof(float));
            tpo_convrot_rotate(xr, k);
            float amax = 0.0f;
            for (size_t c = 0; c < k; c++) {
                const float a = fabsf(xr[c]);
                amax = a > amax ? a : amax; /* @max(amax, @abs(v)) */
            }
            float s = amax / maxq;
            s = s > 1e-12f ? s : 1e-12f; /* @max(amax / maxq, 1e-12) */
            act_scale[i] = s;
            for (size_t c = 0; c < k; c++) {
                int qi = (int)roundf(xr[c] / s); /* @round: half away from zero */
                qi = qi < lo ? lo : (qi > hi ? hi : qi);
                q[(size_t)i * k + c] = (int8_t)qi;
            }
        }
        free(tmp);
    }
}

void tpo_igemm_s32(const int8_t *a, const int8_t *w, size_t m, size_t n,
                   size_t k, int32_t *acc) {
#pragma omp parallel for schedule(dynamic, 4)
    for (long long i = 0; i < (long long)m; i++) {
        const int8_t *ar = a + (size_t)i * k;
        for (size_t j = 0; j < n; j++) {
            const int8_t *wr = w + j * k;
            int32_t s = 0;
            for (size_t c = 0; c < k; c++) s += (int32_t)ar[c] * (int32_t)wr[c];
            acc[(size_t)i * n + j] = s;
        }
    }
}

void tpo_dequant_sim(const int32_t *acc, const float *act_scale,
                     const float *w_scale, size_t m, size_t n, double *y) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++)
            y[i * n + j] = (double)acc[i * n + j] * (double)act_scale[i] * (double)w_scale[j];
}

void tpo_linear_truth(const float *xr, const int8_t *w, const float *w_scale,
                      size_t m, size_t n, size_t k, double *y) {
#pragma omp parallel for schedule(dynamic, 4)
    for (long long i = 0; i < (long long)m; i++) {
        for (size_t j = 0; j < n; j++) {
            double t = 0.0;
            for (size_t c = 0; c < k; c++)
                t += (double)xr[(size_t)i * k + c] *
                     ((double)w[j * k + c] * (double)w_scale[j]);
            y[(size_t)i * n + j] = t;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* `--backend cpu` float path -- src/ops/matmul.zig                          */
/* ------------------------------------------------------------------------ */

enum { MR = 6, NR = 16, KC = 512 }; /* matmul.zig:69-71 (vlen 8 => NR 16) */

/* matmul.zig:580-639: MRC x NR register tile, one FMA per (row, k) in k order,
 * continuing from y when this is not the first k block. */
static void micro_kernel(int mrc, float *y, const float *x, const float *sub,
                         size_t t0, size_t col0, size_t rows, size_t cols,
                         size_t kc0, size_t kl, const float *bias, int accumulate) {
    const int full = col0 + NR <= rows;
    __m256 acc[MR][2];
    for (int mi = 0; mi < mrc; mi++) {
        float tmp[NR];
        memset(tmp, 0, sizeof tmp);
        if (accumulate) {
            const size_t lim = full ? NR : rows - col0;
            for (size_t c = 0; c < lim; c++) tmp[c] = y[(t0 + mi) * rows + col0 + c];
        } else if (bias) {
            const size_t lim = full ? NR : rows - col0;
            for (size_t c = 0; c < lim; c++) tmp[c] = bias[col0 + c];
        }
        acc[mi][0] = _mm256_loadu_ps(tmp);
        acc[mi][1] = _mm256_loadu_ps(tmp + 8);
    }
    for (size_t k = 0; k < kl; k++) {
        const __m256 b0 = _mm256_loadu_ps(sub + k * NR);
        const __m256 b1 = _mm256_loadu_ps(sub + k * NR + 8);
        for (int mi = 0; mi < mrc; mi++) {
            const __m256 a = _mm256_set1_ps(x[(t0 + mi) * cols + kc0 + k]);
            acc[mi][0] = _mm256_fmadd_ps(a, b0, acc[mi][0]);
            acc[mi][1] = _mm256_fmadd_ps(a, b1, acc[mi][1]);
        }
    }
    for (int mi = 0; mi < mrc; mi++) {
        float tmp[NR];
        _mm256_storeu_ps(tmp, acc[mi][0]);
        _mm256_storeu_ps(tmp + 8, acc[mi][1]);
        const size_t lim = full ? NR : rows - col0;
        for (size_t c = 0; c < lim; c++) y[(t0 + mi) * rows + col0 + c] = tmp[c];
    }
}

/* matmul.zig:408-484 (.i8) and :502-563 (.i4): per KC-wide k block, dequantise
 * each weight row of the chunk (q * row_scale), un-rotate, scatter k-major into
 * NR-wide subpanels, then sweep the microkernel over all activation rows. */
static void packed_task(float *y, const float *x, size_t m, const void *w,
                        int w_bits, const float *row_scale, size_t rows,
                        size_t cols, int convrot, const float *bias,
                        size_t row_start, size_t row_end, float *panel) {
    const size_t n_nr = (row_end - row_start + NR - 1) / NR;
    for (size_t kc0 = 0; kc0 < cols; kc0 += KC) {
        const size_t kl = cols - kc0 < KC ? cols - kc0 : KC;
        for (size_t nr = 0; nr < n_nr; nr++) {
            float *sub = panel + nr * KC * NR;
            for (size_t j = 0; j < NR; j++) {
                const size_t row = row_start + nr * NR + j;
                if (row >= rows) {
                    for (size_t k = 0; k < kl; k++) sub[k * NR + j] = 0.0f;
                    continue;
                }
                float tmp[KC];
                const float rs = row_scale[row];
                if (w_bits == 8) {
                    const int8_t *src = (const int8_t *)w + row * cols + kc0;
                    for (size_t k = 0; k < kl; k++) tmp[k] = (float)src[k] * rs;
                } else {
                    const uint8_t *src = (const uint8_t *)w + (row * cols + kc0) / 2;
                    for (size_t k = 0; k < kl; k++)
                        tmp[k] = (float)tpo_nibble_i4(src[k / 2], (int)(k & 1)) * rs;
                }
                if (convrot) tpo_convrot_rotate(tmp, kl);
                for (size_t k = 0; k < kl; k++) sub[k * NR + j] = tmp[k];
            }
        }
        for (size_t t0 = 0; t0 < m; t0 += MR) {
            const int mr = (int)(m - t0 < MR ? m - t0 : MR);
            for (size_t nr = 0; nr < n_nr; nr++)
                micro_kernel(mr, y, x, panel + nr * KC * NR, t0, row_start + nr * NR,
                             rows, cols, kc0, kl, kc0 == 0 ? bias : NULL, kc0 != 0);
        }
    }
}

/* matmul.zig:669-717 (runRangeTyped, .i8) and :722-767 (runRangeI4): the path for fewer than
 * small_m_max = 16 activation rows.  Panels of 8 weight rows are dequantised (q * row_scale)
 * and un-rotated whole; every output is a vlen-lane vector accumulator over k (a multiply and
 * an add per step, as the Zig source writes `acc += xv * wv` in strict float mode: no fused
 * multiply-add), reduced lane 0..7 in order, plus the scalar tail, plus the bias.  vlen = 8 is
 * what std.simd.suggestVectorLength(f32) gives on the AVX2 targets the reference is built for
 * (matmul.zig:63).  A row's sum does not depend on how rows are grouped into panels or tasks. */
enum { PANEL_ROWS = 8, VLEN = 8, SMALL_M_MAX = 16 }; /* matmul.zig:61-72 */

void tpo_linear_cpu_small_m(const float *x, size_t m, const void *w, int w_bits,
                            const float *row_scale, size_t n, size_t k,
                            int convrot, const float *bias, float *y,
                            int nthreads) {
    if (m == 0 || n == 0) return;
    const int nt = nthreads > 0 ? nthreads : tpo_num_threads();
#pragma omp parallel num_threads(nt)
    {
        float *row = (float *)aligned_alloc(64, ((k * sizeof(float) + 63) / 64) * 64);
#pragma omp for schedule(dynamic, PANEL_ROWS)
        for (long long r = 0; r < (long long)n; r++) {
            const float rs = row_scale[r];
            if (w_bits == 8) {
                const int8_t *src = (const int8_t *)w + (size_t)r * k;
                for (size_t c = 0; c < k; c++) row[c] = (float)src[c] * rs;
            } else {
                const uint8_t *src = (const uint8_t *)w + ((size_t)r * k) / 2;
                for (size_t c = 0; c < k; c++)
                    row[c] = (float)tpo_nibble_i4(src[c / 2], (int)(c & 1)) * rs;
            }
            if (convrot) tpo_convrot_rotate(row, k);
            for (size_t t = 0; t < m; t++) {
                const float *xr = x + t * k;
                float acc[VLEN];
                for (int l = 0; l < VLEN; l++) acc[l] = 0.0f;
                float tail = 0.0f;
                size_t c = 0;
                for (; c + VLEN <= k; c += VLEN)
                    for (int l = 0; l < VLEN; l++) {
                        volatile float prod = xr[c + l] * row[c + l]; /* rounded product, then the add */
                        acc[l] += prod;
                    }
                for (; c < k; c++) {
                    volatile float prod = xr[c] * row[c];
                    tail += prod;
                }
                float sum = acc[0];
                for (int l = 1; l < VLEN; l++) sum += acc[l];
                sum += tail;
                if (bias) sum += bias[r];
                y[t * n + (size_t)r] = sum;
            }
        }
        free(row);
    }
}

void tpo_linear_cpu_packed(const float *x, size_t m, const void *w, int w_bits,
                           const float *row_scale, size_t n, size_t k,
                           int convrot, const float *bias, float *y,
                           int nthreads);

/* matmul.zig:105-194: fewer than 16 activation rows take the small-m path, the rest the
 * packed outer-product path. */
void tpo_linear_cpu_backend(const float *x, size_t m, const void *w, int w_bits,
                            const float *row_scale, size_t n, size_t k,
                            int convrot, const float *bias, float *y,
                            int nthreads) {
    if (m < SMALL_M_MAX)
        tpo_linear_cpu_small_m(x, m, w, w_bits, row_scale, n, k, convrot, bias, y, nthreads);
    else
        tpo_linear_cpu_packed(x, m, w, w_bits, row_scale, n, k, convrot, bias, y, nthreads);
}

void tpo_linear_cpu_packed(const float *x, size_t m, const void *w, int w_bits,
                           const float *row_scale, size_t n, size_t k,
                           int convrot, const float *bias, float *y,
                           int nthreads) {
    if (m == 0 || n == 0) return;
    int nt = nthreads > 0 ? nthreads : tpo_num_threads();
    /* matmul.zig:206-211: 4 x ncpu row chunks, rounded up to whole NR panels. */
    const size_t want = nt == 1 ? 1 : (size_t)4 * (size_t)nt;
    size_t per = (n + want - 1) / want;
    if (per < NR) per = NR;
    const size_t chunk = (per + NR - 1) / NR * NR;
    const size_t n_tasks = (n + chunk - 1) / chunk;
    const size_t stride = (chunk / NR) * KC * NR;
#pragma omp parallel num_threads(nt)
    {
        float *panel = (float *)aligned_alloc(64, stride * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (long long t = 0; t < (long long)n_tasks; t++) {
            const size_t r0 = (size_t)t * chunk;
            const size_t r1 = r0 + chunk < n ? r0 + chunk : n;
            packed_task(y, x, m, w, w_bits, row_scale, n, k, convrot, bias, r0, r1, panel);
        }
        free(panel);
    }
}

/* ------------------------------------------------------------------------ */
/* GGUF Q8_0                                                                  */
/* ------------------------------------------------------------------------ */

float tpo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t tpo_f32_to_f16(float f) {
    /* round to nearest even, via the F16C conversion instruction */
    const __m128 v = _mm_set_ss(f);
    const __m128i h = _mm_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
    return (uint16_t)_mm_extract_epi16(h, 0);
}

void tpo_q8_0_dequant_row(const uint8_t *blocks, size_t k, float *out) {
    for (size_t b = 0; b < k / 32; b++) {
        const uint8_t *blk = blocks + b * TPO_Q8_0_BLOCK_BYTES;
        uint16_t dh;
        memcpy(&dh, blk, 2);
        const float d = tpo_f16_to_f32(dh);
        const int8_t *qs = (const int8_t *)(blk + 2);
        for (int e = 0; e < 32; e++) out[b * 32 + e] = (float)qs[e] * d;
    }
}

void tpo_q8_1_quantize(const float *x, size_t n, int tie_mode, float *d, int8_t *qs) {
    for (size_t b = 0; b < n / 32; b++) {
        float amax = 0.0f;
        for (int e = 0; e < 32; e++) {
            const float a = fabsf(x[b * 32 + e]);
            amax = a > amax ? a : amax;
        }
        d[b] = amax / 127.0f;
        const float inv = amax == 0.0f ? 0.0f : 127.0f / amax;
        for (int e = 0; e < 32; e++) {
            const float v = x[b * 32 + e] * inv;
            const float r = tie_mode ? roundf(v) : nearbyintf(v);
            qs[b * 32 + e] = (int8_t)(int)r;
        }
    }
}

void tpo_q8_0_gemv_f64(const uint8_t *w, size_t n, size_t k, const float *x,
                       size_t m, float scale, float *y) {
    const size_t row_bytes = k / 32 * TPO_Q8_0_BLOCK_BYTES;
#pragma omp parallel
    {
        float *row = (float *)malloc(k * sizeof(float));
#pragma omp for schedule(static)
        for (long long r = 0; r < (long long)n; r++) {
            tpo_q8_0_dequant_row(w + (size_t)r * row_bytes, k, row);
            for (size_t t = 0; t < m; t++) {
                double acc = 0.0;
                for (size_t c = 0; c < k; c++) acc += (double)row[c] * (double)x[t * k + c];
                y[t * n + (size_t)r] = (float)(acc * (double)scale);
            }
        }
        free(row);
    }
}

void tpo_q8_0_gemv_q8(const uint8_t *w, size_t n, size_t k, const float *x,
                      size_t m, float scale, int tie_mode, float *y) {
    float *xq = (float *)malloc(m * k * sizeof(float));
    float *d = (float *)malloc(m * k / 32 * sizeof(float));
    int8_t *qs = (int8_t *)malloc(m * k);
    tpo_q8_1_quantize(x, m * k, tie_mode, d, qs);
    for (size_t i = 0; i < m * k; i++) xq[i] = d[i / 32] * (float)qs[i];
    tpo_q8_0_gemv_f64(w, n, k, xq, m, scale, y);
    free(xq);
    free(d);
    free(qs);
}

void tpo_q8_0_block_sumi(const uint8_t *w, size_t n, size_t k, const int8_t *xq,
                         size_t m, int32_t *sumi) {
    const size_t nblk = k / 32;
    const size_t row_bytes = nblk * TPO_Q8_0_BLOCK_BYTES;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)n; r++) {
        for (size_t t = 0; t < m; t++) {
            for (size_t b = 0; b < nblk; b++) {
                const int8_t *qw = (const int8_t *)(w + (size_t)r * row_bytes +
                                                    b * TPO_Q8_0_BLOCK_BYTES + 2);
                const int8_t *qx = xq + t * k + b * 32;
                int32_t s = 0;
                for (int e = 0; e < 32; e++) s += (int32_t)qw[e] * (int32_t)qx[e];
                sumi[(t * n + (size_t)r) * nblk + b] = s;
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Elementwise neighbours of the quantized linears in the DiT block          */
/* (the producers that feed the activation prep, and the gated residual).    */
/* ------------------------------------------------------------------------ */

/* src/ops/vmath.zig:56-59: 1 / (1 + exp(-x)); the reference's own test compares its
 * vector exp against libm at 2e-7 (vmath.zig:81-88), so libm stands in here. */
static inline float tpo_sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

/* src/ops/act.zig:61-70: gate[i] = gate[i] * sigmoid(gate[i]) * up[i]. */
void tpo_silu_mul(const float *gate, const float *up, size_t n, float *out) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++) out[i] = gate[i] * tpo_sigmoidf(gate[i]) * up[i];
}

/* src/ops/act.zig:141-149: dst[i] *= sigmoid(gate[i]). */
void tpo_sigmoid_mul(const float *dst, const float *gate, size_t n, float *out) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++) out[i] = dst[i] * tpo_sigmoidf(gate[i]);
}

/* RMS norm + AdaLN modulation as the GPU step applies it: out = (x * inv) * premul[c] +
 * shift[c], inv = 1/sqrt(mean(x^2) + eps), premul = (1 + scale) * norm_weight prepared by the
 * host (src/gpu/cuda/backend.zig:2738-2760, src/gpu/cuda/elt.zig:9-66; CPU form
 * src/ops/norm.zig:12-23, :63-76 followed by modulate, src/models/dit.zig:575-581).
 * The sum of squares is taken in double: every float summation order the reference uses
 * (8-lane vectors on the CPU, 256 partials on the GPU) lies within its own 2e-6 gate of it. */
void tpo_rms_mod(const float *x, size_t rows, size_t dim, const float *premul, const float *shift,
                 float eps, float *out) {
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)rows; r++) {
        const float *xr = x + (size_t)r * dim;
        double ss = 0.0;
        for (size_t c = 0; c < dim; c++) ss += (double)xr[c] * (double)xr[c];
        const float mean = (float)(ss / (double)dim);
        const float inv = 1.0f / sqrtf(mean + eps);
        for (size_t c = 0; c < dim; c++) out[(size_t)r * dim + c] = xr[c] * inv * premul[c] + shift[c];
    }
}

/* src/models/dit.zig:584-590: x[row][c] += gate[c] * delta[row][c]. */
void tpo_gated_add(const float *x, const float *delta, const float *gate, size_t rows, size_t dim,
                   float *out) {
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)rows; r++)
        for (size_t c = 0; c < dim; c++) {
            const size_t i = (size_t)r * dim + c;
            out[i] = x[i] + gate[c] * delta[i];
        }
}

/* ------------------------------------------------------------------------ */
/* Other GGUF block formats (ggml's published decoders; the reference calls   */
/* ggml for them, src/core/quants.zig:60-68, and pins them with golden        */
/* blocks, src/core/quants_fixtures.zig -- which pin these restatements too). */
/* Layouts: src/core/quants.zig:9-16.                                         */
/* ------------------------------------------------------------------------ */

/* 6-bit sub-block scale and min number j (0..7) of a q4_k / q5_k super-block. */
static inline void tpo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* q4_k: 144 bytes per 256 elements: f16 d, f16 dmin, scales[12], qs[128]. */
void tpo_q4_k_dequant_row(const uint8_t *blocks, size_t k, float *out) {
    for (size_t sb = 0; sb < k / 256; sb++) {
        const uint8_t *b = blocks + sb * 144;
        uint16_t hd, hm;
        memcpy(&hd, b, 2);
        memcpy(&hm, b + 2, 2);
        const float d = tpo_f16_to_f32(hd), dmin = tpo_f16_to_f32(hm);
        const uint8_t *sc = b + 4, *q = b + 16;
        float *y = out + sb * 256;
        int is = 0;
        for (int j = 0; j < 256; j += 64) {
            uint8_t s, m;
            tpo_scale_min_k4(is + 0, sc, &s, &m);
            const float d1 = d * s, m1 = dmin * m;
            tpo_scale_min_k4(is + 1, sc, &s, &m);
            const float d2 = d * s, m2 = dmin * m;
            for (int l = 0; l < 32; l++) *y++ = d1 * (q[l] & 0xF) - m1;
            for (int l = 0; l < 32; l++) *y++ = d2 * (q[l] >> 4) - m2;
            q += 32;
            is += 2;
        }
    }
}

/* q5_k: 176 bytes: f16 d, f16 dmin, scales[12], qh[32], qs[128]. */
void tpo_q5_k_dequant_row(const uint8_t *blocks, size_t k, float *out) {
    for (size_t sb = 0; sb < k / 256; sb++) {
        const uint8_t *b = blocks + sb * 176;
        uint16_t hd, hm;
        memcpy(&hd, b, 2);
        memcpy(&hm, b + 2, 2);
        const float d = tpo_f16_to_f32(hd), dmin = tpo_f16_to_f32(hm);
        const uint8_t *sc = b + 4, *qh = b + 16, *ql = b + 48;
        float *y = out + sb * 256;
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < 256; j += 64) {
            uint8_t s, m;
            tpo_scale_min_k4(is + 0, sc, &s, &m);
            const float d1 = d * s, m1 = dmin * m;
            tpo_scale_min_k4(is + 1, sc, &s, &m);
            const float d2 = d * s, m2 = dmin * m;
            for (int l = 0; l < 32; l++) *y++ = d1 * ((ql[l] & 0xF) + (qh[l] & u1 ? 16 : 0)) - m1;
            for (int l = 0; l < 32; l++) *y++ = d2 * ((ql[l] >> 4) + (qh[l] & u2 ? 16 : 0)) - m2;
            ql += 32;
            is += 2;
            u1 <<= 2;
            u2 <<= 2;
        }
    }
}

/* q6_k: 210 bytes: ql[128], qh[64], int8 scales[16], f16 d. */
void tpo_q6_k_dequant_row(const uint8_t *blocks, size_t k, float *out) {
    for (size_t sb = 0; sb < k / 256; sb++) {
        const uint8_t *b = blocks + sb * 210;
        const uint8_t *ql = b, *qh = b + 128;
        const int8_t *sc = (const int8_t *)(b + 192);
        uint16_t hd;
        memcpy(&hd, b + 208, 2);
        const float d = tpo_f16_to_f32(hd);
        float *y = out + sb * 256;
        for (int n = 0; n < 256; n += 128) {
            for (int l = 0; l < 32; l++) {
                const int is = l / 16;
                const int8_t q1 = (int8_t)((ql[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int8_t q3 = (int8_t)((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[l + 0] = d * sc[is + 0] * q1;
                y[l + 32] = d * sc[is + 2] * q2;
                y[l + 64] = d * sc[is + 4] * q3;
                y[l + 96] = d * sc[is + 6] * q4;
            }
            y += 128;
            ql += 64;
            qh += 32;
            sc += 8;
        }
    }
}

/* q4_0: 18 bytes per 32 elements: f16 d, 16 nibble bytes; element j in the low nibble of
 * byte j, element j + 16 in the high nibble; v = d * (nibble - 8).  No golden block in the
 * reference for this one: parity unpinned. */
void tpo_q4_0_dequant_row(const uint8_t *blocks, size_t k, float *out) {
    for (size_t blk = 0; blk < k / 32; blk++) {
        const uint8_t *b = blocks + blk * 18;
        uint16_t hd;
        memcpy(&hd, b, 2);
        const float d = tpo_f16_to_f32(hd);
        for (int j = 0; j < 16; j++) {
            out[blk * 32 + j] = ((b[2 + j] & 0xF) - 8) * d;
            out[blk * 32 + j + 16] = ((b[2 + j] >> 4) - 8) * d;
        }
    }
}

/* iq4_nl: 18 bytes per 32 elements like q4_0, but the nibble indexes a non-linear table:
 * v = d * kvalues[nibble] (ggml's kvalues_iq4nl; layout and table as the reference's test states
 * them, src/core/quants.zig:133-151). */
static const int8_t tpo_kvalues_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

void tpo_iq4_nl_dequant_row(const uint8_t *blocks, size_t k, float *out) {
    for (size_t blk = 0; blk < k / 32; blk++) {
        const uint8_t *b = blocks + blk * 18;
        uint16_t hd;
        memcpy(&hd, b, 2);
        const float d = tpo_f16_to_f32(hd);
        for (int j = 0; j < 16; j++) {
            out[blk * 32 + j] = d * (float)tpo_kvalues_iq4nl[b[2 + j] & 0xF];
            out[blk * 32 + j + 16] = d * (float)tpo_kvalues_iq4nl[b[2 + j] >> 4];
        }
    }
}

/* GEMV against q8_1-quantised activations for any of the formats above, the way the
 * reference's device test forms its CPU truth (src/gpu/cuda/backend.zig:3750-3790):
 * dequantise the weight row, dequantise the activations (d * q per 32-block), f64 dot.
 * fmt: 0 q8_0, 1 q4_0, 2 q4_k, 3 q5_k, 4 q6_k, 5 iq4_nl. */
size_t tpo_gguf_row_bytes(int fmt, size_t k) {
    switch (fmt) {
        case 0: return k / 32 * 34;
        case 1: return k / 32 * 18;
        case 2: return k / 256 * 144;
        case 3: return k / 256 * 176;
        case 4: return k / 256 * 210;
        case 5: return k / 32 * 18;
    }
    return 0;
}

void tpo_gguf_dequant_row(int fmt, const uint8_t *row, size_t k, float *out) {
    switch (fmt) {
        case 0: tpo_q8_0_dequant_row(row, k, out); break;
        case 1: tpo_q4_0_dequant_row(row, k, out); break;
        case 2: tpo_q4_k_dequant_row(row, k, out); break;
        case 3: tpo_q5_k_dequant_row(row, k, out); break;
        case 4: tpo_q6_k_dequant_row(row, k, out); break;
        case 5: tpo_iq4_nl_dequant_row(row, k, out); break;
    }
}

void tpo_gguf_gemv_q8(int fmt, const uint8_t *w, size_t n, size_t k, const float *x, size_t m, float scale,
                      float *y) {
    const size_t rb = tpo_gguf_row_bytes(fmt, k);
    float *xh = (float *)malloc(m * k * sizeof(float));
    {
        float *d = (float *)malloc(m * k / 32 * sizeof(float));
        int8_t *qs = (int8_t *)malloc(m * k);
        tpo_q8_1_quantize(x, m * k, 0, d, qs);
        for (size_t i = 0; i < m * k; i++) xh[i] = d[i / 32] * (float)qs[i];
        free(d);
        free(qs);
    }
#pragma omp parallel
    {
        float *wr = (float *)malloc(k * sizeof(float));
#pragma omp for schedule(static)
        for (long long r = 0; r < (long long)n; r++) {
            tpo_gguf_dequant_row(fmt, w + (size_t)r * rb, k, wr);
            for (size_t t = 0; t < m; t++) {
                double acc = 0.0;
                for (size_t c = 0; c < k; c++) acc += (double)wr[c] * (double)xh[t * k + c];
                y[t * n + r] = (float)(acc * (double)scale);
            }
        }
        free(wr);
    }
}

/* ------------------------------------------------------------------------ */
/* Attention of the DiT block: per-head RMS norm of q and k, interleaved-pair */
/* RoPE, softmax attention with grouped-query heads.                          */
/* ------------------------------------------------------------------------ */

/* src/ops/norm.zig:12-23 applied per head row of `hd` (dit.zig:623-624): x * inv_rms * w. */
void tpo_qk_norm(const float *x, size_t rows, size_t hd, const float *w, float eps, float *out) {
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)rows; r++) {
        const float *xr = x + (size_t)r * hd;
        double ss = 0.0;
        for (size_t c = 0; c < hd; c++) ss += (double)xr[c] * (double)xr[c];
        const float inv = 1.0f / sqrtf((float)(ss / (double)hd) + eps);
        for (size_t c = 0; c < hd; c++) out[(size_t)r * hd + c] = xr[c] * inv * w[c];
    }
}

/* src/ops/rope.zig:28-66: FLUX multi-axis tables; positions [seq][n_axes], angles in f64. */
void tpo_flux_freqs(const float *positions, size_t seq, const int *axes_dim, int n_axes, double theta, float *cosv,
                    float *sinv) {
    size_t half = 0;
    for (int a = 0; a < n_axes; a++) half += (size_t)axes_dim[a] / 2;
    for (size_t p = 0; p < seq; p++) {
        size_t off = 0;
        for (int a = 0; a < n_axes; a++) {
            const double pos = positions[p * (size_t)n_axes + (size_t)a];
            const int dh = axes_dim[a] / 2;
            for (int i = 0; i < dh; i++) {
                const double omega = 1.0 / pow(theta, (double)(2 * i) / (double)axes_dim[a]);
                cosv[p * half + off + (size_t)i] = (float)cos(pos * omega);
                sinv[p * half + off + (size_t)i] = (float)sin(pos * omega);
            }
            off += (size_t)dh;
        }
    }
}

/* src/ops/rope.zig:68-90: (x0, x1) -> (x0 c - x1 s, x0 s + x1 c) on consecutive pairs; x is [seq][heads*hd]. */
void tpo_rope_interleaved(float *x, const float *cosv, const float *sinv, size_t seq, size_t heads, size_t hd) {
    const size_t half = hd / 2;
    for (size_t p = 0; p < seq; p++)
        for (size_t h = 0; h < heads; h++) {
            float *b = x + (p * heads + h) * hd;
            for (size_t i = 0; i < half; i++) {
                const float x0 = b[2 * i], x1 = b[2 * i + 1];
                const float c = cosv[p * half + i], s = sinv[p * half + i];
                b[2 * i] = x0 * c - x1 * s;
                b[2 * i + 1] = x0 * s + x1 * c;
            }
        }
}

/* src/ops/attention.zig:46-60, :104-150 (non-causal, no mask): out[seq_q][heads*hd] =
 * softmax(q k^T * scale) v per head, kv head = h / (heads / kv_heads); f64 accumulation. */
void tpo_attention(const float *q, const float *k, const float *v, size_t seq_q, size_t seq_kv, size_t heads,
                   size_t kv_heads, size_t hd, float scale, float *out) {
    const size_t rep = heads / kv_heads;
#pragma omp parallel
    {
        double *sc = (double *)malloc(seq_kv * sizeof(double));
#pragma omp for schedule(static) collapse(2)
        for (long long h = 0; h < (long long)heads; h++)
            for (long long i = 0; i < (long long)seq_q; i++) {
                const size_t hk = (size_t)h / rep;
                const float *qr = q + ((size_t)i * heads + (size_t)h) * hd;
                double mx = -1e300;
                for (size_t j = 0; j < seq_kv; j++) {
                    const float *kr = k + (j * kv_heads + hk) * hd;
                    double d = 0.0;
                    for (size_t c = 0; c < hd; c++) d += (double)qr[c] * (double)kr[c];
                    sc[j] = d * (double)scale;
                    if (sc[j] > mx) mx = sc[j];
                }
                double sum = 0.0;
                for (size_t j = 0; j < seq_kv; j++) {
                    sc[j] = exp(sc[j] - mx);
                    sum += sc[j];
                }
                float *o = out + ((size_t)i * heads + (size_t)h) * hd;
                for (size_t c = 0; c < hd; c++) {
                    double a = 0.0;
                    for (size_t j = 0; j < seq_kv; j++) a += sc[j] * (double)v[(j * kv_heads + hk) * hd + c];
                    o[c] = (float)(a / sum);
                }
            }
        free(sc);
    }
}
