/*
 * tpb_oracle.h -- CPU restatement of TensorPencil's quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker the CUDA path is
 * compared against and the timed CPU baseline.  It is never linked into, nor
 * called from, the shipped library: only tests/, the smoke check and the
 * CPU-baseline legs of bench.py load it.
 *
 * Every function names the TensorPencil source (path:line within that project)
 * whose arithmetic it restates.  The restatement is pinned against the
 * reference's own golden vectors (tests/golden): the ComfyUI int4 ConvRot
 * dequant fixture, the ggml Q8_0 dequant block, the nibble-decode known-answer
 * cases and the Hadamard property tests.
 *
 * Parity unpinned: the bit-level behaviour of ggml's CPU activation quantiser
 * and vec_dot (ggml @ af97976c, a fetched dependency of the reference that is
 * not vendored).  The Q8_0 GEMV oracle here follows the reference's own test
 * references for that path instead (f64 dequant-dot and the q8_1 emulation).
 */
#ifndef TPB_ORACLE_H
#define TPB_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TPO_GROUP 256 /* src/ops/convrot.zig:17 */

/* -- ConvRot rotation ------------------------------------------------------ */

/* In-place H*v per 256-chunk, radix-4 FWHT with strides 1,4,16,64, then /16.
 * src/ops/convrot.zig:56-87.  n must be a multiple of 256. */
void tpo_convrot_rotate(float *data, size_t n);

/* Explicit normalised 256x256 regular Hadamard (kron of the 4x4 block, /16).
 * src/ops/convrot.zig:19-47.  out is [256][256] row-major. */
void tpo_hadamard256(float *out);

/* -- Storage layouts ------------------------------------------------------- */

/* Signed nibble decode: idx 0 = low nibble, 1 = high.  src/core/dtype.zig:146-149 */
int8_t tpo_nibble_i4(uint8_t byte, int idx);

/* Unpack n_elems int4 values (element 2j in the low nibble of byte j). */
void tpo_unpack_i4(const uint8_t *packed, size_t n_elems, int8_t *out);

/* Pack int8 values in [-8,7] two per byte, low nibble first (the inverse of
 * tpo_unpack_i4; packing rule of src/gpu/cuda/kernels.zig:2441-2443). */
void tpo_pack_i4(const int8_t *vals, size_t n_elems, uint8_t *packed);

/* int4 ConvRot weight dequant used by the fixture test: unpack * row scale,
 * then rotate back.  src/ops/convrot.zig:172-181.  out is [rows][cols] f32. */
void tpo_i4_convrot_dequant(const uint8_t *packed, const float *row_scale,
                            size_t rows, size_t cols, float *out);

/* -- Integer-domain replica ("cpu-sim") ------------------------------------ */

/* Rotate each row, per-row absmax, s = max(amax/maxq, 1e-12), q = clamp(round
 * half away (x/s)).  bits = 8 -> maxq 127, clamp [-127,127]; bits = 4 -> maxq
 * 7, clamp [-8,7].  src/gpu/cuda/kernels.zig:2638-2653 (int8), :2487-2502
 * (int4).  q is int8 [m][k] for both widths; xr (optional, may be NULL)
 * receives the rotated f32 rows.  Threaded over rows. */
void tpo_convrot_prep(const float *x, size_t m, size_t k, int bits,
                      int8_t *q, float *act_scale, float *xr);

/* acc[i][j] = sum_k a[i][k] * w[j][k] in int32.  kernels.zig:2660-2664.
 * Threaded over rows of a. */
void tpo_igemm_s32(const int8_t *a, const int8_t *w, size_t m, size_t n,
                   size_t k, int32_t *acc);

/* sim[i][j] = (double)acc * as[i] * ws[j] in f64.  kernels.zig:2667. */
void tpo_dequant_sim(const int32_t *acc, const float *act_scale,
                     const float *w_scale, size_t m, size_t n, double *y);

/* f64 truth of the same linear on rotated, un-quantised activations:
 * sum_k xr[i][k] * (w[j][k] * ws[j]).  kernels.zig:2665. */
void tpo_linear_truth(const float *xr, const int8_t *w, const float *w_scale,
                      size_t m, size_t n, size_t k, double *y);

/* -- The `--backend cpu` float path ----------------------------------------- */

/* y[m][n] = x[m][k] . (rot(q * row_scale))^T (+bias): per weight row dequantise
 * (q*row_scale), un-rotate with the group Hadamard, then an f32 FMA chain over
 * k ascending per output.  src/ops/matmul.zig:196-234 (task split), :408-484
 * (int8 pack), :502-563 (int4 pack), :580-639 (microkernel).  w_bits 8: w is
 * int8 [n][k]; 4: packed [n][k/2].  convrot = 0 skips the rotation.
 * nthreads <= 0 uses every core. */
void tpo_linear_cpu_backend(const float *x, size_t m, const void *w, int w_bits,
                            const float *row_scale, size_t n, size_t k,
                            int convrot, const float *bias, float *y,
                            int nthreads);
/* The two halves of the above, callable on their own: the path for m < 16 activation rows
 * (src/ops/matmul.zig:669-767) and the packed outer-product path (:196-234, :408-639). */
void tpo_linear_cpu_small_m(const float *x, size_t m, const void *w, int w_bits,
                            const float *row_scale, size_t n, size_t k,
                            int convrot, const float *bias, float *y,
                            int nthreads);
void tpo_linear_cpu_packed(const float *x, size_t m, const void *w, int w_bits,
                           const float *row_scale, size_t n, size_t k,
                           int convrot, const float *bias, float *y,
                           int nthreads);

/* -- GGUF Q8_0 -------------------------------------------------------------- */

#define TPO_Q8_0_BLOCK_BYTES 34 /* f16 d + 32 x i8; src/core/dtype.zig:93 */

float tpo_f16_to_f32(uint16_t h);
uint16_t tpo_f32_to_f16(float f);

/* Dequantise k elements (k % 32 == 0) of one Q8_0 row: y = d * q.
 * Layout src/gpu/cuda/elt.zig:666-669; golden bits src/core/quants_fixtures.zig:6-15. */
void tpo_q8_0_dequant_row(const uint8_t *blocks, size_t k, float *out);

/* Per 32-element block: d = amax/127, inv = amax==0 ? 0 : 127/amax, q = round(x*inv).
 * tie_mode 0: round to nearest even (the device kernel, elt.zig:1253-1265);
 * tie_mode 1: half away from zero (the host emulation in the reference's
 * tests, backend.zig:3641-3651).  d is [n/32], qs is [n]. */
void tpo_q8_1_quantize(const float *x, size_t n, int tie_mode, float *d, int8_t *qs);

/* y[t][r] = scale * sum_k dequant(W[r])[k] * x[t][k], accumulated in f64 --
 * the reference the reference's own f32-GEMV test compares with.
 * src/gpu/cuda/backend.zig:3608-3614.  Threaded over rows. */
void tpo_q8_0_gemv_f64(const uint8_t *w, size_t n, size_t k, const float *x,
                       size_t m, float scale, float *y);

/* Same, against activations passed through the q8_1 quantiser first
 * (x_hat = d * q): the reference of the dp4a GEMV tests, backend.zig:3776-3782. */
void tpo_q8_0_gemv_q8(const uint8_t *w, size_t n, size_t k, const float *x,
                      size_t m, float scale, int tie_mode, float *y);

/* Integer inner products of the dp4a path: sumi[t][r][b] = sum_{e<32} qw*qx for
 * every (activation row, weight row, block).  elt.zig:1984-1996. */
void tpo_q8_0_block_sumi(const uint8_t *w, size_t n, size_t k, const int8_t *xq,
                         size_t m, int32_t *sumi);

/* Elementwise neighbours of the quantized linears (producers of the prep input and the
 * gated residual): src/ops/act.zig:61-70, :141-149; src/ops/norm.zig:12-23 + src/models/dit.zig:575-590. */
void tpo_silu_mul(const float *gate, const float *up, size_t n, float *out);
void tpo_sigmoid_mul(const float *dst, const float *gate, size_t n, float *out);
void tpo_rms_mod(const float *x, size_t rows, size_t dim, const float *premul, const float *shift,
                 float eps, float *out);
void tpo_gated_add(const float *x, const float *delta, const float *gate, size_t rows, size_t dim,
                   float *out);

/* Other GGUF block formats (ggml's decoders, pinned by src/core/quants_fixtures.zig) and a
 * format-generic GEMV truth (src/gpu/cuda/backend.zig:3750-3790).  fmt: 0 q8_0, 1 q4_0,
 * 2 q4_k, 3 q5_k, 4 q6_k, 5 iq4_nl. */
void tpo_q4_k_dequant_row(const uint8_t *blocks, size_t k, float *out);
void tpo_q5_k_dequant_row(const uint8_t *blocks, size_t k, float *out);
void tpo_q6_k_dequant_row(const uint8_t *blocks, size_t k, float *out);
void tpo_q4_0_dequant_row(const uint8_t *blocks, size_t k, float *out);
void tpo_iq4_nl_dequant_row(const uint8_t *blocks, size_t k, float *out);
size_t tpo_gguf_row_bytes(int fmt, size_t k);
void tpo_gguf_dequant_row(int fmt, const uint8_t *row, size_t k, float *out);
void tpo_gguf_gemv_q8(int fmt, const uint8_t *w, size_t n, size_t k, const float *x, size_t m, float scale,
                      float *y);

/* Attention of the DiT block (src/ops/norm.zig:12-23, src/ops/rope.zig:28-90, src/ops/attention.zig:46-150). */
void tpo_qk_norm(const float *x, size_t rows, size_t hd, const float *w, float eps, float *out);
void tpo_flux_freqs(const float *positions, size_t seq, const int *axes_dim, int n_axes, double theta, float *cosv,
                    float *sinv);
void tpo_rope_interleaved(float *x, const float *cosv, const float *sinv, size_t seq, size_t heads, size_t hd);
void tpo_attention(const float *q, const float *k, const float *v, size_t seq_q, size_t seq_kv, size_t heads,
                   size_t kv_heads, size_t hd, float scale, float *out);

int tpo_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
