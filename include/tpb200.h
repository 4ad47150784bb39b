/*
 * tpb200.h -- C ABI of libtpb200.so, the B200-native (sm_100a) implementation
 * of TensorPencil's quantized-linear path.
 *
 * Each entry point names the TensorPencil interface it stands in for
 * (path:line within that project).  The reference binds its GPU libraries by
 * dlopen + symbol table (src/gpu/cuda/cu.zig:252-345); this header is what such
 * a table would list.
 *
 * Conventions
 *   - plain C linkage, plain pointers and sizes; no CUDA or C++ types in the
 *     signatures.  `stream` is a CUstream / cudaStream_t passed as void*.
 *   - every call returns 0 (TPB_OK) or a negative tpb_status; the text of the
 *     last failure on a handle is available from tpb_last_error().
 *   - the library never creates a CUDA context: tpb_create() binds to the
 *     device's primary context / whatever context is current, and all work is
 *     enqueued on the caller's stream.  No entry point synchronises unless its
 *     comment says so.
 *   - a handle is thread-compatible, not thread-safe: one thread at a time.
 *   - there is no CPU fallback anywhere behind this interface.
 */
#ifndef TPB200_H
#define TPB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tpb_handle_s *tpb_handle_t;
typedef struct tpb_streamer_s *tpb_streamer_t;
typedef void *tpb_stream_t; /* CUstream / cudaStream_t */

typedef enum tpb_status {
    TPB_OK = 0,
    TPB_ERR_INVALID_ARG = -1, /* bad pointer, shape, alignment or enum */
    TPB_ERR_CUDA = -2,        /* a CUDA call failed (reference: error.CudaError) */
    TPB_ERR_OOM = -3,         /* device or pinned-host allocation failed (error.DeviceOutOfMemory / OutOfMemory) */
    TPB_ERR_TIMEOUT = -4,     /* a bounded device-side wait ran out; see tpb_status_poll */
    TPB_ERR_STATE = -5,       /* call order violated (e.g. acquire of an unregistered layer) */
    TPB_ERR_NO_DEVICE = -6    /* no usable sm_100 device (error.NoSuitableDevice) */
} tpb_status;

typedef enum tpb_dtype {
    TPB_F32 = 0,
    TPB_BF16 = 1,
    TPB_F16 = 2,
    TPB_S32 = 3 /* raw int32 accumulators; output only */
} tpb_dtype;

/* ---- lifetime ------------------------------------------------------------
 * Stands in for cuda.Backend.init / deinit (src/gpu/cuda/backend.zig:196,
 * src/gpu/cuda/context.zig:103-116) for this path only. */
int tpb_version(void);
int tpb_create(tpb_handle_t *out, int device_ordinal);
int tpb_destroy(tpb_handle_t h);
const char *tpb_last_error(tpb_handle_t h);
const char *tpb_status_string(int status);

/* Reads (and clears) the device status word that bounded waits inside the
 * kernels write when they give up.  Synchronises `stream` first.  Returns
 * TPB_OK or TPB_ERR_TIMEOUT; *detail (optional) receives the raw word:
 * (role << 24) | stage, role 1 = tile loader, 2 = MMA issuer, 3 = epilogue. */
int tpb_status_poll(tpb_handle_t h, tpb_stream_t stream, uint32_t *detail);

/* Device facts the host side sizes its work with. */
int tpb_device_sm_count(tpb_handle_t h);

/* ---- ConvRot activation prep ----------------------------------------------
 * Replaces Backend.opI8Prep / opI4Prep + kernels.buildPrep
 * (src/gpu/cuda/backend.zig:2454-2480, :2532-2553; src/gpu/cuda/kernels.zig:971-1212).
 *
 * Per row of x[m][k]: rotate every 256-group with the regular Hadamard
 * (src/ops/convrot.zig:56-87, same add order), take the row absmax,
 * scale = max(absmax / maxq, 1e-12), q = clamp(round-half-away(v / scale)).
 * bits = 8: maxq 127, clamp [-127,127].  bits = 4: maxq 7, clamp [-8,7].
 *
 * Outputs (device, caller-owned; they replace the reference's hidden
 * i8_x / i8_scale backend scratch):
 *   q         int8 [m][k]   one value per byte for both widths
 *   act_scale f32  [m]
 *   act_sum   int32 [m]     sum of the row's q values; required when bits = 4
 *                           (the int4 GEMM consumes it), optional (NULL) for 8.
 * x_dtype: TPB_F32, TPB_F16 or TPB_BF16 (the reference's in_f16 switch).
 * k must be a multiple of 256 and at most 32768; x and q 16-byte aligned. */
int tpb_convrot_prep(tpb_handle_t h, tpb_stream_t stream, const void *x, int x_dtype,
                     int64_t m, int64_t k, int bits, int8_t *q, float *act_scale,
                     int32_t *act_sum);

/* ---- ConvRot GEMM + fused dequant ------------------------------------------
 * Replaces Backend.opI8Gemm / opI4Gemm + kernels.buildIgemmPipe(fuse) and the
 * irescale pass (src/gpu/cuda/backend.zig:2484-2501, :2558-2573, :2427-2450;
 * src/gpu/cuda/kernels.zig:557-958, :1216-1328).
 *
 *   y[i][j] = (float(sum_k q[i][k] * w[j][k]) * act_scale[i]) * w_scale[j]
 *
 * q int8 [m][k] and act_scale from tpb_convrot_prep.  w_bits = 8: w is int8
 * [n][k].  w_bits = 4: w is [n][k/2] bytes, element 2j in the low nibble
 * (src/core/dtype.zig:146-149), q holds int4-range values and act_sum is
 * required.  w_scale is one f32 per output row [n] for both widths
 * (src/ops/matmul.zig:82-89).  y is [m][ldy] with ldy >= n elements;
 * y_dtype TPB_F32 or TPB_BF16, or TPB_S32 to store the raw int32 accumulators
 * (scales ignored) for exact integer checks.
 * Requirements: k % 256 == 0, n % 16 == 0, all pointers 16-byte aligned, ldy
 * a multiple of 4 elements (8 for bf16).  Any m >= 1: no padding of m to 128
 * is needed (out-of-range rows are never read or written). */
int tpb_convrot_gemm(tpb_handle_t h, tpb_stream_t stream, void *y, int y_dtype, int64_t ldy,
                     const int8_t *q, const float *act_scale, const int32_t *act_sum,
                     const void *w, int w_bits, const float *w_scale,
                     int64_t m, int64_t n, int64_t k);

/* One whole ConvRot linear per call: tpb_convrot_prep followed by tpb_convrot_gemm, same
 * arguments, same results, everything enqueued on `stream`.  The reference issues prep and
 * GEMM separately (one prep can feed several GEMMs:
 * use the separate calls for that); this entry point is for the one-prep-one-GEMM case. */
int tpb_convrot_linear(tpb_handle_t h, tpb_stream_t stream, void *y, int y_dtype, int64_t ldy,
                       const void *x, int x_dtype, int8_t *q, float *act_scale, int32_t *act_sum,
                       const void *w, int w_bits, const float *w_scale,
                       int64_t m, int64_t n, int64_t k);

/* GEMM with the gated residual folded into the epilogue: replaces opI{8,4}Gemm followed by
 * Backend.gatedAdd (src/models/dit_cuda.zig:492-493, :515-516; src/gpu/cuda/backend.zig:3342-3347):
 *   x[i][j] = fma(gate[j], (float(acc) * act_scale[i]) * w_scale[j], x[i][j])
 * x is f32 [m][ldx], read and written in place; the result is bit-identical to
 * tpb_convrot_gemm (f32) followed by tpb_gated_add.  gate is an f32 vector of n. */
int tpb_convrot_gemm_gated_add(tpb_handle_t h, tpb_stream_t stream, float *x, int64_t ldx,
                               const float *gate, const int8_t *q, const float *act_scale,
                               const int32_t *act_sum, const void *w, int w_bits,
                               const float *w_scale, int64_t m, int64_t n, int64_t k);

/* The MLP's gate and up projections with the SiLU gate folded into the epilogue: replaces
 * op{I8,I4}Gemm (mlp.gate), op{I8,I4}Gemm (mlp.up) and Backend.siluMul
 * (src/models/dit_cuda.zig:508-513; src/gpu/cuda/backend.zig:3294-3315) by one launch:
 *   g = (float(acc_gate) * act_scale[i]) * w_gate_scale[j],  u = likewise with w_up
 *   y[i][j] = (g * sigmoid(g)) * u                           f32 arithmetic, then f32 or bf16
 * Both weights are [n][k] with their own scales; a tile's two halves come from the two weights,
 * so they are read as they lie in the checkpoint.  With y_dtype f32 the result is bit-identical to
 * the two GEMMs (f32) followed by tpb_silu_mul; bf16 is its round-to-nearest-even (the separate
 * route with bf16 GEMM outputs rounds g and u first, so it differs from that one in the last bits).
 * Always runs the two-CTA kernel.  For w_bits = 4 the reservation (tpb_convrot_w4_reserve) must
 * cover both weights: 2 n x k elements.  act_sum as for tpb_convrot_gemm. */
int tpb_convrot_gemm_silu_pair(tpb_handle_t h, tpb_stream_t stream, void *y, int y_dtype, int64_t ldy,
                               const int8_t *q, const float *act_scale, const int32_t *act_sum,
                               const void *w_gate, const float *w_gate_scale, const void *w_up,
                               const float *w_up_scale, int w_bits, int64_t m, int64_t n, int64_t k);

/* Up to four weights of the same shape multiplied with the same quantised activations in one launch:
 * replaces the op{I8,I4}Gemm calls that follow one prep -- q, k, v and gate of a DiT block
 * (src/models/dit_cuda.zig:473-478).  y[g] = dequant(q w[g]^T) exactly as tpb_convrot_gemm computes it, bit for
 * bit; all outputs share y_dtype (f32 or bf16) and ldy.  The weights' tiles follow one another in one
 * persistent kernel, so its pipeline fills and drains once instead of count times (4608 x 3072 x 3072, four
 * weights: 4 x 36 us -> 131 us).  y, w and w_scale are host arrays of `count` device pointers (1 <= count <= 4).
 * For w_bits = 4 the reservation (tpb_convrot_w4_reserve) must cover all weights: count * n x k elements.
 * Problems too small for the two-CTA kernel run as `count` ordinary launches. */
int tpb_convrot_gemm_group(tpb_handle_t h, tpb_stream_t stream, int count, void *const *y, int y_dtype, int64_t ldy,
                           const int8_t *q, const float *act_scale, const int32_t *act_sum, const void *const *w,
                           const float *const *w_scale, int w_bits, int64_t m, int64_t n, int64_t k);

/* INT4 weights run on the int8 tensor-core path: unless TPB_W4_FUSED=1 selects the kernel that
 * unpacks nibbles in shared memory, every int4 GEMM first widens its weight into a scratch
 * buffer the handle owns.  tpb_convrot_w4_reserve sizes that buffer for weights of up to n x k
 * elements (cudaMalloc; it may cudaFree a smaller one, which waits for the device).  Call it
 * once per handle, at set-up, outside any stream capture: the stream-ordered entry points
 * (tpb_convrot_gemm, tpb_convrot_linear, tpb_convrot_gemm_gated_add, tpb_convrot_gemm_silu_pair, tpb_convrot_gemm_group,
 * the all-gather forms)
 * never allocate, and return TPB_ERR_STATE for an int4 weight larger than the reservation.
 * Replaces the reference's ensureDeviceBuffer growth of its backend scratch
 * (src/gpu/cuda/backend.zig:2457-2470), made explicit. */
int tpb_convrot_w4_reserve(tpb_handle_t h, int64_t n, int64_t k);

/* Bytes of the int8 expansion of an [n][k] int4 weight. */
size_t tpb_convrot_w4_expanded_bytes(int64_t n, int64_t k);

/* Expands a packed int4 weight [n][k/2] into int8 [n][k] (device to device), so
 * a resident weight can be expanded once and then used with w_bits = 8.  No
 * counterpart in the reference, whose int4 kernel always reads packed nibbles. */
int tpb_convrot_w4_expand(tpb_handle_t h, tpb_stream_t stream, const void *w4, int64_t n,
                          int64_t k, int8_t *w8);

/* ---- GGUF Q8_0 decode GEMV ---------------------------------------------------
 * Q8_0 row = k/32 blocks of 34 bytes: f16 d, then 32 int8 (src/core/dtype.zig:93,
 * src/gpu/cuda/elt.zig:666-669).
 *
 * tpb_q8_1_quantize replaces Backend.opGemvQuantizeX + elt.quantize_q8_1
 * (src/gpu/cuda/backend.zig:1687-1695, src/gpu/cuda/elt.zig:1226-1269): per
 * 32-element block d = amax/127, q = round-to-nearest-even(x * (127/amax)),
 * 0 when amax == 0.  xq layout is the reference's: f32 d[n_elems/32] followed
 * by int8 qs[n_elems]; xq must hold n_elems/32*4 + n_elems bytes, 16-byte aligned,
 * n_elems % 32 == 0. */
int tpb_q8_1_quantize(tpb_handle_t h, tpb_stream_t stream, const float *x, int64_t n_elems,
                      void *xq);

/* Replaces Backend.opGemvQuantQ8N(.q8_0) + elt.gemv_q8_0_q8n
 * (src/gpu/cuda/backend.zig:1719-1735, src/gpu/cuda/elt.zig:1926-2006):
 *   y[i*rows + r] = scale * sum_b float(sum_e qw*qx) * (d_w * d_x),  i < ng <= 8
 * against activation rows row_off .. row_off+ng-1 of an xq buffer that holds
 * n_total rows of `cols` elements.  The weight streams from HBM once for all
 * ng rows.  cols % 32 == 0; w 16-byte aligned.
 *
 * Ordering: the GEMV kernels (this one, tpb_q8_0_gemv, tpb_q8_0_gemv_static and tpb_gguf_gemv_q8n) are launched
 * with programmatic stream serialisation and begin streaming the WEIGHT while the kernel before them in the
 * stream is still finishing; everything else (xq, y) is ordered as usual.  A weight is a constant of the model,
 * so this is invisible -- except to a host that produces `w` with a kernel launched on the same stream directly
 * before the call (a conversion or a copy kernel): put anything between the two (another kernel, an event), or
 * set TPB_NO_PDL=1, which launches every kernel of the library fully serialised.  Copies enqueued with
 * cudaMemcpyAsync and work ordered through events, as the weight streamer does it, are not affected. */
int tpb_q8_0_gemv_q8n(tpb_handle_t h, tpb_stream_t stream, float *y, const void *w, float scale,
                      int64_t rows, int64_t cols, const void *xq, int ng, int row_off,
                      int n_total);

/* Replaces Backend.opGemvQuant(.q8_0) + elt.gemv_q8_0
 * (src/gpu/cuda/backend.zig:1660-1681, src/gpu/cuda/elt.zig:671-727): the M = 1
 * GEMV in f32 arithmetic on un-quantised activations,
 *   y[r] = scale * sum_k (q_w * d_w) * x[k]. */
int tpb_q8_0_gemv_f32(tpb_handle_t h, tpb_stream_t stream, float *y, const float *x,
                      const void *w, float scale, int64_t rows, int64_t cols);

/* Decode linear that allocates nothing: quantises x[m][cols] (f32, m <= 8) and runs
 * the Q8_0 GEMV, y[i*rows + r] as tpb_q8_0_gemv_q8n (same kernels, same dispatch), keeping the quantised
 * activations in a fixed array inside the library instead of a buffer somebody has
 * to allocate.  It has no counterpart in the reference, whose backend grows its
 * q8 scratch with ensureDeviceBuffer.  It exists for hosts that cannot let a
 * plugin call cudaMalloc -- an engine that owns all device memory through its own
 * budgeted arena, or a decode loop that must not hit cudaMalloc's implicit device
 * synchronisation.  This call and everything under it makes no cudaMalloc/cudaFree
 * and calls no allocating library routine.
 *   - limit: m * cols <= TPB_STATIC_GEMV_MAX_ELEMS (8 rows of 32768 columns); larger
 *     requests return TPB_ERR_INVALID_ARG.  The array (TPB_STATIC_GEMV_SCRATCH_BYTES,
 *     288 KiB) is resident on every GPU that loads the library until the process ends.
 *   - the first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture begins.
 *   - all calls share the one array and it keeps the last call's contents: calls
 *     that may overlap on the GPU (different streams without ordering) race. */
#define TPB_STATIC_GEMV_MAX_ELEMS (8 * 32768)
#define TPB_STATIC_GEMV_SCRATCH_BYTES (TPB_STATIC_GEMV_MAX_ELEMS + TPB_STATIC_GEMV_MAX_ELEMS / 32 * 4)
int tpb_q8_0_gemv_static(tpb_handle_t h, tpb_stream_t stream, float *y, const float *x, int m,
                         const void *w, float scale, int64_t rows, int64_t cols);

/* ---- weight streaming ---------------------------------------------------------
 * Replaces the diffusion weight cache's streaming half: Backend.prefetchWeight,
 * cachedWeight's wait on a prefetch, the deferred free behind a compute-stream
 * event and Context.uploadStaged (src/gpu/cuda/backend.zig:617-736, :954-961,
 * :1376-1429; src/gpu/cuda/context.zig:151-187).
 *
 * A streamer owns n_slots device buffers of slot_bytes each (n_slots *
 * slot_bytes <= budget_bytes, the `--vram-budget` of src/main.zig:1454-1464) and
 * one transfer stream.  Layers are registered once with their pinned host
 * image.  prefetch(layer) copies host -> slot on the transfer stream as soon as
 * the slot's previous user has released it; acquire(layer) makes the compute
 * stream wait for that copy and returns the device address; release(layer)
 * records, on the compute stream, the point after which the slot may be
 * overwritten.  Nothing here blocks the host.  Calls for one streamer come from
 * one thread. */
int tpb_stream_open(tpb_handle_t h, size_t budget_bytes, size_t slot_bytes, int n_slots,
                    tpb_streamer_t *out);
int tpb_stream_close(tpb_streamer_t s);
int tpb_stream_register(tpb_streamer_t s, int layer_id, const void *pinned_host, size_t bytes);
int tpb_stream_prefetch(tpb_streamer_t s, int layer_id);
int tpb_stream_acquire(tpb_streamer_t s, int layer_id, tpb_stream_t compute, void **dev_ptr);
int tpb_stream_release(tpb_streamer_t s, int layer_id, tpb_stream_t compute);
/* Bytes copied host -> device since open (for the achieved-H2D-bandwidth figure). */
uint64_t tpb_stream_bytes_copied(tpb_streamer_t s);

/* Sharing the host link between the GPUs of a node (no counterpart in the reference, which
 * opens one device: src/gpu/cuda/context.zig:111).  When g processes, one per GPU, stream the
 * same layers in the same order, each can pull 1/g of every layer through PCIe and get the
 * rest from the others over NVLink:
 *   tpb_stream_prefetch_part(s, L, r, g, &dev) gives L a slot like prefetch does, copies only
 *     piece r of g of its image to the same offset in the slot, and returns the slot's device
 *     address.  Pieces are tpb_stream_piece_bytes(bytes, g) long (the image cut into g equal
 *     parts, rounded up to 256 bytes; the last is shorter); g * piece must fit a slot.  It
 *     may be called for several pieces of one layer.  No event is recorded yet.  For a layer
 *     that is resident (or on its way) already it copies nothing and returns a null address:
 *     skip the exchange and the commit -- processes that made the same calls all see the same.
 *   The host then enqueues, on tpb_stream_transfer_stream(s), whatever brings the other
 *     pieces into the slot (an in-place all-gather over the g slots).
 *   tpb_stream_commit(s, L) records the layer's "copied" event behind that work; from then on
 *     acquire / release work as usual.  acquire on a layer with uncommitted pieces and commit
 *     without pieces return TPB_ERR_STATE. */
size_t tpb_stream_piece_bytes(size_t bytes, int n_parts);
int tpb_stream_prefetch_part(tpb_streamer_t s, int layer_id, int part, int n_parts, void **dev_ptr);
int tpb_stream_commit(tpb_streamer_t s, int layer_id);
tpb_stream_t tpb_stream_transfer_stream(tpb_streamer_t s);

/* Pinned host memory for weight images (cuMemHostAlloc in src/gpu/cuda/context.zig:151-160). */
int tpb_host_alloc(tpb_handle_t h, size_t bytes, void **out);
int tpb_host_free(tpb_handle_t h, void *p);

/* ---- One GEMM split along N over the GPUs of a node, all-gather fused in ------------
 *
 * No reference counterpart: the reference drives one GPU (src/gpu/cuda/context.zig:111).
 * One process per GPU.  Rank r holds rows [r*n_shard, (r+1)*n_shard) of the weight and
 * of w_scale and the whole quantised activations; every rank owns a full row-major
 * y[m][ldy] in a peer-mapped buffer.  The GEMM's epilogue writes each output tile into
 * its columns [rank*n_shard, ...) of EVERY rank's y (local copy through TMA, peers with
 * 16-byte NVLink stores), so the exchange overlaps the tensor-core work tile by tile
 * and the result lands row-major, bit-identical to the single-GPU GEMM.  A y is complete
 * on rank r once every rank's launch has finished: run tpb_peer_barrier on the same
 * stream before reading it, and again before the next launch overwrites it. */

#define TPB_PEER_HANDLE_BYTES 64

/* cudaMalloc + zero fill on the handle's device; ipc_handle receives TPB_PEER_HANDLE_BYTES
 * opaque bytes to hand to the other processes. */
int tpb_peer_alloc(tpb_handle_t h, size_t bytes, void **ptr, void *ipc_handle);
/* Maps another process's buffer (enables peer access on first use). */
int tpb_peer_open(tpb_handle_t h, const void *ipc_handle, void **ptr);
int tpb_peer_close(tpb_handle_t h, void *ptr);
int tpb_peer_free(tpb_handle_t h, void *ptr);
/* flags[r] = rank r's flag row (>= world uint32, zero at start, inside a peer buffer);
 * epoch must grow by one per call on every rank.  The wait is bounded by timeout_ms;
 * on expiry the kernel records it and tpb_status_poll returns TPB_ERR_TIMEOUT. */
int tpb_peer_barrier(tpb_handle_t h, tpb_stream_t stream, uint32_t *const *flags, int world,
                     int rank, uint32_t epoch, int timeout_ms);
/* y_all[r] = base of rank r's y (y_all[rank] is local); other arguments as
 * tpb_convrot_gemm, with w_shard / w_scale_shard this rank's n_shard rows. */
int tpb_convrot_gemm_allgather(tpb_handle_t h, tpb_stream_t stream, void *const *y_all, int world,
                               int rank, int y_dtype, int64_t ldy, const int8_t *q,
                               const float *act_scale, const int32_t *act_sum,
                               const void *w_shard, int w_bits, const float *w_scale_shard,
                               int64_t m, int64_t n_shard, int64_t k);
/* The building block of the above for any destination layout: an ordinary GEMM whose
 * epilogue writes each output tile to y_local and, at the same (row, column, ldy), to every
 * y_peers[i] (peer-mapped pointers, 0 <= n_peers <= 7).  With ldy = n and each rank writing
 * at its own block offset the gathered result is column-blocked [rank][m][n] instead of
 * row-major, which keeps a sender's writes inside one contiguous region per destination. */
int tpb_convrot_gemm_multi(tpb_handle_t h, tpb_stream_t stream, void *y_local, void *const *y_peers,
                           int n_peers, int y_dtype, int64_t ldy, const int8_t *q,
                           const float *act_scale, const int32_t *act_sum, const void *w,
                           int w_bits, const float *w_scale, int64_t m, int64_t n, int64_t k);

/* The same with ONE store per output element: y_mc is an NVSwitch multicast address that
 * maps every rank's y (a CUDA multicast object bound to all the ranks' buffers, e.g.
 * torch's symmetric memory `multicast_ptr`); the epilogue writes each tile with
 * multimem.st and the switch replicates it into all copies, this rank's included, so a
 * GPU sends its shard once instead of world-1 times.  y_local is this rank's ordinary
 * address of the same buffer.  Completion: as above (tpb_peer_barrier). */
int tpb_convrot_gemm_allgather_mc(tpb_handle_t h, tpb_stream_t stream, void *y_mc, void *y_local,
                                  int world, int rank, int y_dtype, int64_t ldy, const int8_t *q,
                                  const float *act_scale, const int32_t *act_sum,
                                  const void *w_shard, int w_bits, const float *w_scale_shard,
                                  int64_t m, int64_t n_shard, int64_t k);

/* ---- Elementwise neighbours of the linears, and the prep with them fused in --------
 *
 * The DiT block computes every quantised linear's input with an elementwise op first
 * (src/models/dit_cuda.zig:473-514).  Stand-alone forms (HBM-bound, f32 results):
 *
 *   tpb_silu_mul     out = silu(gate) * up         Backend.siluMul      src/gpu/cuda/backend.zig:3310-3315
 *   tpb_sigmoid_mul  out = a * sigmoid(gate)       Backend.sigmoidMul   src/gpu/cuda/backend.zig:3294-3299
 *   tpb_rms_mod      out = x*inv*premul + shift    Backend.rmsMod       src/gpu/cuda/backend.zig:2738-2760
 *                    inv = 1/sqrt(mean(x^2) + eps) over each row of `dim`
 *   tpb_gated_add    x  += gate[c] * delta         Backend.gatedAdd     src/gpu/cuda/backend.zig:3342-3347
 *
 * out may alias the first input when that input is f32 (the reference's ops are in
 * place).  Inputs f32 or bf16 (in_dtype); premul/shift/gate are f32 vectors of `dim`
 * (the reference passes one `mod` buffer plus offsets: pass mod + offset here).
 * sigmoid uses the fast exponential/reciprocal, like the reference's kernels
 * (src/gpu/cuda/elt.zig:4-7); results agree with the CPU definitions
 * (src/ops/act.zig:61-70, :141-149; src/ops/norm.zig:12-23) to ~1e-6.
 *
 * tpb_convrot_prep_fused applies the same producer to the values as they are loaded
 * and goes straight on to rotate + quantise (as tpb_convrot_prep): the f32 activation
 * is never written.  q / act_scale / act_sum are bit-identical to running the
 * stand-alone op and then tpb_convrot_prep.  No reference counterpart (it runs the two
 * steps separately).  op: 1 = silu_mul (a = gate, b = up), 2 = sigmoid_mul (a, b = gate),
 * 3 = rms_mod (a = x, premul, shift, eps; b unused). */
#define TPB_OP_SILU_MUL 1
#define TPB_OP_SIGMOID_MUL 2
#define TPB_OP_RMS_MOD 3
int tpb_silu_mul(tpb_handle_t h, tpb_stream_t stream, const void *gate, const void *up, int in_dtype,
                 float *out, int64_t n);
int tpb_sigmoid_mul(tpb_handle_t h, tpb_stream_t stream, const void *a, const void *gate, int in_dtype,
                    float *out, int64_t n);
int tpb_rms_mod(tpb_handle_t h, tpb_stream_t stream, const void *x, int x_dtype, float *out,
                const float *premul, const float *shift, float eps, int64_t rows, int64_t dim);
int tpb_gated_add(tpb_handle_t h, tpb_stream_t stream, float *x, const void *delta, int delta_dtype,
                  const float *gate, int64_t rows, int64_t dim);
int tpb_convrot_prep_fused(tpb_handle_t h, tpb_stream_t stream, int op, const void *a, const void *b,
                           const float *premul, const float *shift, float eps, int in_dtype,
                           int64_t m, int64_t k, int bits, int8_t *q, float *act_scale,
                           int32_t *act_sum);

/* ---- Decode GEMV for the other GGUF block formats -----------------------------------
 * Replaces Backend.opGemvQuantQ8N for .q4_0 / .q4_k / .q5_k / .q6_k / .iq4_nl (src/gpu/cuda/backend.zig:1719-1735;
 * kernels src/gpu/cuda/elt.zig:2014-2110, :1831-1925, :1526-1713, :1714-1830); TPB_GGUF_Q8_0 forwards to
 * tpb_q8_0_gemv_q8n.  Same arguments and activation buffer (tpb_q8_1_quantize) as
 * tpb_q8_0_gemv_q8n; w holds `rows` rows of tpb_gguf_row_bytes(fmt, cols) bytes in ggml's
 * block layout (src/core/quants.zig:9-16).  cols % 256 == 0.
 *   y[i*rows + r] = scale * sum_k dequant(w[r])[k] * (d_x * q_x)[i][k]
 * q6_k rows are not multiples of 16 bytes: the kernel's bulk copies are rounded out to 16-byte
 * boundaries, so the copy of the last row may read (and ignore) up to 14 bytes beyond the
 * weights -- never beyond the 16-byte word their last byte lies in.  With w 16-byte aligned, as
 * required, that word cannot straddle a page or an allocation boundary, so the read cannot
 * fault; when rows * row_bytes is a multiple of 16 nothing outside the weights is read at all.
 * iq4_nl: q4_0's layout with ggml's 16-entry value table. */
typedef enum tpb_gguf_format {
    TPB_GGUF_Q8_0 = 0,
    TPB_GGUF_Q4_0 = 1,
    TPB_GGUF_Q4_K = 2,
    TPB_GGUF_Q5_K = 3,
    TPB_GGUF_Q6_K = 4,
    TPB_GGUF_IQ4_NL = 5
} tpb_gguf_format;
size_t tpb_gguf_row_bytes(int fmt, int64_t cols);
int tpb_gguf_gemv_q8n(tpb_handle_t h, tpb_stream_t stream, int fmt, float *y, const void *w, float scale,
                      int64_t rows, int64_t cols, const void *xq, int ng, int row_off, int n_total);

/* ---- Attention of the DiT block (the op between the quantised linears of a block) ---
 * Replaces Backend.qkNorm + rope + attn / opAttnTC for the non-causal, unmasked case
 * (src/models/dit_cuda.zig:479-489; src/gpu/cuda/backend.zig:2939-3196; CPU definitions
 * src/ops/norm.zig:12-23, src/ops/rope.zig:68-90, src/ops/attention.zig:46-150).
 *
 * tpb_attn_prepare: q [seq][heads*128], k and v [seq][kv_heads*128] (f32 or bf16) ->
 *   qb [heads][seq][128] and kb [kv_heads][seq][128] = rope(x * inv_rms(x) * norm_weight) in bf16
 *   (per-head RMS norm over the 128 elements, then the interleaved-pair rotation with the
 *   per-position tables cos/sin [seq][64]), and vt = v transposed per head,
 *   [kv_heads][128][seq_pad] bf16 with seq_pad = seq rounded up to 8 (tpb_attn_vt_elems elements).
 * tpb_attention: out [seq_q][heads*128] (bf16 or f32) = softmax(q k^T * scale) v per head,
 *   kv head = head / (heads / kv_heads); flash-style on tcgen05, f32 softmax and accumulation,
 *   probabilities rounded to bf16 for the second product.  head_dim must be 128. */
size_t tpb_attn_vt_elems(int64_t seq_kv, int kv_heads);
int tpb_attn_prepare(tpb_handle_t h, tpb_stream_t stream, const void *q, const void *k, const void *v,
                     int in_dtype, const float *q_norm, const float *k_norm, float eps,
                     const float *cosv, const float *sinv, int64_t seq, int heads, int kv_heads,
                     int head_dim, void *qb, void *kb, void *vt);
int tpb_attention(tpb_handle_t h, tpb_stream_t stream, void *out, int out_dtype, const void *qb,
                  const void *kb, const void *vt, int64_t seq_q, int64_t seq_kv, int heads,
                  int kv_heads, int head_dim, float scale);

#ifdef __cplusplus
}
#endif
#endif /* TPB200_H */
