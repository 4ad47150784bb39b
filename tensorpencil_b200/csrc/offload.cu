// Weight-streaming offloader: pinned host -> HBM copies on a transfer stream,
// running ahead of the compute stream by as many layers as there are free slots.
//
// Stands in for the streaming half of the reference's weight cache
// (src/gpu/cuda/backend.zig:617-736 prefetch, :954-961 deferred free behind a
// compute-stream event, :1391-1408 consumer wait on the prefetch event;
// src/gpu/cuda/context.zig:175-187 staged upload).  Differences by design: the
// weight images already live in pinned memory, so there is no mmap -> staging
// memcpy and no helper thread; ordering is carried entirely by CUDA events, so
// no call blocks the host.
//
//   prefetch(L): pick the free slot released longest ago; transfer stream waits
//                for that slot's release event, copies L's image, records
//                L's "copied" event.
//   acquire(L) : (prefetches on demand) compute stream waits for "copied".
//   release(L) : records the slot's release event on the compute stream.
//
// Several GPUs of a node that stream the same weights share the host link instead of each
// pulling every byte through it: prefetch_part(L, r, g) copies only piece r of g of the image
// into the slot, the host then fills in the other pieces from the other GPUs' slots over
// NVLink (an all-gather enqueued on the transfer stream, whose handle transfer_stream()
// returns) and commit(L) records the "copied" event behind it.
#include <new>
#include <vector>

#include "tpb_internal.h"

namespace {

struct Layer {
    const void *host = nullptr;
    size_t bytes = 0;
    int slot = -1;  // slot holding (or receiving) this layer's image, -1 = not resident
    bool registered = false;
};

struct Slot {
    void *dev = nullptr;
    int layer = -1;
    bool in_use = false;        // acquired and not yet released
    bool filling = false;       // pieces are being copied in; "copied" is recorded by commit()
    bool has_release = false;   // `released` has been recorded at least once
    uint64_t release_seq = 0;   // order of the last release (0 = never used)
    cudaEvent_t copied = nullptr;
    cudaEvent_t released = nullptr;
};

}  // namespace

struct tpb_streamer_s {
    tpb_handle_t h = nullptr;
    cudaStream_t xfer = nullptr;
    size_t slot_bytes = 0;
    std::vector<Slot> slots;
    std::vector<Layer> layers;
    uint64_t bytes_copied = 0;
    uint64_t seq = 0;
};

// Gives layer L a slot: the free one released longest ago (never-used slots first); the transfer
// stream waits for that slot's release.  *fresh says whether the slot was assigned by this call.
static int stream_take_slot(tpb_streamer_t s, int layer_id, const char *who, bool *fresh) {
    tpb_handle_t h = s->h;
    Layer &L = s->layers[layer_id];
    *fresh = false;
    if (L.slot >= 0) return TPB_OK;  // already resident or on its way
    int best = -1;
    for (int i = 0; i < (int)s->slots.size(); i++) {
        const Slot &c = s->slots[i];
        if (c.in_use || c.filling) continue;
        if (best < 0 || c.release_seq < s->slots[best].release_seq) best = i;
    }
    if (best < 0)
        return tpb_fail(h, TPB_ERR_STATE,
                        "%s: every slot holds an acquired layer (release one first, or open more slots)", who);
    Slot &c = s->slots[best];
    if (c.layer >= 0) s->layers[c.layer].slot = -1;  // evict
    if (c.has_release) TPB_CUDA(h, cudaStreamWaitEvent(s->xfer, c.released, 0));
    c.layer = layer_id;
    // Keep a slot that was just filled from being picked again before it is used:
    // it now counts as the most recently touched one.
    c.release_seq = ++s->seq;
    L.slot = best;
    *fresh = true;
    return TPB_OK;
}

static int stream_prefetch_impl(tpb_streamer_t s, int layer_id) {
    tpb_handle_t h = s->h;
    bool fresh = false;
    const int rc = stream_take_slot(s, layer_id, "stream_prefetch", &fresh);
    if (rc != TPB_OK || !fresh) return rc;
    Layer &L = s->layers[layer_id];
    Slot &c = s->slots[L.slot];
    TPB_CUDA(h, cudaMemcpyAsync(c.dev, L.host, L.bytes, cudaMemcpyHostToDevice, s->xfer));
    TPB_CUDA(h, cudaEventRecord(c.copied, s->xfer));
    s->bytes_copied += L.bytes;
    return TPB_OK;
}

extern "C" {

int tpb_stream_open(tpb_handle_t h, size_t budget_bytes, size_t slot_bytes, int n_slots,
                    tpb_streamer_t *out) {
    if (!h || !out) return TPB_ERR_INVALID_ARG;
    *out = nullptr;
    TPB_CHECK_ARG(h, n_slots >= 1 && n_slots <= 64 && slot_bytes > 0, "stream_open: need 1..64 slots of non-zero size");
    TPB_CHECK_ARG(h, (size_t)n_slots * slot_bytes <= budget_bytes,
                  "stream_open: %d slots of %zu bytes exceed the budget of %zu bytes", n_slots, slot_bytes,
                  budget_bytes);
    tpb_streamer_s *s = new (std::nothrow) tpb_streamer_s();
    if (!s) return tpb_fail(h, TPB_ERR_OOM, "stream_open: host allocation failed");
    s->h = h;
    s->slot_bytes = slot_bytes;
    tpb_device_guard guard(h->device);   // the stream, the slots and the events belong to the handle's device
    cudaError_t e = guard.err;
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->xfer, cudaStreamNonBlocking);
    s->slots.resize(n_slots);
    for (int i = 0; i < n_slots && e == cudaSuccess; i++) {
        Slot &c = s->slots[i];
        e = cudaMalloc(&c.dev, slot_bytes);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c.copied, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c.released, cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        const int code = e == cudaErrorMemoryAllocation ? TPB_ERR_OOM : TPB_ERR_CUDA;
        tpb_fail(h, code, "stream_open: %s", cudaGetErrorString(e));
        cudaGetLastError();
        tpb_stream_close(s);
        return code;
    }
    *out = s;
    return TPB_OK;
}

int tpb_stream_close(tpb_streamer_t s) {
    if (!s) return TPB_ERR_INVALID_ARG;
    if (s->xfer) cudaStreamSynchronize(s->xfer);
    for (Slot &c : s->slots) {
        if (c.released) cudaEventSynchronize(c.released);
        if (c.dev) cudaFree(c.dev);
        if (c.copied) cudaEventDestroy(c.copied);
        if (c.released) cudaEventDestroy(c.released);
    }
    if (s->xfer) cudaStreamDestroy(s->xfer);
    delete s;
    return TPB_OK;
}

int tpb_stream_register(tpb_streamer_t s, int layer_id, const void *pinned_host, size_t bytes) {
    if (!s) return TPB_ERR_INVALID_ARG;
    tpb_handle_t h = s->h;
    TPB_CHECK_ARG(h, layer_id >= 0 && layer_id < (1 << 20), "stream_register: layer id out of range");
    TPB_CHECK_ARG(h, pinned_host && bytes > 0, "stream_register: null or empty image");
    TPB_CHECK_ARG(h, bytes <= s->slot_bytes, "stream_register: layer of %zu bytes does not fit a slot of %zu", bytes,
                  s->slot_bytes);
    if ((size_t)layer_id >= s->layers.size()) s->layers.resize(layer_id + 1);
    Layer &L = s->layers[layer_id];
    if (L.registered && L.slot >= 0) {
        if (s->slots[L.slot].in_use || s->slots[L.slot].filling)
            return tpb_fail(h, TPB_ERR_STATE, "stream_register: layer %d is acquired or being filled", layer_id);
        s->slots[L.slot].layer = -1;  // drop the stale image
    }
    L.host = pinned_host;
    L.bytes = bytes;
    L.slot = -1;
    L.registered = true;
    return TPB_OK;
}

static int check_layer(tpb_streamer_t s, int layer_id, const char *who) {
    if (layer_id < 0 || (size_t)layer_id >= s->layers.size() || !s->layers[layer_id].registered)
        return tpb_fail(s->h, TPB_ERR_STATE, "%s: layer %d was never registered", who, layer_id);
    return TPB_OK;
}

int tpb_stream_prefetch(tpb_streamer_t s, int layer_id) {
    if (!s) return TPB_ERR_INVALID_ARG;
    const int rc = check_layer(s, layer_id, "stream_prefetch");
    if (rc != TPB_OK) return rc;
    return stream_prefetch_impl(s, layer_id);
}

int tpb_stream_acquire(tpb_streamer_t s, int layer_id, tpb_stream_t compute, void **dev_ptr) {
    if (!s || !dev_ptr) return TPB_ERR_INVALID_ARG;
    int rc = check_layer(s, layer_id, "stream_acquire");
    if (rc != TPB_OK) return rc;
    tpb_handle_t h = s->h;
    rc = stream_prefetch_impl(s, layer_id);  // no-op when already on its way
    if (rc != TPB_OK) return rc;
    Layer &L = s->layers[layer_id];
    Slot &c = s->slots[L.slot];
    if (c.in_use) return tpb_fail(h, TPB_ERR_STATE, "stream_acquire: layer %d is already acquired", layer_id);
    if (c.filling)
        return tpb_fail(h, TPB_ERR_STATE, "stream_acquire: layer %d is being filled piece by piece and was not committed", layer_id);
    TPB_CUDA(h, cudaStreamWaitEvent((cudaStream_t)compute, c.copied, 0));
    c.in_use = true;
    *dev_ptr = c.dev;
    return TPB_OK;
}

int tpb_stream_release(tpb_streamer_t s, int layer_id, tpb_stream_t compute) {
    if (!s) return TPB_ERR_INVALID_ARG;
    const int rc = check_layer(s, layer_id, "stream_release");
    if (rc != TPB_OK) return rc;
    tpb_handle_t h = s->h;
    Layer &L = s->layers[layer_id];
    if (L.slot < 0 || !s->slots[L.slot].in_use)
        return tpb_fail(h, TPB_ERR_STATE, "stream_release: layer %d is not acquired", layer_id);
    Slot &c = s->slots[L.slot];
    TPB_CUDA(h, cudaEventRecord(c.released, (cudaStream_t)compute));
    c.has_release = true;
    c.in_use = false;
    c.release_seq = ++s->seq;
    return TPB_OK;
}

size_t tpb_stream_piece_bytes(size_t bytes, int n_parts) {
    if (n_parts < 1) return 0;
    const size_t piece = (bytes + (size_t)n_parts - 1) / (size_t)n_parts;
    return (piece + 255) / 256 * 256;
}

int tpb_stream_prefetch_part(tpb_streamer_t s, int layer_id, int part, int n_parts, void **dev_ptr) {
    if (!s || !dev_ptr) return TPB_ERR_INVALID_ARG;
    int rc = check_layer(s, layer_id, "stream_prefetch_part");
    if (rc != TPB_OK) return rc;
    tpb_handle_t h = s->h;
    TPB_CHECK_ARG(h, n_parts >= 1 && part >= 0 && part < n_parts, "stream_prefetch_part: part %d of %d", part, n_parts);
    Layer &L = s->layers[layer_id];
    const size_t piece = tpb_stream_piece_bytes(L.bytes, n_parts);
    TPB_CHECK_ARG(h, piece * (size_t)n_parts <= s->slot_bytes,
                  "stream_prefetch_part: %d pieces of %zu bytes need a slot of %zu bytes, slots have %zu", n_parts, piece,
                  piece * (size_t)n_parts, s->slot_bytes);
    if (L.slot >= 0 && !s->slots[L.slot].filling) {
        // resident or on its way already (every process of the group sees the same, having made the
        // same calls): nothing to copy, nothing to exchange, nothing to commit
        *dev_ptr = nullptr;
        return TPB_OK;
    }
    bool fresh = false;
    rc = stream_take_slot(s, layer_id, "stream_prefetch_part", &fresh);
    if (rc != TPB_OK) return rc;
    Slot &c = s->slots[L.slot];
    c.filling = true;
    const size_t off = piece * (size_t)part;
    if (off < L.bytes) {
        const size_t n = L.bytes - off < piece ? L.bytes - off : piece;
        TPB_CUDA(h, cudaMemcpyAsync(static_cast<char *>(c.dev) + off, static_cast<const char *>(L.host) + off, n,
                                    cudaMemcpyHostToDevice, s->xfer));
        s->bytes_copied += n;
    }
    *dev_ptr = c.dev;
    return TPB_OK;
}

int tpb_stream_commit(tpb_streamer_t s, int layer_id) {
    if (!s) return TPB_ERR_INVALID_ARG;
    const int rc = check_layer(s, layer_id, "stream_commit");
    if (rc != TPB_OK) return rc;
    tpb_handle_t h = s->h;
    Layer &L = s->layers[layer_id];
    if (L.slot < 0 || !s->slots[L.slot].filling)
        return tpb_fail(h, TPB_ERR_STATE, "stream_commit: layer %d has no pieces on their way", layer_id);
    Slot &c = s->slots[L.slot];
    TPB_CUDA(h, cudaEventRecord(c.copied, s->xfer));
    c.filling = false;
    return TPB_OK;
}

tpb_stream_t tpb_stream_transfer_stream(tpb_streamer_t s) { return s ? (tpb_stream_t)s->xfer : nullptr; }

uint64_t tpb_stream_bytes_copied(tpb_streamer_t s) { return s ? s->bytes_copied : 0; }

}  // extern "C"
