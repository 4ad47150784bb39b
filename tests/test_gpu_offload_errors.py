"""Error paths of the weight streamer (tpb_stream_*), driven from the host: wrong call order,
exhausted slots, oversize layers, budgets that do not hold the slots.  Every case must come back
as a status code with a message -- nothing is enqueued, nothing faults, and the streamer stays
usable afterwards.  The reference reports the matching conditions as Zig errors from its weight
cache (src/gpu/cuda/backend.zig:740-764 for the out-of-memory ladder, :1376-1429 for the cache);
here they are TPB_ERR_STATE / TPB_ERR_INVALID_ARG."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from tensorpencil_b200._lib import TPB_ERR_INVALID_ARG, TPB_ERR_STATE, TPB_OK, TpbError  # noqa: E402

pytestmark = pytest.mark.gpu
SLOT = 1 << 16


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


def make(be, n_slots=2, slot=SLOT, budget=None):
    from tensorpencil_b200.offload import Streamer
    return Streamer(be, budget if budget is not None else n_slots * slot, slot, n_slots)


def layer(seed, nbytes=SLOT // 2):
    return [np.random.default_rng(seed).integers(0, 256, nbytes, dtype=np.uint8)]


def status_of(fn):
    with pytest.raises(TpbError) as e:
        fn()
    return e.value.status, str(e.value)


def test_open_rejects_slots_beyond_the_budget(be):
    st, msg = status_of(lambda: make(be, n_slots=3, budget=2 * SLOT))
    assert st == TPB_ERR_INVALID_ARG and "exceed the budget" in msg
    st, _ = status_of(lambda: make(be, n_slots=0))
    assert st == TPB_ERR_INVALID_ARG
    st, _ = status_of(lambda: make(be, n_slots=65))
    assert st == TPB_ERR_INVALID_ARG


def test_layer_larger_than_a_slot_is_refused(be):
    s = make(be)
    try:
        st, msg = status_of(lambda: s.register(0, layer(1, SLOT + 256)))
        assert st == TPB_ERR_INVALID_ARG and "does not fit a slot" in msg
        s.register(0, layer(1))                     # the streamer still works
        assert torch.equal(s.acquire(0)[0].cpu(), torch.from_numpy(layer(1)[0]))
        s.release(0)
    finally:
        s.close()


def test_unregistered_layer(be):
    s = make(be)
    try:
        for call in (lambda: s.prefetch(5), lambda: s.acquire(5), lambda: s.release(5), lambda: s.prefetch(-1)):
            st, msg = status_of(call)
            assert st == TPB_ERR_STATE and "never registered" in msg
    finally:
        s.close()


def test_acquire_twice_and_release_unacquired(be):
    s = make(be)
    try:
        s.register(0, layer(2))
        s.register(1, layer(3))
        st, msg = status_of(lambda: s.release(0))
        assert st == TPB_ERR_STATE and "not acquired" in msg
        s.acquire(0)
        st, msg = status_of(lambda: s.acquire(0))
        assert st == TPB_ERR_STATE and "already acquired" in msg
        s.release(0)
        st, _ = status_of(lambda: s.release(0))     # released once already
        assert st == TPB_ERR_STATE
        s.prefetch(1)                               # prefetched, never acquired: release is refused
        st, _ = status_of(lambda: s.release(1))
        assert st == TPB_ERR_STATE
    finally:
        s.close()


def test_every_slot_acquired(be):
    s = make(be, n_slots=2)
    try:
        for i in range(3):
            s.register(i, layer(10 + i))
        s.acquire(0)
        s.acquire(1)
        for call in (lambda: s.prefetch(2), lambda: s.acquire(2)):
            st, msg = status_of(call)
            assert st == TPB_ERR_STATE and "every slot holds an acquired layer" in msg
        s.release(0)
        got = s.acquire(2)[0]                       # a slot is free again: the data is layer 2's
        assert torch.equal(got.cpu(), torch.from_numpy(layer(12)[0]))
        s.release(2)
        s.release(1)
    finally:
        s.close()


def test_reregister_while_acquired_is_refused_and_allowed_after_release(be):
    s = make(be)
    try:
        s.register(0, layer(20))
        s.acquire(0)
        st, msg = status_of(lambda: s.register(0, layer(21)))
        assert st == TPB_ERR_STATE and "is acquired" in msg
        s.release(0)
        s.register(0, layer(21))                    # the stale device image must not be served
        assert torch.equal(s.acquire(0)[0].cpu(), torch.from_numpy(layer(21)[0]))
        s.release(0)
    finally:
        s.close()


def test_null_arguments(be):
    lib = be.lib
    out = C.c_void_p()
    assert lib.tpb_stream_open(None, SLOT, SLOT, 1, C.byref(out)) == TPB_ERR_INVALID_ARG
    assert lib.tpb_stream_open(be.h, SLOT, SLOT, 1, None) == TPB_ERR_INVALID_ARG
    assert lib.tpb_stream_acquire(None, 0, None, C.byref(out)) == TPB_ERR_INVALID_ARG
    assert lib.tpb_stream_close(None) == TPB_ERR_INVALID_ARG
    s = make(be)
    try:
        assert lib.tpb_stream_register(s.s, 0, None, 16) == TPB_ERR_INVALID_ARG
        assert lib.tpb_stream_acquire(s.s, 0, None, None) == TPB_ERR_INVALID_ARG
        assert lib.tpb_stream_bytes_copied(s.s) == 0
    finally:
        s.close()
    assert TPB_OK == 0


def test_a_layer_brought_in_piece_by_piece(be):
    """The entry points behind the shared host link, on one GPU: both halves of a layer copied by this
    process, then commit -- the slot holds the image; the misuse around it is reported."""
    lib = be.lib
    nbytes = SLOT // 2 - 40                                  # not a multiple of the piece size
    piece = int(lib.tpb_stream_piece_bytes(nbytes, 2))
    assert piece % 256 == 0 and 2 * piece >= nbytes
    s = make(be, n_slots=2, slot=SLOT)
    try:
        img = layer(11, nbytes)
        s.register(0, img)
        s.register(1, layer(12, nbytes))
        dev = C.c_void_p()
        st, msg = status_of(lambda: s._check(lib.tpb_stream_commit(s.s, 0)))
        assert st == TPB_ERR_STATE and "no pieces" in msg
        st, _ = status_of(lambda: s._check(lib.tpb_stream_prefetch_part(s.s, 0, 2, 2, C.byref(dev))))
        assert st == TPB_ERR_INVALID_ARG                      # part out of range
        st, msg = status_of(lambda: s._check(lib.tpb_stream_prefetch_part(s.s, 0, 0, 512, C.byref(dev))))
        assert st == TPB_ERR_INVALID_ARG and "need a slot" in msg   # 512 pieces of 256 bytes
        s._check(lib.tpb_stream_prefetch_part(s.s, 0, 1, 2, C.byref(dev)))
        first = dev.value
        assert first
        st, msg = status_of(lambda: s.acquire(0))             # pieces under way, not committed
        assert st == TPB_ERR_STATE and "not committed" in msg
        s._check(lib.tpb_stream_prefetch_part(s.s, 0, 0, 2, C.byref(dev)))
        assert dev.value == first                             # same slot
        s._check(lib.tpb_stream_commit(s.s, 0))
        got = s.acquire(0)[0]
        assert torch.equal(got.cpu(), torch.from_numpy(img[0]))
        # resident now: another piece request copies nothing and says so with a null address
        s._check(lib.tpb_stream_prefetch_part(s.s, 0, 0, 2, C.byref(dev)))
        assert not dev.value
        s.release(0)
        assert s.bytes_copied() == nbytes
        assert int(lib.tpb_stream_transfer_stream(s.s)) != 0
        # the whole-layer path still works beside it
        assert torch.equal(s.acquire(1)[0].cpu(), torch.from_numpy(layer(12, nbytes)[0]))
        s.release(1)
    finally:
        s.close()
