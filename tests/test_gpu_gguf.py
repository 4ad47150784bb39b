"""Decode GEMV for the other GGUF block formats (q4_0, q4_k, q5_k, q6_k) through the C ABI,
against the CPU truth the reference's own device test uses
(src/gpu/cuda/backend.zig:3727-3792): dequantised weight row times q8_1-dequantised
activations, f64 accumulation.  The weight decoders behind that truth are pinned bit for
bit to the reference's golden super-blocks (tests/test_oracle.py).

Tolerance: the kernel accumulates in f32, so the error is bounded relative to the sum of
the absolute products, not to the (possibly cancelling) result: |err| <= 2e-5 * sum|w||x|.
The reference's gate for the same comparison is 2e-2 absolute at cols = 512.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tensorpencil_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu

FORMATS = ["q4_0", "iq4_nl", "q4_k", "q5_k", "q6_k", "q8_0"]


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


def run(be, fmt, w, n, k, x):
    m = x.shape[0]
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    be.opGemvQuantizeX(torch.from_numpy(x).cuda(), m * k)
    wd = torch.from_numpy(w).cuda()
    for r0 in range(0, m, 8):
        ng = min(8, m - r0)
        be.opGemvQuantQ8N(fmt, y[r0:], wd, 1.0, n, k, ng, r0, m)
    be.status_poll()
    return y.cpu().numpy()


def bound(fmt, w, n, k, x):
    d, qs = oracle.q8_1_quantize(x.reshape(-1))
    xh = (np.repeat(d, 32) * qs.astype(np.float32)).reshape(x.shape)
    wf = np.stack([oracle.gguf_dequant_row(fmt, w[r], k) for r in range(n)])
    return np.abs(xh).astype(np.float64) @ np.abs(wf).astype(np.float64).T


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("n,k", [(24, 512), (40, 256), (129, 2048), (64, 5120), (7, 8192)])
def test_gguf_gemv_matches_truth(be, fmt, m, n, k):
    w = synth.gguf_weights(fmt, n, k, seed=n + k)
    x = (np.random.default_rng(m + k).random((m, k), dtype=np.float32) * 2 - 1).astype(np.float32)
    got = run(be, fmt, w, n, k, x)
    want = oracle.gguf_gemv_q8(fmt, w, n, k, x)
    err = np.abs(got.astype(np.float64) - want)
    assert (err <= 2e-5 * bound(fmt, w, n, k, x) + 1e-6).all(), f"max err {err.max():.3e}"
    assert np.abs(got - want).max() <= 2e-2 * max(1.0, k / 512)          # the reference's own gate, scaled with k


@pytest.mark.parametrize("fmt", ["q4_0", "iq4_nl", "q4_k", "q5_k", "q6_k"])
def test_gguf_gemv_reference_test_shape(be, fmt):
    """rows 24, cols 512, 5 activation rows in one partial group: the reference's case."""
    w = synth.gguf_weights(fmt, 24, 512, seed=314)
    x = (np.random.default_rng(4242).random((5, 512), dtype=np.float32) * 2 - 1).astype(np.float32)
    got = run(be, fmt, w, 24, 512, x)
    want = oracle.gguf_gemv_q8(fmt, w, 24, 512, x)
    assert np.abs(got - want).max() <= 2e-2


@pytest.mark.parametrize("fmt", ["q4_k", "q5_k", "q6_k"])
def test_gguf_gemv_config2_size(be, fmt):
    """N = 17408, K = 5120 (the decode MLP shape), M = 1 and 8, against the truth on a row sample."""
    n, k = 17408, 5120
    w = synth.gguf_weights(fmt, n, k, seed=2)
    x = (np.random.default_rng(3).standard_normal((8, k))).astype(np.float32)
    got8 = run(be, fmt, w, n, k, x)
    got1 = run(be, fmt, w, n, k, x[:1])
    assert np.array_equal(got1[0], got8[0])          # the same row gives the same bits in any group size
    rows = np.arange(0, n, 61)
    want = oracle.gguf_gemv_q8(fmt, w[rows], rows.size, k, x)
    err = np.abs(got8[:, rows].astype(np.float64) - want)
    assert (err <= 2e-5 * bound(fmt, w[rows], rows.size, k, x) + 1e-6).all(), f"max err {err.max():.3e}"


@pytest.mark.parametrize("fmt", ["q4_0", "iq4_nl", "q4_k", "q5_k", "q6_k"])
@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("n,k", [(1, 256), (15, 5120), (16, 17408), (333, 17408), (2500, 1024), (40, 6144)])
def test_gguf_gemv_ring_kernel_gives_the_per_warp_kernels_bits(be, fmt, m, n, k, monkeypatch):
    """One or two activation rows take a second kernel (one producer warp, sixteen-row stages) where rows are
    long or many; it adds the same terms in the same order, so forcing either kernel gives identical bits --
    ragged row counts, rows of one and of several chunks -- and both match the truth."""
    w = synth.gguf_weights(fmt, n, k, seed=7 * n + k)
    x = (np.random.default_rng(m + n).standard_normal((m, k))).astype(np.float32)
    monkeypatch.setenv("TPB_GEMVK_KERNEL", "ring")
    ring = run(be, fmt, w, n, k, x)
    monkeypatch.setenv("TPB_GEMVK_KERNEL", "warp")
    warp = run(be, fmt, w, n, k, x)
    monkeypatch.delenv("TPB_GEMVK_KERNEL")
    auto = run(be, fmt, w, n, k, x)
    assert np.array_equal(ring, warp) and np.array_equal(auto, warp)
    want = oracle.gguf_gemv_q8(fmt, w, n, k, x)
    err = np.abs(ring.astype(np.float64) - want)
    assert (err <= 2e-5 * bound(fmt, w, n, k, x) + 1e-6).all(), f"max err {err.max():.3e}"


@pytest.mark.parametrize("fmt", ["q4_0", "q4_k", "q5_k", "q6_k"])
def test_gguf_gemv_group_too_large_for_shared_memory_is_split(be, fmt):
    """Eight activation rows of 17408 columns take 209 KB of shared memory, more than the kernels can spare; the
    library then runs the group as two launches.  Same bits as the rows run one at a time, and the truth."""
    n, k = 48, 17408
    w = synth.gguf_weights(fmt, n, k, seed=91)
    x = (np.random.default_rng(92).standard_normal((8, k))).astype(np.float32)
    got8 = run(be, fmt, w, n, k, x)
    for r in (0, 3, 7):
        assert np.array_equal(run(be, fmt, w, n, k, x[r:r + 1])[0], got8[r])
    want = oracle.gguf_gemv_q8(fmt, w, n, k, x)
    err = np.abs(got8.astype(np.float64) - want)
    assert (err <= 2e-5 * bound(fmt, w, n, k, x) + 1e-6).all(), f"max err {err.max():.3e}"


def test_gguf_gemv_rejects_bad_arguments(be):
    from tensorpencil_b200 import _lib
    y = torch.zeros(8, device="cuda")
    w = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    xq = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    f = be.lib.tpb_gguf_gemv_q8n
    assert f(be.h, None, 9, y.data_ptr(), w.data_ptr(), 1.0, 8, 256, xq.data_ptr(), 1, 0, 1) == _lib.TPB_ERR_INVALID_ARG
    assert f(be.h, None, 2, y.data_ptr(), w.data_ptr(), 1.0, 8, 288, xq.data_ptr(), 1, 0, 1) == _lib.TPB_ERR_INVALID_ARG
    assert f(be.h, None, 2, y.data_ptr(), w.data_ptr(), 1.0, 8, 256, xq.data_ptr(), 9, 0, 9) == _lib.TPB_ERR_INVALID_ARG
    assert be.lib.tpb_gguf_row_bytes(2, 5120) == 20 * 144 and be.lib.tpb_gguf_row_bytes(3, 5120) == 20 * 176


def test_q6k_weight_at_the_very_end_of_its_allocation(be):
    """q6_k rows (210 bytes per 256 columns) are not multiples of 16 bytes, and the kernel's bulk
    copies round the last row's copy out to the next 16-byte boundary.  The weight is placed so
    that its last byte is the last byte but two of a torch allocation (7 rows of 2 super-blocks =
    2940 bytes, 12 short of a multiple of 16): the rounded copy ends exactly at the allocation's
    end, never beyond it, and the results are those of the same weight elsewhere in memory."""
    n, k = 7, 512
    w = synth.gguf_weights("q6_k", n, k, seed=3)
    nbytes = w.size
    assert nbytes % 16 == 12
    x = (np.random.default_rng(8).random((3, k), dtype=np.float32) * 2 - 1).astype(np.float32)
    want = run(be, "q6_k", w, n, k, x)
    total = 1 << 20                                   # a whole allocator block of its own
    store = torch.zeros(total, dtype=torch.uint8, device="cuda")
    off = total - (nbytes + 4)                        # 16-byte aligned start, 4 spare bytes at the end
    assert off % 16 == 0 and store.data_ptr() % 512 == 0
    store[off:off + nbytes] = torch.from_numpy(w.reshape(-1)).cuda()
    y = torch.empty((3, n), dtype=torch.float32, device="cuda")
    be.opGemvQuantizeX(torch.from_numpy(x).cuda(), 3 * k)
    be.opGemvQuantQ8N("q6_k", y, store[off:off + nbytes], 1.0, n, k, 3, 0, 3)
    be.status_poll()
    assert np.array_equal(y.cpu().numpy(), want)
