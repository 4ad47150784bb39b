"""The allocation-free decode linear (tpb_q8_0_gemv_static) against the regular
entry points.

Some hosts may not let this library allocate device memory: an engine that keeps
the whole GPU in its own budgeted arena, or a decode loop that cannot afford the
device-wide synchronisation a cudaMalloc implies.  For them the quantised
activations live in a fixed array inside the library.  This test calls the entry
point through the C ABI twice in a row, with different shapes, so the second call
runs over the first call's leftovers, and expects exactly what
tpb_q8_1_quantize + tpb_q8_0_gemv_q8n produce (same kernels, so bit-identical,
which is inside the few-ulp tolerance the other GEMV tests use).

Collected last on purpose (file name), so a run that stops at the first failure
has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from tensorpencil_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu


def _regular(be, x, w, n, k):
    return be.q8_0_linear(x, w, n, k, scale=0.25)


def _static(be, x, w_dev, m, n, k):
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    rc = be.lib.tpb_q8_0_gemv_static(be.h, be._stream(), y.data_ptr(), x.data_ptr(), m,
                                     w_dev.data_ptr(), C.c_float(0.25), n, k)
    assert rc == 0, be.lib.tpb_last_error(be.h)
    return y


def test_static_scratch_gemv_matches_regular_entry_points_twice():
    from tensorpencil_b200.backend import Backend
    be = Backend(0)
    try:
        # call 1: 8 rows x 5120 columns (fast path); call 2: fewer, shorter rows (stale tail in the array)
        for m, n, k, seed in ((8, 512, 5120, 11), (3, 200, 1024, 12)):
            g = synth.q8_0_gemv(m, n, k, seed=seed)
            x = torch.from_numpy(g["x"]).cuda()
            w_dev = torch.from_numpy(g["w"]).cuda()
            want = _regular(be, x, w_dev, n, k)
            got = _static(be, x, w_dev, m, n, k)
            torch.cuda.synchronize()
            be.status_poll()
            assert torch.equal(got, want), float((got - want).abs().max())
    finally:
        be.close()


def test_static_scratch_gemv_rejects_oversize():
    from tensorpencil_b200._lib import TPB_ERR_INVALID_ARG
    from tensorpencil_b200.backend import Backend
    be = Backend(0)
    try:
        x = torch.zeros(8 * 32768 + 32, device="cuda")
        y = torch.zeros(16, device="cuda")
        w = torch.zeros(64, dtype=torch.uint8, device="cuda")
        # 8 rows of 32800 columns: one block per row beyond the fixed array
        rc = be.lib.tpb_q8_0_gemv_static(be.h, be._stream(), y.data_ptr(), x.data_ptr(), 8,
                                         w.data_ptr(), C.c_float(1.0), 1, 32800)
        assert rc == TPB_ERR_INVALID_ARG
        assert b"exceeds the fixed scratch" in be.lib.tpb_last_error(be.h)
        rc = be.lib.tpb_q8_0_gemv_static(be.h, be._stream(), y.data_ptr(), x.data_ptr(), 9,
                                         w.data_ptr(), C.c_float(1.0), 1, 256)
        assert rc == TPB_ERR_INVALID_ARG
    finally:
        be.close()
