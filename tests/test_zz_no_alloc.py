"""The allocation-free decode linear (tpb_q8_0_gemv_static) against the regular
entry points.

Some hosts may not let this library allocate device memory: an engine that keeps
the whole GPU in its own budgeted arena, or a decode loop that cannot afford the
device-wide synchronisation a cudaMalloc implies.  For them the quantised
activations live in a fixed array inside the library.  This test calls the entry
point through the C ABI several times in a row, with different shapes, so every call
after the first runs over the previous call's leftovers, and expects exactly what
tpb_q8_1_quantize + tpb_q8_0_gemv_q8n produce (same kernels, so bit-identical,
which is inside the few-ulp tolerance the other GEMV tests use).  It also watches
the device's free memory (cudaMemGetInfo) across the calls: it must not move.

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


def _static_into(be, y, x, w_dev, m, n, k):
    rc = be.lib.tpb_q8_0_gemv_static(be.h, be._stream(), y.data_ptr(), x.data_ptr(), m,
                                     w_dev.data_ptr(), C.c_float(0.25), n, k)
    assert rc == 0, be.lib.tpb_last_error(be.h)


# (m, n, k): 8 rows x 5120 columns (the streaming kernel); fewer, shorter rows (stale tail in the
# array); the size limit, 8 x 32768 (activations too large for shared memory); a row length the
# streaming kernel cannot take (96 columns: rows of 102 bytes), which runs the plain kernel.
CASES = ((8, 512, 5120, 11), (3, 200, 1024, 12), (8, 96, 32768, 13), (2, 40, 96, 14))


def test_static_scratch_gemv_matches_regular_entry_points_in_a_row():
    from tensorpencil_b200.backend import Backend
    be = Backend(0)
    try:
        prepared = []
        for m, n, k, seed in CASES:
            g = synth.q8_0_gemv(m, n, k, seed=seed)
            x = torch.from_numpy(g["x"]).cuda()
            w_dev = torch.from_numpy(g["w"]).cuda()
            want = _regular(be, x, w_dev, n, k)
            y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
            prepared.append((m, n, k, x, w_dev, want, y))
        # first call on this device: looks the array's address up (and loads the kernels)
        m, n, k, x, w_dev, want, y = prepared[0]
        _static_into(be, y, x, w_dev, m, n, k)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        for _ in range(2):
            for m, n, k, x, w_dev, want, y in prepared:
                y.fill_(float("nan"))
                _static_into(be, y, x, w_dev, m, n, k)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        be.status_poll()
        assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
        for m, n, k, x, w_dev, want, y in prepared:
            assert torch.equal(y, want), (m, n, k, float((y - want).abs().max()))
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
