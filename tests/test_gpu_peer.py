"""The GEMM with the all-gather fused into its epilogue, on ONE GPU: the two ranks'
launches run one after the other on the same device, writing into two ordinary
buffers that play the two ranks' copies of y (neither launch waits for the other).
The two-GPU run over NVLink is in test_gpu_multi.py.

Also the bounded barrier: alone (world 1) it passes; with a second rank's flag that
nothing ever sets it gives up after its limit, reports TPB_ERR_TIMEOUT through
status_poll, and the context keeps working."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tensorpencil_b200 import _lib, synth  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


def _ydt(dt):
    return {torch.float32: _lib.TPB_F32, torch.bfloat16: _lib.TPB_BF16, torch.int32: _lib.TPB_S32}[dt]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
@pytest.mark.parametrize("m,n,k,world", [(300, 1024, 512, 2), (4608, 12288, 256, 2), (130, 2048, 256, 4),
                                         (1100, 4640, 512, 2)])
def test_fused_allgather_epilogue_single_device(be, bits, dtype, m, n, k, world):
    c = synth.convrot_linear(m, n, k, bits, seed=m + n + bits)
    x = torch.from_numpy(c["x"]).cuda()
    w = torch.from_numpy(c["w_i8"] if bits == 8 else c["w_packed"]).cuda()
    ws = torch.from_numpy(c["w_scale"]).cuda()
    be._prep(x, m, k, bits)
    # single launch over all of n: what every rank's y must equal, bit for bit
    y_one = torch.empty((m, n), dtype=dtype, device="cuda")
    be._gemm(y_one, w, ws, n, bits)
    ys = [torch.full((m, n), -7, dtype=dtype, device="cuda") for _ in range(world)]
    y_all = (C.c_void_p * world)(*[t.data_ptr() for t in ys])
    ns = n // world
    for r in range(world):
        rc = be.lib.tpb_convrot_gemm_allgather(
            be.h, be._stream(), y_all, world, r, _ydt(dtype), n, be.i8_x.data_ptr(), be.i8_scale.data_ptr(),
            be.i8_sum.data_ptr() if bits == 4 else None, w[r * ns:(r + 1) * ns].data_ptr(), bits,
            ws[r * ns:(r + 1) * ns].data_ptr(), m, ns, k)
        be._check(rc)
    be.status_poll()
    for r in range(world):
        assert torch.equal(ys[r].view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           y_one.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), f"copy {r} differs"
    if dtype == torch.int32 and m * n * k <= 300 * 1024 * 512:
        q, _ = oracle.convrot_prep(c["x"], bits)
        assert np.array_equal(ys[0].cpu().numpy(), oracle.igemm_s32(q, c["w_i8"]))


def test_fused_allgather_rejects_bad_arguments(be):
    y = torch.empty((16, 64), dtype=torch.float32, device="cuda")
    y_all = (C.c_void_p * 2)(y.data_ptr(), y.data_ptr())
    q = torch.zeros((16, 256), dtype=torch.int8, device="cuda")
    s = torch.ones(64, dtype=torch.float32, device="cuda")
    args = (y_all, 2, 0, _lib.TPB_F32)
    tail = (q.data_ptr(), s.data_ptr(), None, q.data_ptr(), 8, s.data_ptr(), 16, 32, 256)
    assert be.lib.tpb_convrot_gemm_allgather(be.h, None, *args, 48, *tail) == _lib.TPB_ERR_INVALID_ARG   # ldy < world*n_shard
    assert be.lib.tpb_convrot_gemm_allgather(be.h, None, y_all, 9, 0, _lib.TPB_F32, 64, *tail) == _lib.TPB_ERR_INVALID_ARG
    assert be.lib.tpb_convrot_gemm_allgather(be.h, None, y_all, 2, 2, _lib.TPB_F32, 64, *tail) == _lib.TPB_ERR_INVALID_ARG


def test_barrier_alone_and_timeout(be):
    flags = torch.zeros(128, dtype=torch.int32, device="cuda")
    mine = (C.c_void_p * 1)(flags.data_ptr())
    for epoch in (1, 2, 3):
        be._check(be.lib.tpb_peer_barrier(be.h, be._stream(), mine, 1, 0, epoch, 1000))
    be.status_poll()
    assert int(flags[0]) == 3
    # world 2, and the other rank never arrives: the wait runs out after 50 ms
    other = torch.zeros(128, dtype=torch.int32, device="cuda")
    both = (C.c_void_p * 2)(flags.data_ptr(), other.data_ptr())
    be._check(be.lib.tpb_peer_barrier(be.h, be._stream(), both, 2, 0, 4, 50))
    with pytest.raises(_lib.TpbError) as e:
        be.status_poll()
    assert "wait expired" in str(e.value)
    assert int(other[0]) == 4          # our announcement did reach the other rank's row
    # the context is still usable and the status word is clear again
    be._check(be.lib.tpb_peer_barrier(be.h, be._stream(), mine, 1, 0, 5, 1000))
    be.status_poll()
