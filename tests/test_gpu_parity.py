"""GPU parity tests: the CUDA path (called through the C ABI) against the CPU
oracle on the same seeded inputs.

Parity ladder, as the reference's own device tests apply it
(src/gpu/cuda/kernels.zig:2208-2301, :2411-2529, :2557-2701):
  1. quantised activations and per-token scales  -- bit-exact
  2. int32 accumulators (raw-s32 output)         -- bit-exact
  3. dequantised output vs the integer replica   -- 1e-3 relative / 1e-4 absolute
  4. output vs the `--backend cpu` float path    -- rel-L2 <= 0.03 (int8 gate)
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tensorpencil_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3
ABS_TOL = 1e-4


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assert_close_to_sim(y, sim):
    y = np.asarray(y, np.float64)
    err = np.abs(y - sim)
    ok = err <= ABS_TOL + REL_TOL * np.abs(sim)
    assert ok.all(), f"max abs err {err.max():.3e}, worst rel {np.max(err / (np.abs(sim) + 1e-30)):.3e}"


# ---------------------------------------------------------------------------------
# K1: activation prep
# ---------------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k", [(1, 256), (7, 512), (33, 768), (129, 1024), (64, 1280),
                                 (256, 3072), (40, 6144), (24, 12288), (16, 16384), (5, 32768)])
def test_prep_bit_exact(be, bits, m, k):
    x = synth.activations(m, k, seed=10 * m + bits)
    q_ref, s_ref = oracle.convrot_prep(x, bits)
    be._prep(dev(x), m, k, bits)
    be.status_poll()
    q = be.i8_x[: m * k].cpu().numpy().reshape(m, k)
    s = be.i8_scale[:m].cpu().numpy()
    asum = be.i8_sum[:m].cpu().numpy()
    assert np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(q, q_ref), f"{np.count_nonzero(q != q_ref)} of {q.size} quantised values differ"
    assert np.array_equal(asum, q_ref.astype(np.int32).sum(axis=1))


def test_prep_edge_values(be):
    """All-zero rows take the 1e-12 floor scale; exact half-way quotients round
    away from zero; huge and tiny magnitudes survive."""
    k = 512
    x = np.zeros((6, k), np.float32)
    x[1, 3] = 1.0                      # a single spike: after rotation every |v| is 1/16
    x[2] = synth.activations(1, k, 5)[0] * 1e-20
    x[3] = synth.activations(1, k, 6)[0] * 1e20
    x[4, :256] = np.arange(256) % 7 - 3  # small integers: many exact ties after scaling
    x[5] = 127.0 * 0.5                   # constant row
    for bits in (8, 4):
        q_ref, s_ref = oracle.convrot_prep(x, bits)
        be._prep(dev(x), 6, k, bits)
        q = be.i8_x[: 6 * k].cpu().numpy().reshape(6, k)
        s = be.i8_scale[:6].cpu().numpy()
        assert np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
        assert np.array_equal(q, q_ref)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_prep_half_inputs(be, dtype):
    m, k = 19, 1536
    x = synth.activations(m, k, seed=77)
    xt = torch.from_numpy(x).to(getattr(torch, dtype))
    x_as_f32 = xt.to(torch.float32).numpy()
    q_ref, s_ref = oracle.convrot_prep(x_as_f32, 8)
    be._prep(xt.cuda(), m, k, 8)
    assert np.array_equal(be.i8_scale[:m].cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(be.i8_x[: m * k].cpu().numpy().reshape(m, k), q_ref)


def test_prep_rejects_bad_shapes(be):
    from tensorpencil_b200._lib import TPB_ERR_INVALID_ARG, TpbError
    x = torch.zeros(4, 300, device="cuda")
    with pytest.raises(TpbError) as e:
        be._prep(x, 4, 300, 8)
    assert e.value.status == TPB_ERR_INVALID_ARG
    with pytest.raises(TpbError):
        be._prep(torch.zeros(2, 256, device="cuda"), 2, 256, 5)


# ---------------------------------------------------------------------------------
# K2: int8 GEMM, raw int32 accumulators
# ---------------------------------------------------------------------------------

def run_gemm(be, q, s, asum, w, ws, n, k, out_dtype, w_bits=8, ldy=None):
    m = q.shape[0]
    be.i8_x = dev(q.reshape(-1))
    be.i8_scale = dev(s)
    be.i8_sum = dev(asum.astype(np.int32))
    be.i8_m, be.i8_cols, be.i8_bits = m, k, w_bits
    ld = n if ldy is None else ldy
    y = torch.zeros((m, ld), dtype=out_dtype, device="cuda")
    be._gemm(y, dev(w), dev(ws), n, w_bits, ldy=ld)
    be.status_poll()
    return y.cpu()


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 256), (256, 384, 512), (128, 256, 6144),      # the reference's exact-integer cases (k rounded to 256)
    (1, 16, 256), (7, 48, 256), (129, 80, 512), (200, 272, 768), (16, 8 * 16, 1024),
    (300, 1040, 512),                                         # BN=64, ragged m and n
    (1024, 2432, 512),                                        # BN=128 (152 tiles)
    (2048, 4096, 256), (1100, 5136, 512),                     # BN=256 (>=148 tiles), ragged n
])
def test_gemm_raw_s32_exact(be, m, n, k):
    rng = np.random.default_rng(m * 7 + n)
    q = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-128, 128, size=(n, k), dtype=np.int8)
    want = oracle.igemm_s32(q, w)
    got = run_gemm(be, q, np.ones(m, np.float32), np.zeros(m), w, np.ones(n, np.float32), n, k,
                   torch.int32).numpy()
    bad = np.count_nonzero(got != want)
    assert bad == 0, f"{bad} of {got.size} accumulators differ"


@pytest.mark.parametrize("out", ["int32", "float32", "bfloat16"])
def test_gemm_ragged_tail_repeated(be, out):
    """Tiles that hang over the right and bottom edges skip some of their stores;
    repeat the launch to shake out any ordering slip between staging buffers."""
    m, n, k = 1100, 5136, 512
    rng = np.random.default_rng(99)
    q = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-128, 128, size=(n, k), dtype=np.int8)
    s = rng.uniform(0.5, 1.5, m).astype(np.float32)
    ws = rng.uniform(0.5, 1.5, n).astype(np.float32)
    acc = oracle.igemm_s32(q, w)
    want32 = (acc.astype(np.float32) * s[:, None]) * ws[None, :]
    want = {"int32": torch.from_numpy(acc), "float32": torch.from_numpy(want32),
            "bfloat16": torch.from_numpy(want32).to(torch.bfloat16)}[out]
    be.i8_x, be.i8_scale, be.i8_sum = dev(q.reshape(-1)), dev(s), dev(np.zeros(m, np.int32))
    be.i8_m, be.i8_cols, be.i8_bits = m, k, 8
    wd, wsd = dev(w), dev(ws)
    for _ in range(25):
        y = torch.zeros((m, n), dtype=getattr(torch, out), device="cuda")
        be._gemm(y, wd, wsd, n, 8)
        assert torch.equal(y.cpu(), want)
    be.status_poll()


def test_gemm_extreme_values_no_overflow_surprises(be):
    m, n, k = 128, 128, 8192
    q = np.full((m, k), -127, np.int8)
    w = np.full((n, k), -128, np.int8)
    got = run_gemm(be, q, np.ones(m, np.float32), np.zeros(m), w, np.ones(n, np.float32), n, k,
                   torch.int32).numpy()
    assert np.all(got == 127 * 128 * k)


def test_gemm_respects_ldy_and_leaves_padding_untouched(be):
    m, n, k, ld = 70, 96, 256, 128
    rng = np.random.default_rng(3)
    q = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    got = run_gemm(be, q, np.ones(m, np.float32), np.zeros(m), w, np.ones(n, np.float32), n, k,
                   torch.int32, ldy=ld).numpy()
    assert np.array_equal(got[:, :n], oracle.igemm_s32(q, w))
    assert np.all(got[:, n:] == 0)


# ---------------------------------------------------------------------------------
# full ConvRot linear (prep + GEMM + fused dequant)
# ---------------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,n,k", [(128, 128, 1024), (128, 256, 6144), (128, 128, 16384),
                                   (256, 384, 6144), (77, 208, 2048)])
def test_linear_vs_replica(be, bits, m, n, k):
    c = synth.convrot_linear(m, n, k, bits, seed=9 + m + bits)
    q_ref, s_ref, acc_ref, sim = oracle.convrot_linear_sim(c["x"], c["w_i8"], c["w_scale"], bits)
    w = c["w_packed"] if bits == 4 else c["w_i8"]
    x = dev(c["x"])
    y = be.convrot_linear(x, w, c["w_scale"], n, bits, torch.float32)
    acc = be.convrot_linear(x, w, c["w_scale"], n, bits, torch.int32)
    yb = be.convrot_linear(x, w, c["w_scale"], n, bits, torch.bfloat16)
    be.status_poll()
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert_close_to_sim(y.cpu().numpy(), sim)
    # the f32 result is exactly (float(acc) * as) * ws in f32
    want32 = (acc_ref.astype(np.float32) * s_ref[:, None]) * c["w_scale"][None, :]
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want32.view(np.uint32))
    # bf16 output = f32 result rounded to nearest-even bf16
    want16 = torch.from_numpy(want32).to(torch.bfloat16)
    assert torch.equal(yb.cpu(), want16)


def test_config0_full_ladder(be):
    """BASELINE config 0: INT8 ConvRot linear, M=256, K=N=3072."""
    c = synth.config0()
    q_ref, s_ref, acc_ref, sim = oracle.convrot_linear_sim(c["x"], c["w_i8"], c["w_scale"], 8)
    x = dev(c["x"])
    y = be.convrot_linear(x, c["w_i8"], c["w_scale"], 3072, 8, torch.float32).cpu().numpy()
    q = be.i8_x[: 256 * 3072].cpu().numpy().reshape(256, 3072)
    s = be.i8_scale[:256].cpu().numpy()
    acc = be.convrot_linear(x, c["w_i8"], c["w_scale"], 3072, 8, torch.int32).cpu().numpy()
    be.status_poll()
    assert np.array_equal(q, q_ref)                                   # rung 1
    assert np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(acc, acc_ref)                               # rung 2
    assert_close_to_sim(y, sim)                                       # rung 3
    y_cpu = oracle.linear_cpu_backend(c["x"], c["w_i8"], 8, c["w_scale"], 3072, 3072)
    rel = np.sqrt(np.sum((y - y_cpu.astype(np.float64)) ** 2) / np.sum(y_cpu.astype(np.float64) ** 2))
    assert rel <= 0.03, rel                                           # rung 4


def test_config1_full_size_sampled(be):
    """BASELINE config 1 at full size (M=4608, K=3072, N=12288, INT4): the whole
    prep output is checked exactly; accumulators and outputs are checked on a
    random sample of rows (the oracle's triple loop over everything would take
    minutes), plus a size-independent property: doubling x leaves q unchanged
    and doubles every scale and output."""
    c = synth.config1()
    m, n, k = 4608, 12288, 3072
    x = dev(c["x"])
    y = be.convrot_linear(x, c["w_packed"], c["w_scale"], n, 4, torch.float32)
    q = be.i8_x[: m * k].cpu().numpy().reshape(m, k)
    s = be.i8_scale[:m].cpu().numpy()
    acc = be.convrot_linear(x, c["w_packed"], c["w_scale"], n, 4, torch.int32).cpu().numpy()
    be.status_poll()
    q_ref, s_ref = oracle.convrot_prep(c["x"], 4)
    assert np.array_equal(q, q_ref)
    assert np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
    rows = np.sort(np.random.default_rng(0).choice(m, 96, replace=False))
    acc_ref = oracle.igemm_s32(q_ref[rows], c["w_i8"])
    assert np.array_equal(acc[rows], acc_ref)
    sim = oracle.dequant_sim(acc_ref, s_ref[rows], c["w_scale"])
    assert_close_to_sim(y.cpu().numpy()[rows], sim)
    # scaling property
    y2 = be.convrot_linear(x * 2.0, c["w_packed"], c["w_scale"], n, 4, torch.float32)
    assert np.array_equal(be.i8_x[: m * k].cpu().numpy().reshape(m, k), q)
    assert torch.equal(y2, y * 2.0)


@pytest.mark.parametrize("m,n,k", [(2048, 4864, 1024), (1100, 5136, 512)])
def test_int4_fused_unpack_kernel(be, monkeypatch, m, n, k):
    """The opt-in kernel that unpacks the packed weight in shared memory inside the
    GEMM (TPB_W4_FUSED=1) gives the same accumulators and outputs as the default
    route (expand to int8, then the int8 kernel) and as the replica."""
    c = synth.convrot_linear(m, n, k, 4, seed=m + n)
    x = dev(c["x"])
    wp, wsc = dev(c["w_packed"]), dev(c["w_scale"])
    monkeypatch.delenv("TPB_W4_FUSED", raising=False)
    acc_default = be.convrot_linear(x, wp, wsc, n, 4, torch.int32).clone()
    y_default = be.convrot_linear(x, wp, wsc, n, 4, torch.float32).clone()
    monkeypatch.setenv("TPB_W4_FUSED", "1")       # read once, when a handle is created
    from tensorpencil_b200.backend import Backend
    bf = Backend(0)
    try:
        for _ in range(3):
            acc_fused = bf.convrot_linear(x, wp, wsc, n, 4, torch.int32)
            y_fused = bf.convrot_linear(x, wp, wsc, n, 4, torch.float32)
            yb_fused = bf.convrot_linear(x, wp, wsc, n, 4, torch.bfloat16)
            bf.status_poll()
            assert torch.equal(acc_fused, acc_default)
            assert torch.equal(y_fused, y_default)
            assert torch.equal(yb_fused, y_default.to(torch.bfloat16))
        rows = np.sort(np.random.default_rng(1).choice(m, 48, replace=False))
        q_ref, s_ref = oracle.convrot_prep(c["x"][rows], 4)
        assert np.array_equal(acc_fused.cpu().numpy()[rows], oracle.igemm_s32(q_ref, c["w_i8"]))
    finally:
        bf.close()


def test_w4_expand_matches_nibble_decode(be):
    rng = np.random.default_rng(4)
    w = rng.integers(-8, 8, size=(48, 512), dtype=np.int8)
    packed = dev(synth.pack_i4(w))
    out = torch.empty((48, 512), dtype=torch.int8, device="cuda")
    rc = be.lib.tpb_convrot_w4_expand(be.h, be._stream(), packed.data_ptr(), 48, 512, out.data_ptr())
    assert rc == 0
    assert np.array_equal(out.cpu().numpy(), w)


# ---------------------------------------------------------------------------------
# K4: Q8_0 GEMV
# ---------------------------------------------------------------------------------

def test_q8_1_quantize_bit_exact(be):
    rng = np.random.default_rng(1337)
    x = (rng.random(3 * 512, dtype=np.float32) * 2 - 1).astype(np.float32)
    x[64:96] = 0
    be.opGemvQuantizeX(dev(x), x.size)
    raw = be.q8_act[: x.size // 32 * 4 + x.size].cpu().numpy()
    d = raw[: x.size // 32 * 4].view(np.float32)
    qs = raw[x.size // 32 * 4:].view(np.int8)
    d_ref, qs_ref = oracle.q8_1_quantize(x, tie_mode=0)
    assert np.array_equal(d.view(np.uint32), d_ref.view(np.uint32))
    assert np.array_equal(qs, qs_ref)


def gemv_tolerance(w, n, k, x):
    """Float accumulation order is not pinned by the reference (its gate is 2e-2
    absolute); bound the error by a few ulps of the sum of |terms| instead."""
    wf = np.abs(np.stack([oracle.q8_0_dequant_row(w[r], k) for r in range(min(n, 64))]))
    mag = (np.abs(x).astype(np.float64) @ wf.astype(np.float64).T).max()
    return 1e-5 * mag + 1e-6


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("n,k", [(24, 512), (16, 512), (64, 2048), (37, 1280), (100, 5120), (8, 96)])
def test_q8_0_gemv_q8n_vs_oracle(be, m, n, k):
    g = synth.q8_0_gemv(m, n, k, seed=271 + m)
    y = be.q8_0_linear(dev(g["x"]), g["w"], n, k, scale=0.5).cpu().numpy()
    be.status_poll()
    want = oracle.q8_0_gemv_q8(g["w"], n, k, g["x"], scale=0.5, tie_mode=0)
    tol = gemv_tolerance(g["w"], n, k, g["x"])
    assert np.max(np.abs(y - want)) <= tol, (np.max(np.abs(y - want)), tol)
    # and within the reference's own gate of the tie-away emulation it tests against
    want_ref = oracle.q8_0_gemv_q8(g["w"], n, k, g["x"], scale=0.5, tie_mode=1)
    assert np.max(np.abs(y - want_ref)) <= 2e-2


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n,k", [(1, 17408), (7, 17408), (100, 24576), (33, 32768), (600, 16384), (9, 49152), (300, 12288)])
@pytest.mark.parametrize("route", ["default", "mma", "mma, K in one CTA", "dp4a"])
def test_q8_0_gemv_long_rows(be, monkeypatch, m, n, k, route):
    """Rows too long for one CTA's registers: K split over a CTA pair, several passes over K, both
    together, and the same calls forced down the other routes -- every route within a few ulps of
    the sum of |terms| of the q8_1-emulating reference (src/gpu/cuda/backend.zig:3641-3651)."""
    if route != "default":
        monkeypatch.setenv("TPB_GEMV_KERNEL", "dp4a" if route == "dp4a" else "mma")
    if route == "mma, K in one CTA":
        monkeypatch.setenv("TPB_GEMV_KSPLIT", "0")
    g = synth.q8_0_gemv(m, n, k, seed=911 + m)
    y = be.q8_0_linear(dev(g["x"]), g["w"], n, k, scale=0.25).cpu().numpy()
    be.status_poll()
    be.dropWeights()
    want = oracle.q8_0_gemv_q8(g["w"], n, k, g["x"], scale=0.25, tie_mode=0)
    tol = gemv_tolerance(g["w"], n, k, g["x"])
    assert np.max(np.abs(y - want)) <= tol, (np.max(np.abs(y - want)), tol)


def test_q8_0_gemv_more_than_8_rows_groups(be):
    g = synth.q8_0_gemv(19, 32, 1024, seed=5)
    y = be.q8_0_linear(dev(g["x"]), g["w"], 32, 1024).cpu().numpy()
    want = oracle.q8_0_gemv_q8(g["w"], 32, 1024, g["x"])
    assert np.max(np.abs(y - want)) <= gemv_tolerance(g["w"], 32, 1024, g["x"])


@pytest.mark.parametrize("down", [False, True])
@pytest.mark.parametrize("m", [1, 4, 8])
def test_config2_full_size(be, m, down):
    """BASELINE config 2: K=5120 -> N=17408 and the down projection."""
    g = synth.config2(m=m, down=down)
    n, k = g["n"], g["k"]
    y = be.q8_0_linear(dev(g["x"]), g["w"], n, k).cpu().numpy()
    be.status_poll()
    be.dropWeights()
    want = oracle.q8_0_gemv_q8(g["w"], n, k, g["x"])
    assert np.max(np.abs(y - want)) <= gemv_tolerance(g["w"], n, k, g["x"])
    y64 = oracle.q8_0_gemv_f64(g["w"], n, k, g["x"])
    rel = np.sqrt(np.sum((y - y64) ** 2) / np.sum(y64 ** 2))
    assert rel < 0.05  # the reference's q8_0 small-m gate (src/ops/matmul.zig:1138-1165)


@pytest.mark.parametrize("n,k", [(16, 512), (40, 5120), (9, 96)])
def test_q8_0_gemv_f32(be, n, k):
    g = synth.q8_0_gemv(1, n, k, seed=4242)
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    be.opGemvQuant("q8_0", y, dev(g["x"][0]), g["w"], 1.0, n, k)
    want = oracle.q8_0_gemv_f64(g["w"], n, k, g["x"])[0]
    assert np.max(np.abs(y.cpu().numpy() - want)) <= 2e-2  # the reference's gate
    assert np.max(np.abs(y.cpu().numpy() - want)) <= gemv_tolerance(g["w"], n, k, g["x"]) * 10


# ---------------------------------------------------------------------------------
# weight streaming
# ---------------------------------------------------------------------------------

def test_streamed_forward_bit_identical_to_resident(be):
    """Streamed vs resident forward must be bit-identical (the reference's
    cuda-stream-test, src/main.zig:1288-1304)."""
    from tensorpencil_b200.offload import Streamer
    layers = 5
    m, n, k = 64, 256, 512
    rng = np.random.default_rng(1)
    ws = [synth.convrot_weights(n, k, 8, seed=50 + i) for i in range(layers)]
    x = dev(synth.activations(m, k, seed=3))
    resident = [be.convrot_linear(x, w["w_i8"], w["w_scale"], n, 8).clone() for w in ws]
    st = Streamer(be, budget_bytes=2 * (n * k + 4 * n), slot_bytes=n * k + 4 * n, n_slots=2)
    for i, w in enumerate(ws):
        st.register(i, [w["w_i8"], w["w_scale"]])
    st.prefetch(0)
    outs = []
    for i in range(layers):
        wq, wsc = st.acquire(i)
        if i + 1 < layers:
            st.prefetch(i + 1)
        be.opI8Prep(x, m, k)
        y = torch.empty((m, n), dtype=torch.float32, device="cuda")
        be.opI8Gemm(y, wq, wsc, n)
        st.release(i)
        outs.append(y)
    torch.cuda.synchronize()
    for a, b in zip(outs, resident):
        assert torch.equal(a, b)
    assert st.bytes_copied() == layers * (n * k + 4 * n)
    st.close()
    del rng


# ---------------------------------------------------------------------------------
# Host-buffer entry: pinned x in, pinned y out, pipelined in row chunks
# ---------------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,chunk", [(700, 256), (512, 512), (130, 512), (1100, 300)])
def test_host_buffer_linear_matches_resident(be, bits, m, chunk):
    n, k = 1024, 768
    c = synth.convrot_linear(m, n, k, bits, seed=77 + m + bits)
    w = dev(c["w_i8"] if bits == 8 else c["w_packed"])
    ws = dev(c["w_scale"])
    y_dev = be.convrot_linear(dev(c["x"]), w, ws, n, bits)
    x_pin = torch.from_numpy(c["x"]).pin_memory()
    y_pin = torch.full((m, n), float("nan"), dtype=torch.float32).pin_memory()
    for _ in range(2):                      # second call reuses the staging buffers and streams
        be.convrot_linear_host(x_pin, w, ws, n, bits, y_pin, chunk_rows=chunk)
        torch.cuda.current_stream().synchronize()   # the call makes the current stream wait for the last download
        assert np.array_equal(y_pin.numpy().view(np.uint32), y_dev.cpu().numpy().view(np.uint32))
        y_pin.fill_(float("nan"))
    be.status_poll()
    q, s = oracle.convrot_prep(c["x"], bits)
    sim = oracle.dequant_sim(oracle.igemm_s32(q, c["w_i8"]), s, c["w_scale"])
    assert_close_to_sim(y_dev.cpu().numpy(), sim)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(96, 768, 512), (4608, 3072, 256), (700, 1040, 768)])
def test_one_call_linear_matches_prep_then_gemm(be, bits, dtype, m, n, k):
    """tpb_convrot_linear == tpb_convrot_prep + tpb_convrot_gemm, bit for bit, also when
    called back to back."""
    c = synth.convrot_linear(m, n, k, bits, seed=5 + m + bits)
    x = dev(c["x"])
    w = dev(c["w_i8"] if bits == 8 else c["w_packed"])
    ws = dev(c["w_scale"])
    y_two = torch.empty((m, n), dtype=dtype, device="cuda")
    be._prep(x, m, k, bits)
    be._gemm(y_two, w, ws, n, bits)
    q_two = be.i8_x[: m * k].clone()
    for _ in range(3):
        y_one = be.convrot_linear(x, w, ws, n, bits, out_dtype=dtype)
    be.status_poll()
    view = torch.int16 if dtype == torch.bfloat16 else torch.int32
    assert torch.equal(y_one.view(view), y_two.view(view))
    assert torch.equal(be.i8_x[: m * k], q_two)
