"""The elementwise neighbours of the linears (silu_mul, sigmoid_mul, rms_mod, gated_add)
and the activation prep with the producers fused in.

Ladder:
  1. stand-alone ops vs the CPU oracle -- 2e-6 absolute (the reference tests' own gate,
     src/ops/act.zig:162-176, src/ops/norm.zig:84-96) plus 3e-6 relative for large values;
  2. fused prep vs stand-alone op followed by the plain prep -- bit-exact (quantised
     values, scales, row sums), f32 and bf16 inputs, int8 and int4;
  3. fused prep vs the oracle end to end -- scales to 1e-5 relative, quantised values
     equal except for rounding ties moved by the 1e-6 input differences (off by one on
     fewer than 1 in 1000 values).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402
from tensorpencil_b200 import _lib  # noqa: E402

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-6, 3e-6
EPS = 1e-5      # src/models/dit.zig:40


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


def rnd(shape, seed, scale=1.5):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


SHAPES = [(3, 256), (17, 768), (64, 3072), (33, 12288), (5, 32768), (130, 1280)]


@pytest.mark.parametrize("m,k", SHAPES)
def test_standalone_ops_match_oracle(be, m, k):
    g, u = rnd((m, k), 1, 2.5), rnd((m, k), 2)
    a = dev(g)
    be.siluMul(a, dev(u), m * k)
    assert np.allclose(a.cpu().numpy(), oracle.silu_mul(g, u), rtol=RTOL, atol=ATOL)
    a = dev(u)
    be.sigmoidMul(a, dev(g), m * k)
    assert np.allclose(a.cpu().numpy(), oracle.sigmoid_mul(u, g), rtol=RTOL, atol=ATOL)
    mod = rnd((6 * k,), 3, 0.3)
    mod[:k] += 1.0                                   # premul = 1 + scale
    out = torch.empty((m, k), dtype=torch.float32, device="cuda")
    be.rmsMod(dev(u), out, dev(mod), m, k, 0, 4 * k, EPS)
    assert np.allclose(out.cpu().numpy(), oracle.rms_mod(u, mod[:k], mod[4 * k:5 * k], EPS), rtol=RTOL, atol=ATOL)
    x = dev(g)
    be.gatedAdd(x, dev(u), dev(mod), m * k, k, 2 * k)
    assert np.allclose(x.cpu().numpy(), oracle.gated_add(g, u, mod[2 * k:3 * k]), rtol=RTOL, atol=ATOL)
    be.status_poll()


def _prepped(be, m, k):
    return (be.i8_x[: m * k].clone(), be.i8_scale[:m].clone(), be.i8_sum[:m].clone())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k", SHAPES)
def test_fused_prep_is_bit_identical_to_two_steps(be, dtype, bits, m, k):
    g, u = dev(rnd((m, k), 11, 2.5)).to(dtype), dev(rnd((m, k), 12)).to(dtype)
    mod = rnd((6 * k,), 13, 0.3)
    mod[:k] += 1.0
    mod = dev(mod)
    act = torch.empty((m, k), dtype=torch.float32, device="cuda")

    def check(name):
        fused = _prepped(be, m, k)
        be._prep(act, m, k, bits)
        two = _prepped(be, m, k)
        for f, t, what in zip(fused, two, ("q", "scale", "sum")):
            assert torch.equal(f.view(torch.int8 if what == "q" else torch.int32),
                               t.view(torch.int8 if what == "q" else torch.int32)), f"{name}: {what} differs"

    # silu_mul
    be._check(be.lib.tpb_silu_mul(be.h, be._stream(), g.data_ptr(), u.data_ptr(), _lib.TPB_F32 if dtype == torch.float32
                                  else _lib.TPB_BF16, act.data_ptr(), m * k))
    be.prepSiluMul(g, u, m, k, bits)
    check("silu_mul")
    # sigmoid_mul
    be._check(be.lib.tpb_sigmoid_mul(be.h, be._stream(), u.data_ptr(), g.data_ptr(), _lib.TPB_F32 if dtype == torch.float32
                                     else _lib.TPB_BF16, act.data_ptr(), m * k))
    be.prepSigmoidMul(u, g, m, k, bits)
    check("sigmoid_mul")
    # rms_mod
    be.rmsMod(u, act, mod, m, k, 0, 4 * k, EPS)
    be.prepRmsMod(u, mod, m, k, 0, 4 * k, EPS, bits)
    check("rms_mod")
    be.status_poll()


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k", [(64, 3072), (33, 12288)])
def test_fused_prep_vs_oracle(be, bits, m, k):
    g, u = rnd((m, k), 21, 2.5), rnd((m, k), 22)
    mod = rnd((6 * k,), 23, 0.3)
    mod[:k] += 1.0
    cases = {
        "silu_mul": (lambda: be.prepSiluMul(dev(g), dev(u), m, k, bits), oracle.silu_mul(g, u)),
        "sigmoid_mul": (lambda: be.prepSigmoidMul(dev(u), dev(g), m, k, bits), oracle.sigmoid_mul(u, g)),
        "rms_mod": (lambda: be.prepRmsMod(dev(u), dev(mod), m, k, 0, 4 * k, EPS, bits),
                    oracle.rms_mod(u, mod[:k], mod[4 * k:5 * k], EPS)),
    }
    for name, (run, act_ref) in cases.items():
        run()
        q = be.i8_x[: m * k].cpu().numpy().reshape(m, k).astype(np.int32)
        s = be.i8_scale[:m].cpu().numpy()
        q_ref, s_ref = oracle.convrot_prep(act_ref, bits)
        assert np.allclose(s, s_ref, rtol=1e-5, atol=0), name
        d = np.abs(q - q_ref.astype(np.int32))
        assert d.max() <= 1, name
        assert np.count_nonzero(d) < 1e-3 * d.size, f"{name}: {np.count_nonzero(d)} of {d.size} values differ"
        assert np.array_equal(be.i8_sum[:m].cpu().numpy(), q.sum(axis=1)), name
    be.status_poll()


def test_fused_linear_end_to_end(be):
    """mlp.down as the block runs it: y = ConvRotLinear(silu(gate) * up), fused prep, vs
    the integer replica fed the oracle's activation."""
    from tensorpencil_b200 import synth
    m, n, k = 96, 768, 3072
    c = synth.convrot_linear(m, n, k, 8, seed=31)
    g, u = rnd((m, k), 32, 2.0), rnd((m, k), 33)
    be.prepSiluMul(dev(g), dev(u), m, k, 8)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    be.opI8Gemm(y, dev(c["w_i8"]), dev(c["w_scale"]), n)
    be.status_poll()
    q = be.i8_x[: m * k].cpu().numpy().reshape(m, k)
    s = be.i8_scale[:m].cpu().numpy()
    sim = oracle.dequant_sim(oracle.igemm_s32(q, c["w_i8"]), s, c["w_scale"])     # replica on the GPU's own q
    err = np.abs(y.cpu().numpy().astype(np.float64) - sim)
    assert (err <= 1e-4 + 1e-3 * np.abs(sim)).all()
    truth = oracle.linear_truth(oracle.rotate(oracle.silu_mul(g, u)), c["w_i8"], c["w_scale"])
    rel = np.linalg.norm(y.cpu().numpy() - truth) / np.linalg.norm(truth)
    assert rel <= 0.03, rel                                                        # the reference's int8 gate


def test_fused_prep_rejects_bad_arguments(be):
    a = torch.zeros((4, 256), dtype=torch.float32, device="cuda")
    q = torch.zeros((4, 256), dtype=torch.int8, device="cuda")
    s = torch.zeros(4, dtype=torch.float32, device="cuda")
    f = be.lib.tpb_convrot_prep_fused
    ok_tail = (_lib.TPB_F32, 4, 256, 8, q.data_ptr(), s.data_ptr(), None)
    assert f(be.h, None, 0, a.data_ptr(), a.data_ptr(), None, None, 0.0, *ok_tail) == _lib.TPB_ERR_INVALID_ARG   # op
    assert f(be.h, None, 1, a.data_ptr(), None, None, None, 0.0, *ok_tail) == _lib.TPB_ERR_INVALID_ARG           # no b
    assert f(be.h, None, 3, a.data_ptr(), None, None, None, 0.0, *ok_tail) == _lib.TPB_ERR_INVALID_ARG           # no mod
    assert f(be.h, None, 1, a.data_ptr(), a.data_ptr(), None, None, 0.0, _lib.TPB_F16, 4, 256, 8, q.data_ptr(),
             s.data_ptr(), None) == _lib.TPB_ERR_INVALID_ARG                                                      # dtype
    assert f(be.h, None, 1, a.data_ptr(), a.data_ptr(), None, None, 0.0, _lib.TPB_F32, 4, 250, 8, q.data_ptr(),
             s.data_ptr(), None) == _lib.TPB_ERR_INVALID_ARG                                                      # k
    assert f(be.h, None, 1, a.data_ptr(), a.data_ptr(), None, None, 0.0, _lib.TPB_F32, 4, 256, 4, q.data_ptr(),
             s.data_ptr(), None) == _lib.TPB_ERR_INVALID_ARG                                                      # act_sum


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,n,k", [(96, 768, 512), (300, 1040, 256), (4608, 3072, 256), (1100, 3072, 768)])
def test_gemm_with_gated_residual_is_bit_identical_to_two_steps(be, bits, m, n, k):
    """x += gate * linear(...) in the GEMM epilogue == f32 GEMM then gated_add, bit for bit
    (one-CTA kernels for the small shapes, the CTA-pair kernel for the large ones)."""
    from tensorpencil_b200 import synth
    c = synth.convrot_linear(m, n, k, bits, seed=41 + m)
    w = dev(c["w_i8"] if bits == 8 else c["w_packed"])
    ws = dev(c["w_scale"])
    x0 = rnd((m, n), 42)
    mod = dev(rnd((3 * n,), 43, 0.2))
    be._prep(dev(c["x"]), m, k, bits)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    be._gemm(y, w, ws, n, bits)
    two = dev(x0)
    be.gatedAdd(two, y, mod, m * n, n, n)
    one = dev(x0)
    be.gemmGatedAdd(one, w, ws, n, mod, n, bits)
    be.status_poll()
    assert torch.equal(one.view(torch.int32), two.view(torch.int32))
    if m * n * k <= 300 * 1040 * 256:
        q = be.i8_x[: m * k].cpu().numpy().reshape(m, k)
        s = be.i8_scale[:m].cpu().numpy()
        sim = oracle.dequant_sim(oracle.igemm_s32(q, c["w_i8"]), s, c["w_scale"])
        want = x0.astype(np.float64) + mod.cpu().numpy()[n:2 * n].astype(np.float64) * sim
        err = np.abs(one.cpu().numpy() - want)
        assert (err <= 1e-4 + 1e-3 * np.abs(want)).all()


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,n,k", [(96, 768, 512), (300, 1040, 256), (129, 128, 1024), (4608, 3072, 256), (1100, 12288, 768)])
def test_gemm_with_silu_pair_is_bit_identical_to_three_steps(be, bits, m, n, k):
    """silu(gate projection) * (up projection) in one launch == the two f32 GEMMs followed by silu_mul, bit
    for bit; the bf16 output is that result rounded to nearest even; and the whole agrees with the
    oracle's integer replica + silu_mul (src/ops/act.zig) to the usual 1e-3 / 1e-4."""
    from tensorpencil_b200 import synth
    cg = synth.convrot_linear(m, n, k, bits, seed=51 + m)
    cu = synth.convrot_linear(m, n, k, bits, seed=52 + m)
    key = "w_i8" if bits == 8 else "w_packed"
    wg, wu = dev(cg[key]), dev(cu[key])
    sg, su = dev(cg["w_scale"]), dev(cu["w_scale"])
    be._prep(dev(cg["x"]), m, k, bits)
    g = torch.empty((m, n), dtype=torch.float32, device="cuda")
    u = torch.empty_like(g)
    be._gemm(g, wg, sg, n, bits)
    be._gemm(u, wu, su, n, bits)
    be.siluMul(g, u, m * n)                                    # in place: g = silu(g) * u
    one = torch.empty((m, n), dtype=torch.float32, device="cuda")
    be.gemmSiluPair(one, wg, sg, wu, su, n, bits)
    one16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    be.gemmSiluPair(one16, wg, sg, wu, su, n, bits)
    be.status_poll()
    assert torch.equal(one.view(torch.int32), g.view(torch.int32))
    assert torch.equal(one16, g.to(torch.bfloat16))
    if m * n * k <= 300 * 1040 * 256:
        q = be.i8_x[: m * k].cpu().numpy().reshape(m, k)
        s = be.i8_scale[:m].cpu().numpy()
        vg = oracle.dequant_sim(oracle.igemm_s32(q, cg["w_i8"]), s, cg["w_scale"])
        vu = oracle.dequant_sim(oracle.igemm_s32(q, cu["w_i8"]), s, cu["w_scale"])
        want = vg / (1.0 + np.exp(-vg)) * vu
        err = np.abs(one.cpu().numpy() - want)
        assert (err <= 1e-4 + 1e-3 * np.abs(want)).all()


def test_gemm_with_silu_pair_into_a_wider_buffer_and_bad_arguments(be):
    from tensorpencil_b200 import synth
    m, n, k = 200, 256, 512
    cg = synth.convrot_linear(m, n, k, 8, seed=61)
    cu = synth.convrot_linear(m, n, k, 8, seed=62)
    wg, wu, sg, su = dev(cg["w_i8"]), dev(cu["w_i8"]), dev(cg["w_scale"]), dev(cu["w_scale"])
    be._prep(dev(cg["x"]), m, k, 8)
    wide = torch.full((m, n + 64), -7.0, dtype=torch.float32, device="cuda")
    be.gemmSiluPair(wide[:, :n], wg, sg, wu, su, n, 8)           # ldy = n + 64
    tight = torch.empty((m, n), dtype=torch.float32, device="cuda")
    be.gemmSiluPair(tight, wg, sg, wu, su, n, 8)
    be.status_poll()
    assert torch.equal(wide[:, :n], tight) and bool((wide[:, n:] == -7.0).all())
    L = be.lib
    args = lambda y_dt, w2: (be.h, None, tight.data_ptr(), y_dt, n, be.i8_x.data_ptr(), be.i8_scale.data_ptr(), None,
                             wg.data_ptr(), sg.data_ptr(), w2, su.data_ptr(), 8, m, n, k)
    assert L.tpb_convrot_gemm_silu_pair(*args(_lib.TPB_S32, wu.data_ptr())) == _lib.TPB_ERR_INVALID_ARG   # raw sums make no sense here
    assert L.tpb_convrot_gemm_silu_pair(*args(_lib.TPB_F32, None)) == _lib.TPB_ERR_INVALID_ARG            # second weight missing


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("count", [1, 2, 3, 4])
@pytest.mark.parametrize("m,n,k", [(2048, 3072, 512), (2500, 2064, 256), (300, 512, 256)])
def test_gemm_group_is_bit_identical_to_separate_gemms(be, bits, count, m, n, k):
    """Several weights of one shape on the same prepped activations in one launch (the q, k, v and gate
    projections of a block): every output equals the separate GEMM's, bit for bit, f32 and bf16 -- on a
    problem the two-CTA kernel takes, one with ragged edges, and one small enough for the one-by-one path."""
    from tensorpencil_b200 import synth
    cs = [synth.convrot_linear(m, n, k, bits, seed=71 + 3 * g + m) for g in range(count)]
    key = "w_i8" if bits == 8 else "w_packed"
    ws = [dev(c[key]) for c in cs]
    sc = [dev(c["w_scale"]) for c in cs]
    be._prep(dev(cs[0]["x"]), m, k, bits)
    for dt in (torch.float32, torch.bfloat16):
        want = []
        for g in range(count):
            y = torch.empty((m, n), dtype=dt, device="cuda")
            be._gemm(y, ws[g], sc[g], n, bits)
            want.append(y)
        got = [torch.full((m, n), 3.0, dtype=dt, device="cuda") for _ in range(count)]
        be.gemmGroup(got, ws, sc, n, bits)
        be.status_poll()
        for g in range(count):
            assert torch.equal(got[g], want[g]), f"weight {g}, {dt}"


def test_gemm_group_into_wider_buffers_and_bad_arguments(be):
    from tensorpencil_b200 import synth
    m, n, k = 2048, 3072, 256
    cs = [synth.convrot_linear(m, n, k, 8, seed=81 + g) for g in range(2)]
    ws, sc = [dev(c["w_i8"]) for c in cs], [dev(c["w_scale"]) for c in cs]
    be._prep(dev(cs[0]["x"]), m, k, 8)
    wide = [torch.full((m, n + 128), -7.0, dtype=torch.float32, device="cuda") for _ in range(2)]
    be.gemmGroup([t[:, :n] for t in wide], ws, sc, n, 8)         # ldy = n + 128
    tight = [torch.empty((m, n), dtype=torch.float32, device="cuda") for _ in range(2)]
    be.gemmGroup(tight, ws, sc, n, 8)
    be.status_poll()
    for g in range(2):
        assert torch.equal(wide[g][:, :n], tight[g]) and bool((wide[g][:, n:] == -7.0).all())
    import ctypes as C
    L = be.lib
    arr = C.c_void_p * 2
    ys, wp, sp = arr(*[t.data_ptr() for t in tight]), arr(*[w.data_ptr() for w in ws]), arr(*[t.data_ptr() for t in sc])
    call = lambda cnt, y_dt, y_, w_: L.tpb_convrot_gemm_group(be.h, None, cnt, y_, y_dt, n, be.i8_x.data_ptr(),
                                                              be.i8_scale.data_ptr(), None, w_, sp, 8, m, n, k)
    assert call(2, _lib.TPB_F32, ys, wp) == _lib.TPB_OK
    assert call(0, _lib.TPB_F32, ys, wp) == _lib.TPB_ERR_INVALID_ARG
    assert call(5, _lib.TPB_F32, ys, wp) == _lib.TPB_ERR_INVALID_ARG
    assert call(2, _lib.TPB_S32, ys, wp) == _lib.TPB_ERR_INVALID_ARG          # dequantised outputs only
    assert call(2, _lib.TPB_F32, ys, arr(ws[0].data_ptr(), None)) == _lib.TPB_ERR_INVALID_ARG   # a weight missing
    assert call(2, _lib.TPB_F32, None, wp) == _lib.TPB_ERR_INVALID_ARG
    be.status_poll()
