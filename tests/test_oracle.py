"""Pins the CPU oracle against the reference's own golden vectors and
known-answer tests for the quantized-linear path.  No GPU needed.

Mirrors: src/ops/convrot.zig:91-192 (Hadamard properties + ComfyUI int4
fixture), src/core/dtype.zig:264-280 (nibble decode), src/core/quants.zig:118-120
(Q8_0 golden bits), src/ops/matmul.zig:932-1070 (ConvRot matmul vs naive f64).
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from tensorpencil_b200 import synth


# -- Hadamard / rotation (convrot.zig:91-139) ---------------------------------

def test_hadamard_symmetric():
    h = oracle.hadamard256()
    assert np.array_equal(h, h.T)


def test_hadamard_orthonormal():
    h = oracle.hadamard256()
    assert np.allclose(h @ h, np.eye(256, dtype=np.float32), atol=1e-5)


def test_rotation_self_inverse():
    rng = np.random.default_rng(7)
    v = rng.standard_normal(256).astype(np.float32)
    assert np.allclose(oracle.rotate(oracle.rotate(v)), v, atol=1e-4)


def test_rotation_matches_matvec_multi_group():
    rng = np.random.default_rng(11)
    data = rng.standard_normal(512).astype(np.float32)
    got = oracle.rotate(data)
    h = oracle.hadamard256()
    for g in range(2):
        want = h @ data[g * 256:(g + 1) * 256]
        assert np.allclose(got[g * 256:(g + 1) * 256], want, atol=1e-4)


def test_rotation_add_order_is_the_reference_one():
    """One radix-4 pass on values where float association matters: the four
    outputs must be ((a+b)+c)-d, ((a+b)-c)+d, ((a-b)+c)+d, ((-a+b)+c)+d
    (src/ops/convrot.zig:68-71)."""
    rng = np.random.default_rng(3)
    v = (rng.standard_normal(256) * np.array([1e4, 1.0, 1e-3, 37.0] * 64)).astype(np.float32)
    w = v.copy()
    f = np.float32
    for s in (1, 4, 16, 64):
        nxt = w.copy()
        for base in range(0, 256, 4 * s):
            for o in range(s):
                p = base + o
                a, b, c, d = f(w[p]), f(w[p + s]), f(w[p + 2 * s]), f(w[p + 3 * s])
                nxt[p] = f(f(f(a + b) + c) - d)
                nxt[p + s] = f(f(f(a + b) - c) + d)
                nxt[p + 2 * s] = f(f(f(a - b) + c) + d)
                nxt[p + 3 * s] = f(f(f(-a + b) + c) + d)
        w = nxt
    w = (w / f(16.0)).astype(np.float32)
    assert np.array_equal(oracle.rotate(v).view(np.uint32), w.view(np.uint32))


# -- nibble decode (dtype.zig:264-280) -----------------------------------------

def test_nibble_known_answers():
    assert oracle.nibble_i4(0xF7, 0) == 7
    assert oracle.nibble_i4(0xF7, 1) == -1
    assert oracle.nibble_i4(0x80, 0) == 0
    assert oracle.nibble_i4(0x80, 1) == -8


def test_pack_unpack_round_trip():
    rng = np.random.default_rng(5)
    v = rng.integers(-8, 8, size=(3, 64), dtype=np.int8)
    p = oracle.pack_i4(v)
    assert np.array_equal(p, synth.pack_i4(v))
    assert np.array_equal(oracle.unpack_i4(p), v)
    assert np.array_equal(synth.unpack_i4(p), v)


# -- ComfyUI int4 ConvRot fixture (convrot.zig:148-192) -------------------------

def test_int4_convrot_fixture(golden_dir):
    rows, cols = 16, 6144
    packed = np.fromfile(os.path.join(golden_dir, "int4_convrot_weight.u8"), np.uint8)
    scale = np.fromfile(os.path.join(golden_dir, "int4_convrot_scale.f32"), np.float32)
    expected = np.fromfile(os.path.join(golden_dir, "int4_convrot_expected.f32"), np.float32)
    assert packed.size == rows * cols // 2 and scale.size == rows and expected.size == rows * cols
    got = oracle.i4_convrot_dequant(packed, scale, rows, cols).astype(np.float64).ravel()
    rel = np.sqrt(np.sum((expected - got) ** 2) / np.sum(expected.astype(np.float64) ** 2))
    assert rel < 1e-4, rel  # the reference's gate


# -- Q8_0 golden block (quants_fixtures.zig:6-15) --------------------------------

def test_q8_0_golden_bits(golden_dir):
    g = json.load(open(os.path.join(golden_dir, "q8_0_block.json")))
    blk = np.array(g["block_bytes"], np.uint8)
    assert blk.size == 34
    got = oracle.q8_0_dequant_row(blk, 32)
    want = np.array(g["expected_f32_bits"], np.uint32)
    assert np.array_equal(got.view(np.uint32), want)


def test_f16_conversion_matches_numpy():
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(h)) for h in hs], np.float32)
    ok = np.isnan(want) | (got.view(np.uint32) == want.view(np.uint32))
    assert ok.all()


# -- replica vs committed oracle vectors ----------------------------------------

@pytest.mark.parametrize("bits", [8, 4])
def test_replica_matches_committed_vectors(golden_dir, bits):
    g = np.load(os.path.join(golden_dir, "oracle_vectors.npz"))
    q, s, acc, y = oracle.convrot_linear_sim(g[f"i{bits}_x"], g[f"i{bits}_w"], g[f"i{bits}_ws"], bits)
    assert np.array_equal(q, g[f"i{bits}_q"])
    assert np.array_equal(s.view(np.uint32), g[f"i{bits}_as"].view(np.uint32))
    assert np.array_equal(acc, g[f"i{bits}_acc"])
    assert np.array_equal(y, g[f"i{bits}_y"])


def test_replica_quantiser_definition():
    """q = clamp(round_half_away(xr / s)), s = max(amax/maxq, 1e-12), in f32
    (src/gpu/cuda/kernels.zig:2638-2653)."""
    x = synth.activations(4, 768, seed=9)
    for bits, maxq, lo in ((8, 127.0, -127), (4, 7.0, -8)):
        q, s, xr = oracle.convrot_prep(x, bits, want_rotated=True)
        assert np.array_equal(xr.view(np.uint32), oracle.rotate(x).view(np.uint32))
        amax = np.abs(xr).max(axis=1)
        s_want = np.maximum(amax / np.float32(maxq), np.float32(1e-12)).astype(np.float32)
        assert np.array_equal(s.view(np.uint32), s_want.view(np.uint32))
        r = (xr / s_want[:, None]).astype(np.float32)
        q_want = np.clip(np.sign(r) * np.floor(np.abs(r) + np.float32(0.5)), lo, int(maxq))
        assert np.array_equal(q, q_want.astype(np.int8))
        assert np.abs(q).max() == int(maxq)  # absmax element hits full scale


def test_prep_all_zero_row_uses_floor_scale():
    x = np.zeros((2, 256), np.float32)
    q, s = oracle.convrot_prep(x, 8)
    assert np.all(q == 0) and np.all(s == np.float32(1e-12))


def test_igemm_exact_vs_numpy():
    rng = np.random.default_rng(7)
    for m, n, k in ((16, 8, 32), (64, 256, 128), (48, 72, 320)):  # kernels.zig:2208-2231, :2327-2333
        a = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
        w = rng.integers(-128, 128, size=(n, k), dtype=np.int8)
        want = a.astype(np.int32) @ w.astype(np.int32).T
        assert np.array_equal(oracle.igemm_s32(a, w), want)


# -- `--backend cpu` float path (matmul.zig:932-1070) ----------------------------

@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,n,k", [(1, 16, 256), (7, 33, 512), (13, 40, 768), (20, 64, 1024)])
def test_cpu_backend_matches_naive_f64(bits, m, n, k):
    c = synth.convrot_linear(m, n, k, bits, seed=100 + m)
    w = c["w_packed"] if bits == 4 else c["w_i8"]
    y = oracle.linear_cpu_backend(c["x"], w, bits, c["w_scale"], n, k)
    # naive f64 over the un-rotated weight
    wd = oracle.rotate((c["w_i8"].astype(np.float32) * c["w_scale"][:, None]).astype(np.float32))
    e = c["x"].astype(np.float64) @ wd.astype(np.float64).T
    tol = 1e-3 + 1e-5 * np.abs(e) * np.sqrt(k)
    assert np.all(np.abs(y - e) <= tol)


def test_cpu_backend_is_a_sequential_fma_chain():
    """The packed path accumulates one FMA per k, k ascending, per output
    (matmul.zig:611-619), whatever the k-blocking or thread split."""
    c = synth.convrot_linear(3, 16, 1024, 8, seed=77)
    y = oracle.linear_cpu_backend(c["x"], c["w_i8"], 8, c["w_scale"], 16, 1024, path="packed")
    y1 = oracle.linear_cpu_backend(c["x"], c["w_i8"], 8, c["w_scale"], 16, 1024, nthreads=1, path="packed")
    assert np.array_equal(y, y1)
    wd = oracle.rotate((c["w_i8"].astype(np.float32) * c["w_scale"][:, None]).astype(np.float32))
    import math
    for i in range(3):
        for j in (0, 5, 15):
            acc = np.float32(0)
            for kk in range(1024):
                # fma(a, b, acc) rounded once: evaluate exactly in f64 then round
                acc = np.float32(math.fma(float(c["x"][i, kk]), float(wd[j, kk]), float(acc))) \
                    if hasattr(math, "fma") else np.float32(np.float64(c["x"][i, kk]) * np.float64(wd[j, kk]) + np.float64(acc))
            assert abs(float(acc) - float(y[i, j])) <= 2e-6 * max(1.0, abs(float(acc)))


@pytest.mark.parametrize("bits", [8, 4])
def test_cpu_backend_small_m_path(bits):
    """Fewer than 16 activation rows take the reference's small-m path (matmul.zig:152, :669-767):
    eight lane-wise partial sums over k, multiply and add rounded separately, reduced lane 0..7,
    then the scalar tail and the bias.  Checked against that recipe spelled out in numpy, against
    the packed path (another summation order of the same products: close, not equal), and for
    independence from the thread split; 16 rows and more dispatch to the packed path."""
    m, n, k = 5, 24, 1024 + 256       # ConvRot needs k % 256 == 0, so the scalar tail is empty here
    c = synth.convrot_linear(m, n, k, bits, seed=90 + bits)
    w = c["w_packed"] if bits == 4 else c["w_i8"]
    bias = np.random.default_rng(4).standard_normal(n).astype(np.float32)
    y = oracle.linear_cpu_backend(c["x"], w, bits, c["w_scale"], n, k, bias=bias)
    assert np.array_equal(y, oracle.linear_cpu_backend(c["x"], w, bits, c["w_scale"], n, k, bias=bias, path="small"))
    assert np.array_equal(y, oracle.linear_cpu_backend(c["x"], w, bits, c["w_scale"], n, k, bias=bias, nthreads=1))
    wd = oracle.rotate((c["w_i8"].astype(np.float32) * c["w_scale"][:, None]).astype(np.float32))
    for t in (0, m - 1):
        for r in (0, 7, n - 1):
            prod = (c["x"][t] * wd[r]).astype(np.float32).reshape(-1, 8)      # rounded products, 8 lanes
            acc = np.zeros(8, np.float32)
            for row in prod:
                acc = (acc + row).astype(np.float32)
            s = acc[0]
            for lane in range(1, 8):
                s = np.float32(s + acc[lane])
            s = np.float32(np.float32(s + np.float32(0)) + bias[r])
            assert y[t, r] == s, (t, r, y[t, r], s)
    yp = oracle.linear_cpu_backend(c["x"], w, bits, c["w_scale"], n, k, bias=bias, path="packed")
    assert not np.array_equal(y, yp)
    assert np.allclose(y, yp, rtol=2e-5, atol=2e-4 * np.sqrt(k))
    # the dispatch threshold: 15 rows small-m, 16 rows packed
    c16 = synth.convrot_linear(16, n, 512, bits, seed=95)
    w16 = c16["w_packed"] if bits == 4 else c16["w_i8"]
    assert np.array_equal(oracle.linear_cpu_backend(c16["x"], w16, bits, c16["w_scale"], n, 512),
                          oracle.linear_cpu_backend(c16["x"], w16, bits, c16["w_scale"], n, 512, path="packed"))
    assert np.array_equal(oracle.linear_cpu_backend(c16["x"][:15], w16, bits, c16["w_scale"], n, 512),
                          oracle.linear_cpu_backend(c16["x"][:15], w16, bits, c16["w_scale"], n, 512, path="small"))


def test_cpu_backend_bias_and_no_convrot():
    rng = np.random.default_rng(2)
    c = synth.convrot_linear(4, 24, 256, 8, seed=5)
    b = rng.standard_normal(24).astype(np.float32)
    y = oracle.linear_cpu_backend(c["x"], c["w_i8"], 8, c["w_scale"], 24, 256, convrot=0, bias=b)
    e = c["x"].astype(np.float64) @ (c["w_i8"].astype(np.float64) * c["w_scale"][:, None]).T + b
    assert np.allclose(y, e, rtol=1e-4, atol=1e-3)


def test_int_path_close_to_float_path_int8():
    """Activation-quantisation noise of the integer replica against the float
    path stays within the reference's accuracy gate (rel-L2 <= 0.03,
    kernels.zig:2700)."""
    c = synth.convrot_linear(32, 64, 1024, 8, seed=31)
    _, _, _, y_int = oracle.convrot_linear_sim(c["x"], c["w_i8"], c["w_scale"], 8)
    y_f = oracle.linear_cpu_backend(c["x"], c["w_i8"], 8, c["w_scale"], 64, 1024)
    rel = np.sqrt(np.sum((y_int - y_f) ** 2) / np.sum(y_f.astype(np.float64) ** 2))
    assert rel < 0.03, rel


# -- Q8_0 GEMV ---------------------------------------------------------------------

def test_q8_1_quantise_definition():
    rng = np.random.default_rng(1337)
    x = (rng.random(512, dtype=np.float32) * 2 - 1).astype(np.float32)
    x[32:64] = 0  # amax == 0 block -> d = 0, q = 0
    d, qs = oracle.q8_1_quantize(x)
    amax = np.abs(x.reshape(-1, 32)).max(axis=1)
    assert np.array_equal(d, (amax / np.float32(127.0)).astype(np.float32))
    assert np.all(qs[32:64] == 0) and d[1] == 0
    inv = np.where(amax == 0, 0, np.float32(127.0) / np.where(amax == 0, 1, amax)).astype(np.float32)
    want = np.rint((x.reshape(-1, 32) * inv[:, None]).astype(np.float32)).astype(np.int8).ravel()
    assert np.array_equal(qs, want)
    assert np.abs(qs.reshape(-1, 32)).max(axis=1)[0] == 127


def test_q8_0_gemv_f64_matches_numpy():
    g = synth.q8_0_gemv(3, 16, 512, seed=4242)
    y = oracle.q8_0_gemv_f64(g["w"], 16, 512, g["x"], scale=0.5)
    wf = np.stack([oracle.q8_0_dequant_row(g["w"][r], 512) for r in range(16)])
    want = 0.5 * (g["x"].astype(np.float64) @ wf.astype(np.float64).T)
    assert np.allclose(y, want, rtol=1e-6, atol=1e-6)


def test_q8_0_gemv_q8_close_to_f64():
    # same relation the reference tests rely on (matmul.zig:1138-1165: rel-L2 < 0.05)
    g = synth.q8_0_gemv(2, 24, 512, seed=271)
    y64 = oracle.q8_0_gemv_f64(g["w"], 24, 512, g["x"])
    yq = oracle.q8_0_gemv_q8(g["w"], 24, 512, g["x"])
    rel = np.sqrt(np.sum((y64 - yq) ** 2) / np.sum(y64 ** 2))
    assert rel < 0.05, rel


def test_q8_0_block_sumi():
    g = synth.q8_0_gemv(2, 8, 256, seed=12)
    _, xq = oracle.q8_1_quantize(g["x"])
    s = oracle.q8_0_block_sumi(g["w"], 8, 256, xq)
    qw = g["w"].reshape(8, 8, 34)[:, :, 2:].view(np.int8).astype(np.int32)
    want = np.einsum("rbe,tbe->trb", qw, xq.reshape(2, 8, 32).astype(np.int32))
    assert np.array_equal(s, want)


def test_committed_q8_vectors(golden_dir):
    g = np.load(os.path.join(golden_dir, "oracle_vectors.npz"))
    assert np.array_equal(oracle.q8_0_gemv_f64(g["q8_w"], 16, 512, g["q8_x"]), g["q8_y_f64"])
    assert np.array_equal(oracle.q8_0_gemv_q8(g["q8_w"], 16, 512, g["q8_x"]), g["q8_y_q8"])
    d, qs = oracle.q8_1_quantize(g["q8_x"])
    assert np.array_equal(d, g["q8_act_d"]) and np.array_equal(qs, g["q8_act_qs"])


# ---------------------------------------------------------------------------------
# Elementwise neighbours: pinned to the reference's own fixtures
# (src/ops/act.zig:153-158 and :176-188, src/ops/norm.zig:79-96; tolerances are the
# reference tests' own, 2e-6 absolute)
# ---------------------------------------------------------------------------------

ACT_IN = np.array([-3, -1, -0.5, 0, 0.5, 1, 2, 3, 0.100000001, -2.20000005], np.float32)
SILU_OUT = np.array([-0.142277613, -0.268941432, -0.188770339, 0, 0.311229676, 0.731058598, 1.76159406,
                     2.85772252, 0.0524979196, -0.21945107], np.float32)
SIGMOID_OUT = np.array([0.0474258736, 0.268941432, 0.377540678, 0.5, 0.622459352, 0.731058598, 0.880797029,
                        0.952574134, 0.524979174, 0.0997504815], np.float32)


def test_silu_and_sigmoid_match_reference_fixtures():
    ones = np.ones_like(ACT_IN)
    assert np.allclose(oracle.silu_mul(ACT_IN, ones), SILU_OUT, rtol=0, atol=2e-6)
    assert np.allclose(oracle.sigmoid_mul(ones, ACT_IN), SIGMOID_OUT, rtol=0, atol=2e-6)
    # the "fused gates" cases: silu(1)*2, silu(-0.5)*3; 2*sigmoid(0)... as 1.0, 2*sigmoid(1)
    got = oracle.silu_mul(np.array([1, -0.5], np.float32), np.array([2, 3], np.float32))
    assert np.allclose(got, [0.731058598 * 2.0, -0.188770339 * 3.0], rtol=0, atol=1e-6)
    got = oracle.sigmoid_mul(np.array([2, 2], np.float32), np.array([0, 1], np.float32))
    assert np.allclose(got, [1.0, 2.0 * 0.731058598], rtol=0, atol=1e-6)


def test_rms_mod_matches_reference_rmsnorm_fixture():
    x = np.array([0.5, -1.5, 2, 0.25, 3, 0, -0.125, 1], np.float32).reshape(2, 4)
    weight = (1.0 + np.array([0.100000001, -0.200000003, 0, 0.5], np.float32)).astype(np.float32)
    zero = np.zeros(4, np.float32)
    want = np.array([0.429394752, -0.936861217, 1.56143546, 0.292769134, 2.08547044, 0, -0.0789950937,
                     0.947941124], np.float32).reshape(2, 4)
    assert np.allclose(oracle.rms_mod(x, weight, zero, 1e-5), want, rtol=0, atol=2e-6)
    want6 = np.array([0.429395914, -0.93686384, 1.56143963, 0.292769939, 2.08547425, 0, -0.0789952353,
                      0.947942853], np.float32).reshape(2, 4)
    assert np.allclose(oracle.rms_mod(x, weight, zero, 1e-6), want6, rtol=0, atol=2e-6)
    # odd dim, eps 0 (norm.zig:98-107), then modulation on top: (1 + scale) * normed + shift
    x5 = np.array([[1, 2, 3, 4, 5], [-1, -2, -3, -4, -5]], np.float32)
    rms = np.sqrt(np.float32(11.0))
    got = oracle.rms_mod(x5, np.ones(5, np.float32), zero[:1].repeat(5), 0.0)
    assert abs(got[0, 0] - 1.0 / rms) < 1e-6 and abs(got[1, 4] + 5.0 / rms) < 1e-6
    scale, shift = np.float32(0.25), np.float32(-0.5)
    got = oracle.rms_mod(x5, np.full(5, 1 + scale, np.float32), np.full(5, shift, np.float32), 0.0)
    assert np.allclose(got, (1 + scale) * (x5 / rms) + shift, rtol=0, atol=2e-6)


def test_gated_add():
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    d = np.ones((2, 3), np.float32) * 2
    g = np.array([0.5, -1, 0], np.float32)
    assert np.array_equal(oracle.gated_add(x, d, g), x + g * d)


# ---------------------------------------------------------------------------------
# k-quant decoders pinned to the reference's golden super-blocks
# (src/core/quants_fixtures.zig, checked bit for bit as src/core/quants.zig:104-140 does)
# ---------------------------------------------------------------------------------

@pytest.mark.parametrize("fmt", ["q4_k", "q5_k", "q6_k"])
def test_kquant_dequant_matches_reference_golden_block(fmt):
    import json
    import os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "kquant_blocks.json")))[fmt]
    block = np.array(g["block_bytes"], np.uint8)
    want = np.array(g["expected_f32_bits"], np.uint32)
    assert block.size == oracle.gguf_row_bytes(fmt, 256)
    got = oracle.gguf_dequant_row(fmt, block, 256)
    assert np.array_equal(got.view(np.uint32), want)


def test_q4_0_and_generic_gemv_truth():
    rng = np.random.default_rng(5)
    # q4_0: d = 0.5, nibbles 0..15 -> (n - 8) * d, low nibbles first
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blk[2:18] = np.arange(16, dtype=np.uint8) | ((15 - np.arange(16, dtype=np.uint8)) << 4)
    got = oracle.gguf_dequant_row("q4_0", blk, 32)
    assert np.array_equal(got[:16], (np.arange(16) - 8) * 0.5) and np.array_equal(got[16:], (7 - np.arange(16)) * 0.5)
    # the generic GEMV truth agrees with the Q8_0-specific one
    g = synth.q8_0_gemv(m=2, n=8, k=512, seed=9)
    a = oracle.gguf_gemv_q8("q8_0", g["w"], 8, 512, g["x"])
    b = oracle.q8_0_gemv_f64(g["w"], 8, 512, oracle_q8_1_dequant(g["x"]))
    assert np.allclose(a, b, rtol=1e-6, atol=1e-6)


def oracle_q8_1_dequant(x):
    d, qs = oracle.q8_1_quantize(x.reshape(-1))
    return (np.repeat(d, 32) * qs.astype(np.float32)).reshape(x.shape)


def test_iq4_nl_dequant_matches_reference_known_answers():
    """src/core/quants.zig:133-151: d = 2.0, qs[0] = 0x21, the rest 0."""
    kv = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(2.0).tobytes(), np.uint8)
    blk[2] = 0x21
    out = oracle.gguf_dequant_row("iq4_nl", blk, 32)
    assert out[0] == 2.0 * kv[1] and out[16] == 2.0 * kv[2]
    assert np.all(out[1:16] == 2.0 * kv[0]) and np.all(out[17:32] == 2.0 * kv[0])


# ---------------------------------------------------------------------------------
# Attention pieces pinned to the reference's torch-generated fixtures
# (src/ops/attention.zig:291-313 at 3e-6, src/ops/rope.zig:353-366 at 2e-6)
# ---------------------------------------------------------------------------------

def test_attention_matches_reference_sdpa_fixture():
    q = np.array([-1.12583983, -1.1523602, -0.250578582, -0.433878809, 0.166455343, 0.87438184, -0.143473849,
                  -0.111609332, 0.848710358, 0.692009151, -0.31601277, -2.11521935, 0.931826591, 1.25900924, 2.00498056,
                  0.0537369028, 0.468096405, -0.157712445, 1.44366014, 0.266049415, 0.618056655, -0.412802219,
                  -0.841064811, -2.31604195], np.float32)
    k = np.array([0.370393544, 1.45650256, 0.939809918, 0.774848819, 0.191869423, 1.26379478, -1.29043508, -0.791102707,
                  -0.0208794735, -0.718480051, 0.518636763, -1.31252193], np.float32)
    v = np.array([0.191995069, 0.542771339, -2.21877933, 0.258984536, -1.02970219, -0.50075841, 0.273367733,
                  -0.918099999, -0.0404210873, 0.288116813, -0.00753730815, -0.914495468], np.float32)
    want = np.array([-0.233936831, 0.140385717, -0.156303599, -0.80384618, -0.3932935, 0.0334626585, -0.734680712,
                     -0.463540882, -0.583657682, -0.13896063, -0.0424246602, -0.813088059, 0.0828519836, 0.443475634,
                     -1.80830443, 0.0511539057, 0.00270056119, 0.361810803, -1.23623109, -0.249404013, -0.469629675,
                     -0.0521637946, 0.05305776, -0.882563472], np.float32)
    got = oracle.attention(q, k, v, heads=2, kv_heads=1, hd=4)
    assert np.allclose(got.reshape(-1), want, rtol=0, atol=3e-6)


def test_flux_rope_matches_reference_fixture():
    q_in = np.array([-1, -0.899999976, -0.800000012, -0.699999988, -0.600000024, -0.5, -0.399999976, -0.300000012,
                     -0.199999988, -0.100000024, 0, 0.100000024, 0.200000048, 0.299999952, 0.399999976, 0.5, 0.600000024,
                     0.700000048, 0.799999952, 0.899999976, 1, 1.0999999, 1.20000005, 1.29999995], np.float32)
    q_out = np.array([-1, -0.899999976, -0.800000012, -0.699999988, -0.600000024, -0.5, -0.399999976, -0.300000012,
                      -0.0239133313, -0.222324416, -0.0176892225, 0.0984230489, 0.190414816, 0.306173474, 0.397181958,
                      0.502241433, -0.00754925609, 0.921923578, -0.596392035, 1.04609585, 0.734088182, 1.29271591,
                      1.14791059, 1.34621739], np.float32)
    cos, sin = oracle.flux_freqs(np.array([0, 1, 7], np.float32), [8], 1000.0)
    got = oracle.rope_interleaved(q_in, cos, sin, heads=1, hd=8)
    assert np.allclose(got, q_out, rtol=0, atol=2e-6)
    # position zero is the identity (rope.zig:391-398); qk-norm with unit weight has unit RMS
    assert np.array_equal(got[:8], q_in[:8])
    x = np.random.default_rng(0).standard_normal((5, 16)).astype(np.float32)
    n = oracle.qk_norm(x, np.ones(16, np.float32), 0.0)
    assert np.allclose(np.sqrt((n.astype(np.float64) ** 2).mean(axis=1)), 1.0, atol=1e-6)
