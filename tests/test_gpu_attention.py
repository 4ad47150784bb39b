"""Attention of the DiT block (qk-norm + RoPE + softmax attention) through the C ABI against
the CPU oracle (pinned to the reference's torch fixtures in tests/test_oracle.py).

Tolerances.  The prepare pass rounds to bf16: each value within one bf16 ulp (2^-8 relative)
of the oracle's f32 value.  The attention kernel multiplies bf16 operands with f32
accumulation and rounds the probabilities to bf16 for the second product; it is compared with
the oracle run on the SAME bf16-rounded q, k, v: 1e-2 absolute + 2e-2 relative (outputs are
averages of v, |v| ~ 1).  The reference's own gate for its tensor-core attention against the
f32 one is of that order (f16 operands)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
HD = 128


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).float().numpy()


def make(seq, heads, kv_heads, seed):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((seq, heads * HD)).astype(np.float32)
    k = rng.standard_normal((seq, kv_heads * HD)).astype(np.float32)
    v = rng.standard_normal((seq, kv_heads * HD)).astype(np.float32)
    qn = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    kn = (1.0 + 0.1 * rng.standard_normal(HD)).astype(np.float32)
    pos = np.stack([np.zeros(seq), np.arange(seq) // 8, np.arange(seq) % 8], axis=1).astype(np.float32)
    cos, sin = oracle.flux_freqs(pos, [32, 48, 48], 10000.0)      # Krea 2's axes (src/ops/rope.zig:26-28)
    return q, k, v, qn, kn, cos, sin


def prepared_reference(q, k, v, qn, kn, cos, sin, heads, kv_heads):
    seq = q.shape[0]
    qr = oracle.rope_interleaved(oracle.qk_norm(q.reshape(seq * heads, HD), qn, 1e-5).reshape(seq, -1), cos, sin, heads, HD)
    kr = oracle.rope_interleaved(oracle.qk_norm(k.reshape(seq * kv_heads, HD), kn, 1e-5).reshape(seq, -1), cos, sin, kv_heads, HD)
    return qr, kr


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seq,heads,kv_heads", [(128, 2, 2), (300, 4, 2), (77, 2, 1)])
def test_prepare_matches_oracle(be, dtype, seq, heads, kv_heads):
    q, k, v, qn, kn, cos, sin = make(seq, heads, kv_heads, seq)
    if dtype == torch.bfloat16:
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    qr, kr = prepared_reference(q, k, v, qn, kn, cos, sin, heads, kv_heads)
    dev = lambda a: torch.from_numpy(a).cuda().to(dtype)
    be.attention(dev(q), dev(k), dev(v), torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda(),
                 torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), heads, kv_heads)
    be.status_poll()
    qb = be._attn_qb.float().cpu().numpy()                        # [heads][seq][hd]
    kb = be._attn_kb.float().cpu().numpy()
    want_q = qr.reshape(seq, heads, HD).transpose(1, 0, 2)
    want_k = kr.reshape(seq, kv_heads, HD).transpose(1, 0, 2)
    assert np.all(np.abs(qb - want_q) <= 2.0 ** -8 * np.abs(want_q) + 1e-6)
    assert np.all(np.abs(kb - want_k) <= 2.0 ** -8 * np.abs(want_k) + 1e-6)
    seq_pad = (seq + 7) // 8 * 8
    vt = be._attn_vt.float().cpu().numpy().reshape(kv_heads, HD, seq_pad)
    want_v = bf16_round(v).reshape(seq, kv_heads, HD).transpose(1, 2, 0)
    assert np.array_equal(vt[:, :, :seq], want_v) and np.all(vt[:, :, seq:] == 0)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("seq,heads,kv_heads", [(128, 1, 1), (256, 2, 1), (384, 4, 2), (300, 2, 2), (77, 2, 1), (1000, 3, 3)])
def test_attention_matches_oracle(be, out_dtype, seq, heads, kv_heads):
    q, k, v, qn, kn, cos, sin = make(seq, heads, kv_heads, 100 + seq)
    cu = lambda a: torch.from_numpy(a).cuda()
    out = be.attention(cu(q), cu(k), cu(v), cu(qn), cu(kn), cu(cos), cu(sin), heads, kv_heads, out_dtype=out_dtype)
    be.status_poll()
    # the oracle on exactly what the kernel multiplies: the bf16 q', k' and v
    qb = be._attn_qb.float().cpu().numpy().transpose(1, 0, 2).reshape(seq, heads * HD)
    kb = be._attn_kb.float().cpu().numpy().transpose(1, 0, 2).reshape(seq, kv_heads * HD)
    want = oracle.attention(qb, kb, bf16_round(v), heads, kv_heads, HD)
    got = out.float().cpu().numpy()
    err = np.abs(got - want)
    assert np.all(err <= 1e-2 + 2e-2 * np.abs(want)), f"max err {err.max():.4f}"
    # and end to end against the f32 definition (looser: bf16 operands)
    qr, kr = prepared_reference(q, k, v, qn, kn, cos, sin, heads, kv_heads)
    truth = oracle.attention(qr, kr, v, heads, kv_heads, HD)
    rel = np.linalg.norm(got - truth) / np.linalg.norm(truth)
    assert rel < 2e-2, rel


def test_attention_dit_size_sampled(be):
    """seq 4608, 24 heads x 128 (the DiT step's shape): 48 sampled query rows against the oracle."""
    seq, heads, kv_heads = 4608, 24, 24
    q, k, v, qn, kn, cos, sin = make(seq, heads, kv_heads, 7)
    cu = lambda a: torch.from_numpy(a).cuda()
    out = be.attention(cu(q), cu(k), cu(v), cu(qn), cu(kn), cu(cos), cu(sin), heads, kv_heads)
    be.status_poll()
    rows = np.sort(np.random.default_rng(3).choice(seq, 48, replace=False))
    qb = be._attn_qb.float().cpu().numpy().transpose(1, 0, 2).reshape(seq, heads * HD)
    kb = be._attn_kb.float().cpu().numpy().transpose(1, 0, 2).reshape(seq, kv_heads * HD)
    want = oracle.attention(qb[rows], kb, bf16_round(v), heads, kv_heads, HD)
    got = out.float().cpu().numpy()[rows]
    err = np.abs(got - want)
    assert np.all(err <= 1e-2 + 2e-2 * np.abs(want)), f"max err {err.max():.4f}"


def test_attention_rejects_bad_arguments(be):
    from tensorpencil_b200 import _lib
    t = torch.zeros(1 << 16, dtype=torch.bfloat16, device="cuda")
    f = be.lib.tpb_attention
    assert f(be.h, None, t.data_ptr(), _lib.TPB_BF16, t.data_ptr(), t.data_ptr(), t.data_ptr(), 128, 128, 2, 2, 64, 0.1) == _lib.TPB_ERR_INVALID_ARG
    assert f(be.h, None, t.data_ptr(), _lib.TPB_BF16, t.data_ptr(), t.data_ptr(), t.data_ptr(), 128, 128, 3, 2, 128, 0.1) == _lib.TPB_ERR_INVALID_ARG
    assert f(be.h, None, t.data_ptr(), _lib.TPB_S32, t.data_ptr(), t.data_ptr(), t.data_ptr(), 128, 128, 2, 2, 128, 0.1) == _lib.TPB_ERR_INVALID_ARG
    # heads * seq beyond the 32-bit row coordinates of the tensor maps
    assert f(be.h, None, t.data_ptr(), _lib.TPB_BF16, t.data_ptr(), t.data_ptr(), t.data_ptr(), (1 << 24) - 1, 128, 256, 256, 128, 0.1) == _lib.TPB_ERR_INVALID_ARG
