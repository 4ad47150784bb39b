"""The DiT block stack (src/models/dit_cuda.zig:466-520) through the library against the same
sequence composed from the CPU oracle's pieces, on a small synthetic model (2 blocks, hidden 512 =
4 heads x 128, MLP 1024, 300 tokens), with and without attention between the projections.

Tolerances (relative Frobenius error of the latents after the stack): the reference's op sequence
in f32 against the oracle 2e-3 (every op agrees to ~1e-6, but a value that lands on a quantisation
boundary may round the other way and moves one int8 step); the fused f32 sequence against the
unfused one 1e-4 (same arithmetic, one FMA contraction in the gated residual); the bf16 chain 3e-2;
with attention (bf16 operands on the tensor cores) against the oracle's f32 attention 3e-2."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
HID, MLP, BLOCKS, TOKENS, HEADS = 512, 1024, 2, 300, 4


@pytest.fixture(scope="module")
def setup():
    from tensorpencil_b200 import harness
    from tensorpencil_b200.backend import Backend
    be = Backend(0)
    w = harness.DitWeights(be, 8, blocks=BLOCKS, hidden=HID, mlp=MLP, seed=77)
    mod = harness.dit_modulation(be, BLOCKS, HID, seed=5)
    rng = np.random.default_rng(3)
    x0 = rng.standard_normal((TOKENS, HID)).astype(np.float32)
    _, _, _, qn, kn, cos, sin = harness.attention_inputs(TOKENS, 1, 1, be.device)
    attn = {"q_norm": qn, "k_norm": kn, "cos": cos, "sin": sin, "heads": HEADS}
    yield be, harness, w, mod, x0, attn
    w.close()
    be.close()


def oracle_step(w, mod, x, attn=None, eps=1e-5):
    """The reference's sequence from the oracle's functions (f32 activations, exact int32 GEMM)."""
    mod = mod.cpu().numpy()
    x = x.copy()

    def lin(inp, wt):
        wq, ws = wt[0].cpu().numpy(), wt[1].cpu().numpy()
        return oracle.convrot_linear_sim(inp, wq, ws, 8)[3].astype(np.float32)

    for b in range(w.blocks):
        wb, mb = w.dev[b], b * 6 * HID
        row = lambda i: mod[mb + i * HID: mb + (i + 1) * HID]
        t = oracle.rms_mod(x, row(0), row(1), eps)
        q, k, v, g = (lin(t, wb[n]) for n in ("wq", "wk", "wv", "gate"))
        a = v
        if attn is not None:
            cos, sin = attn["cos"].cpu().numpy(), attn["sin"].cpu().numpy()
            qn, kn = attn["q_norm"].cpu().numpy(), attn["k_norm"].cpu().numpy()
            qr = oracle.rope_interleaved(oracle.qk_norm(q.reshape(-1, 128), qn, eps).reshape(TOKENS, -1), cos, sin, HEADS, 128)
            kr = oracle.rope_interleaved(oracle.qk_norm(k.reshape(-1, 128), kn, eps).reshape(TOKENS, -1), cos, sin, HEADS, 128)
            a = oracle.attention(qr, kr, v, HEADS, HEADS, 128).astype(np.float32)
        o = lin(oracle.sigmoid_mul(a, g), wb["wo"])
        x = oracle.gated_add(x, o, row(2))
        t = oracle.rms_mod(x, row(3), row(4), eps)
        act = oracle.silu_mul(lin(t, wb["mlp_gate"]), lin(t, wb["mlp_up"]))
        x = oracle.gated_add(x, lin(act, wb["mlp_down"]), row(5))
    return x


def rel(a, b):
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def run(setup, mode, dtype, attn, mlp_tile, mlp_pair=False, qkvg_group=False):
    be, harness, w, mod, x0, _ = setup
    x = torch.from_numpy(x0.copy()).cuda()
    out = harness.dit_step_linears(be, w, x, out_dtype=dtype, mode=mode, mod=mod, mlp_tile=mlp_tile, attn=attn,
                                   mlp_pair=mlp_pair, qkvg_group=qkvg_group)
    be.status_poll()
    return out.float().cpu().numpy()


def test_reference_sequence_matches_oracle(setup):
    want = oracle_step(setup[2], setup[3], setup[4])
    got = run(setup, "unfused", torch.float32, None, 128)       # three ragged MLP tiles: 128, 128, 44
    assert rel(got, want) < 2e-3
    assert np.abs(got - setup[4]).max() > 1e-3                   # the stack did change the latents


def test_fused_sequence_matches_reference_sequence(setup):
    ref = run(setup, "unfused", torch.float32, None, 128)
    assert rel(run(setup, "fused", torch.float32, None, 128), ref) < 1e-4
    assert rel(run(setup, "fused", torch.float32, None, TOKENS), ref) < 1e-4
    assert rel(run(setup, "fused", torch.bfloat16, None, TOKENS), ref) < 3e-2
    # the MLP's gate and up projections in one launch with the SiLU gate in its epilogue
    assert rel(run(setup, "fused", torch.float32, None, 128, mlp_pair=True), ref) < 1e-4
    assert rel(run(setup, "fused", torch.bfloat16, None, TOKENS, mlp_pair=True), ref) < 3e-2
    # q, k, v and gate in one launch: the same bits as four launches, so the whole step is identical
    for dt in (torch.float32, torch.bfloat16):
        assert np.array_equal(run(setup, "fused", dt, None, TOKENS, mlp_pair=True, qkvg_group=True),
                              run(setup, "fused", dt, None, TOKENS, mlp_pair=True))


def test_sequence_with_attention_matches_oracle(setup):
    attn = setup[5]
    want = oracle_step(setup[2], setup[3], setup[4], attn)
    assert rel(run(setup, "unfused", torch.float32, attn, 128), want) < 3e-2
    assert rel(run(setup, "fused", torch.float32, attn, TOKENS), want) < 3e-2
    assert rel(run(setup, "fused", torch.bfloat16, attn, TOKENS), want) < 3e-2
