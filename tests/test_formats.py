"""On-disk formats (safetensors ConvRot weights, GGUF) and the budgeted weight cache.
CPU tests of the parsing and policy; one GPU test that loads files and runs them."""
import json
import struct

import numpy as np
import pytest

from oracle import oracle
from tensorpencil_b200 import formats, synth
from tensorpencil_b200.formats import FormatError


def _convrot_file(tmp_path, dtype_tag_i4="U8"):
    c8 = synth.convrot_weights(64, 512, 8, seed=1)
    c4 = synth.convrot_weights(48, 256, 4, seed=2)
    p = str(tmp_path / "ckpt.safetensors")
    packed = c4["w_packed"] if dtype_tag_i4 == "U8" else c4["w_packed"].view(np.int8)
    formats.write_safetensors(p, {
        "model.blocks.0.attn.wq.weight": ("I8", c8["w_i8"]),
        "model.blocks.0.attn.wq.weight_scale": ("F32", c8["w_scale"]),
        "model.blocks.0.mlp.up.weight": (dtype_tag_i4, packed),
        "model.blocks.0.mlp.up.weight_scale": ("BF16", (c4["w_scale"].view(np.uint32) >> 16).astype(np.uint16)),
        "model.norm": ("F32", np.ones(4, np.float32)),
    }, metadata={"format": "pt"})
    return p, c8, c4


@pytest.mark.parametrize("i4_tag", ["U8", "I8"])
def test_safetensors_convrot_weights(tmp_path, i4_tag):
    p, c8, c4 = _convrot_file(tmp_path, i4_tag)
    st = formats.SafeTensors(p)
    assert st.metadata == {"format": "pt"} and st.get("nope") is None
    w8 = formats.load_convrot_weight(st, "blocks.0.attn.wq.weight", 64, 512, prefix="model.")
    assert w8.bits == 8 and np.array_equal(w8.w, c8["w_i8"]) and np.array_equal(w8.row_scale, c8["w_scale"])
    # int4: U8 (the reference's converter) or I8 at half the columns (ComfyUI's): same bytes, same decode
    w4 = formats.load_convrot_weight(st, "blocks.0.mlp.up.weight", 48, 256, prefix="model.")
    assert w4.bits == 4 and np.array_equal(w4.w, c4["w_packed"])
    bf = (c4["w_scale"].view(np.uint32) >> 16 << 16).view(np.float32)
    assert np.array_equal(w4.row_scale, bf)
    assert np.array_equal(oracle.unpack_i4(w4.w.reshape(-1)).reshape(48, 256), c4["w_i8"])
    # errors carry the reference's names
    for args, err in ((("blocks.0.attn.wq.weight", 64, 256), "ShapeMismatch"),      # an int8 weight is never "halved"
                      (("blocks.9.attn.wq.weight", 64, 512), "MissingTensor"),
                      (("norm", 1, 4), "UnsupportedCheckpoint")):
        with pytest.raises(FormatError) as e:
            formats.load_convrot_weight(st, args[0], args[1], args[2], prefix="model.")
        assert e.value.name == err
    st.close()


def test_safetensors_int8_at_half_width_is_read_as_int4(tmp_path):
    """The disambiguation rule itself (src/models/dit.zig:698-708): I8 [rows][cols/2] is int4."""
    p = str(tmp_path / "a.safetensors")
    raw = np.arange(32 * 128, dtype=np.uint8).reshape(32, 128).view(np.int8)
    formats.write_safetensors(p, {"w": ("I8", raw), "w_scale": ("F32", np.ones(32, np.float32))})
    st = formats.SafeTensors(p)
    assert formats.load_convrot_weight(st, "w", 32, 256).bits == 4      # asked for 256 columns: packed
    with pytest.raises(FormatError) as e:
        formats.load_convrot_weight(st, "w", 32, 128)                    # 128 is not a multiple of the rotation group
    assert e.value.name == "ShapeMismatch"
    st.close()


def test_safetensors_rejects_bad_headers(tmp_path):
    def write(header: dict, payload=b"\0" * 16):
        p = str(tmp_path / "bad.safetensors")
        hj = json.dumps(header).encode()
        open(p, "wb").write(struct.pack("<Q", len(hj)) + hj + payload)
        return p

    for header, err in (({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, "InvalidOffsets"),
                        ({"t": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, "InvalidShape"),
                        ({"t": {"dtype": "F32", "shape": [8], "data_offsets": [0, 32]}}, "InvalidOffsets"),
                        ({"t": {"dtype": "Q9", "shape": [2], "data_offsets": [0, 8]}}, "UnsupportedDType")):
        with pytest.raises(FormatError) as e:
            formats.SafeTensors(write(header))
        assert e.value.name == err
    p = str(tmp_path / "short.safetensors")
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(FormatError) as e:
        formats.SafeTensors(p)
    assert e.value.name == "InvalidHeader"


def test_gguf_roundtrip_and_errors(tmp_path):
    k = 512
    tensors = {}
    for tag, fmt in (("Q4_K", "q4_k"), ("Q6_K", "q6_k"), ("Q8_0", "q8_0"), ("IQ4_NL", "iq4_nl")):
        tensors[f"blk.0.{fmt}.weight"] = (tag, (24, k), synth.gguf_weights(fmt, 24, k, seed=3))
    tensors["norm.weight"] = ("F32", (k,), np.linspace(0, 1, k, dtype=np.float32))
    p = str(tmp_path / "m.gguf")
    formats.write_gguf(p, tensors, metadata={"general.architecture": "qwen3", "qwen3.block_count": 1, "x.list": [1, 2, 3]},
                       alignment=64)
    g = formats.Gguf(p)
    assert g.version == 3 and g.alignment == 64
    assert g.metadata["general.architecture"] == "qwen3" and g.metadata["x.list"] == [1, 2, 3]
    for name, (tag, shape, raw) in tensors.items():
        v = g.get(name)
        assert v.dtype == tag and v.shape == shape          # dims come back in row-major order
        assert np.array_equal(v.data, np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    # a q4_k row decodes like the oracle's reading of the same bytes
    v = g.get("blk.0.q4_k.weight")
    row_bytes = oracle.gguf_row_bytes("q4_k", k)
    assert v.data.size == 24 * row_bytes
    assert np.array_equal(oracle.gguf_dequant_row("q4_k", v.data[:row_bytes], k),
                          oracle.gguf_dequant_row("q4_k", tensors["blk.0.q4_k.weight"][2][0], k))
    g.close()
    raw = bytearray(open(p, "rb").read())
    for patch, err in (((0, b"GGUX"), "InvalidMagic"), ((4, struct.pack("<I", 9)), "UnsupportedVersion")):
        b = bytearray(raw)
        b[patch[0]:patch[0] + len(patch[1])] = patch[1]
        q = str(tmp_path / "bad.gguf")
        open(q, "wb").write(b)
        with pytest.raises(FormatError) as e:
            formats.Gguf(q)
        assert e.value.name == err
    q = str(tmp_path / "trunc.gguf")
    open(q, "wb").write(raw[:60])
    with pytest.raises(FormatError) as e:
        formats.Gguf(q)
    assert e.value.name == "InvalidHeader"


def test_weight_cache_lru_and_pins():
    uploads = []
    cache = formats.WeightCache(lambda a: uploads.append(a.nbytes) or ("dev", a.nbytes), budget=1000)
    a, b, c, d = (np.zeros(n, np.uint8) for n in (400, 400, 300, 900))
    assert cache.get(a) == ("dev", 400) and cache.get(b) and cache.bytes == 800
    cache.get(a)                                   # a is now the most recent
    cache.get(c)                                   # needs 300: evicts b (least recent), keeps a
    assert cache.bytes == 700 and cache.evictions == 1 and cache.hits == 1 and cache.misses == 3
    cache.get(b)                                   # evicts a now
    assert cache.misses == 4 and cache.bytes == 700 and uploads == [400, 400, 300, 400]
    cache.get(c, pin=True)
    with pytest.raises(MemoryError):               # 900 + pinned 300 > 1000
        cache.get(d)
    cache.unpin(c)
    cache.get(d)                                   # everything else goes
    assert cache.bytes == 900
    with pytest.raises(MemoryError):
        cache.get(np.zeros(2000, np.uint8))


@pytest.mark.gpu
def test_files_to_gpu_results(tmp_path):
    """A ConvRot safetensors linear and GGUF GEMV weights, from file to device results."""
    torch = pytest.importorskip("torch")
    from tensorpencil_b200.backend import Backend
    be = Backend(0)
    try:
        p, c8, c4 = _convrot_file(tmp_path)
        st = formats.SafeTensors(p)
        cache = formats.WeightCache(be.cachedWeight, budget=1 << 20)
        for name, rows, cols, c in (("blocks.0.attn.wq.weight", 64, 512, c8), ("blocks.0.mlp.up.weight", 48, 256, c4)):
            w = formats.load_convrot_weight(st, name, rows, cols, prefix="model.")
            x = synth.activations(33, cols, seed=5)
            y = be.convrot_linear(torch.from_numpy(x).cuda(), cache.get(np.ascontiguousarray(w.w)),
                                  cache.get(w.row_scale), rows, w.bits)
            q, s, acc, sim = oracle.convrot_linear_sim(x, c["w_i8"], c["w_scale"] if w.bits == 8 else w.row_scale, w.bits)
            err = np.abs(y.cpu().numpy() - sim)
            assert (err <= 1e-4 + 1e-3 * np.abs(sim)).all()
        k = 512
        gp = str(tmp_path / "m.gguf")
        ws = {fmt: synth.gguf_weights(fmt, 24, k, seed=3) for fmt in ("q4_k", "q6_k", "q8_0")}
        formats.write_gguf(gp, {f"w.{fmt}": (fmt.upper(), (24, k), w) for fmt, w in ws.items()})
        g = formats.Gguf(gp)
        x = (np.random.default_rng(1).random((3, k), dtype=np.float32) * 2 - 1).astype(np.float32)
        be.opGemvQuantizeX(torch.from_numpy(x).cuda(), 3 * k)
        for fmt in ws:
            v = g.get(f"w.{fmt}")
            wd = torch.from_numpy(np.ascontiguousarray(v.data)).cuda()
            y = torch.empty((3, 24), dtype=torch.float32, device="cuda")
            be.opGemvQuantQ8N(formats.GGUF_GEMV_FORMAT[v.dtype], y, wd, 1.0, 24, k, 3, 0, 3)
            want = oracle.gguf_gemv_q8(fmt, ws[fmt], 24, k, x)
            assert np.abs(y.cpu().numpy() - want).max() <= 2e-2
        be.status_poll()
        g.close()
        st.close()
    finally:
        be.close()


def _fnv1a(b: bytes) -> int:
    h = 1469598103934665603
    for x in b:
        h = ((h ^ x) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def test_cpp_readers_agree_with_python(tmp_path):
    """include/tpb200_formats.hpp reads the same files the same way (tests/cpp/test_formats.cpp)."""
    import os
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "test_formats")
    r = subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(root, "include"),
                        os.path.join(root, "tests", "cpp", "test_formats.cpp"), "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    sp, c8, c4 = _convrot_file(tmp_path)
    k = 512
    tensors = {f"blk.0.{fmt}.weight": (fmt.upper(), (24, k), synth.gguf_weights(fmt, 24, k, seed=3))
               for fmt in ("q4_k", "q6_k", "q8_0", "iq4_nl")}
    tensors["norm.weight"] = ("F32", (k,), np.linspace(0, 1, k, dtype=np.float32))
    gp = str(tmp_path / "m.gguf")
    formats.write_gguf(gp, tensors, metadata={"general.architecture": "qwen3", "qwen3.block_count": 7}, alignment=64)
    bad_st = str(tmp_path / "bad.safetensors")
    hj = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode()
    open(bad_st, "wb").write(struct.pack("<Q", len(hj)) + hj + b"\0" * 16)
    bad_gg = str(tmp_path / "bad.gguf")
    raw = bytearray(open(gp, "rb").read())
    raw[0:4] = b"GGUX"
    open(bad_gg, "wb").write(raw)
    out = subprocess.run([exe, sp, gp, bad_st, bad_gg], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = out.stdout.strip().splitlines()
    got = {ln.split()[1]: ln.split()[2:] for ln in lines if ln.startswith("T ")}
    st, g = formats.SafeTensors(sp), formats.Gguf(gp)
    for src in (st, g):
        for name, v in src.tensors.items():
            dt, shape, nbytes, cs = got[name]
            assert dt == v.dtype and shape == "[" + ",".join(str(s) for s in v.shape) + "]"
            assert int(nbytes) == v.data.size and int(cs) == _fnv1a(v.data.tobytes())
    w8 = formats.load_convrot_weight(st, "model.blocks.0.attn.wq.weight", 64, 512)
    w4 = formats.load_convrot_weight(st, "model.blocks.0.mlp.up.weight", 48, 256)
    l8 = next(ln for ln in lines if ln.startswith("W8 ")).split()
    l4 = next(ln for ln in lines if ln.startswith("W4 ")).split()
    assert l8[1] == "8" and int(l8[3]) == _fnv1a(w8.w.tobytes()) and np.float32(float(l8[4])) == w8.row_scale[5]
    assert l4[1] == "4" and int(l4[3]) == _fnv1a(w4.w.tobytes()) and np.float32(float(l4[4])) == w4.row_scale[5]
    assert next(ln for ln in lines if ln.startswith("E ")).split()[1:] == ["ShapeMismatch", "MissingTensor", "UnsupportedCheckpoint"]
    assert next(ln for ln in lines if ln.startswith("G ")).split()[1:] == ["3", "64", "qwen3", "7"]
    assert [ln.split()[1] for ln in lines if ln.startswith("B ")] == ["InvalidOffsets", "InvalidMagic"]
    named = [ln.split()[1:] for ln in lines if ln.startswith("N ")]
    assert len(named) >= 15
    for raw, arch, canon in named:
        assert canon == formats.canonical_name(raw, arch), (raw, arch)
    assert next(ln for ln in lines if ln.startswith("H ")).split()[1] == "1"
    assert next(ln for ln in lines if ln.startswith("C ")).split()[1] == "1"      # include/tpb200_cache.hpp
    st.close()
    g.close()


# the reference's cases (src/core/gguf.zig:679-727)
CANONICAL_CASES = [
    ("token_embd.weight", "qwen3", "embed_tokens.weight"),
    ("output.weight", "qwen3", "lm_head.weight"),
    ("output_norm.weight", "qwen3", "norm.weight"),
    ("blk.17.ffn_down.weight", "qwen3", "layers.17.mlp.down_proj.weight"),
    ("blk.0.attn_k_norm.weight", "qwen3", "layers.0.self_attn.k_norm.weight"),
    ("blk.0.ssm_conv1d.weight", "qwen35", "layers.0.ssm_conv1d.weight"),
    ("blk.5.ssm_dt.bias", "qwen35", "layers.5.ssm_dt.bias"),
    ("blk.2.post_attention_norm.weight", "qwen3", "layers.2.post_attention_layernorm.weight"),
    ("layers.3.self_attn.q_proj.weight", "qwen3", "layers.3.self_attn.q_proj.weight"),
    ("blk.0.ffn_norm.weight", "gemma3", "layers.0.pre_feedforward_layernorm.weight"),
    ("blk.0.post_attention_norm.weight", "gemma3", "layers.0.post_attention_layernorm.weight"),
    ("blk.0.post_ffw_norm.weight", "gemma3", "layers.0.post_feedforward_layernorm.weight"),
    ("blk.7.attn_output.weight", "gemma3", "layers.7.self_attn.o_proj.weight"),
    # beyond the reference's list: the Qwen reading of ffn_norm, Gemma 4's extra entry, malformed layer ids
    ("blk.3.ffn_norm.weight", "qwen3", "layers.3.post_attention_layernorm.weight"),
    ("blk.1.layer_output_scale.weight", "gemma4", "layers.1.out_scale.weight"),
    ("blk.1.layer_output_scale.weight", "gemma3", "layers.1.layer_output_scale.weight"),
    ("blk.x.attn_q.weight", "qwen3", "blk.x.attn_q.weight"),
    ("blk.4", "qwen3", "blk.4"),
]


def test_canonical_tensor_names(tmp_path):
    for raw, arch, want in CANONICAL_CASES:
        assert formats.canonical_name(raw, arch) == want, (raw, arch)
    # a reader answers to both spellings
    k = 256
    w = synth.gguf_weights("q8_0", 8, k, seed=5)
    p = str(tmp_path / "names.gguf")
    formats.write_gguf(p, {"blk.2.ffn_up.weight": ("Q8_0", (8, k), w), "token_embd.weight": ("Q8_0", (8, k), w)},
                       metadata={"general.architecture": "gemma3"})
    g = formats.Gguf(p)
    assert g.get("layers.2.mlp.up_proj.weight") is g.get("blk.2.ffn_up.weight") is not None
    assert g.get("embed_tokens.weight") is not None and g.get("layers.2.mlp.down_proj.weight") is None
    g.close()
