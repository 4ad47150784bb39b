"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations.

The reference measures on real Krea 2 / GGUF checkpoints; these tensors stand
in for them.  Everything is generated on the host with ``numpy`` from a seed so
the CPU checker and the device path see identical bytes.

* ConvRot linear: activations ~N(0,1) with 1 % of the K channels scaled x20
  (outlier channels), weights uniform over the signed range of the width,
  per-output-channel scales ~U(1e-3, 1e-2).
* Q8_0 GEMV: 34-byte blocks (f16 ``d`` then 32 int8), quants uniform in
  [-127,127], ``d`` ~U(1e-3,1e-2) rounded to f16, activations ~N(0,1).
"""
from __future__ import annotations

import numpy as np

Q8_0_BLOCK_BYTES = 34  # f16 d + 32 x i8 (src/core/dtype.zig:93)


def pack_i4(vals: np.ndarray) -> np.ndarray:
    """int8 values in [-8,7] -> two per byte, element 2j in the low nibble
    (src/core/dtype.zig:19-24)."""
    v = np.ascontiguousarray(vals, np.int8).view(np.uint8)
    return ((v[..., 0::2] & 0xF) | ((v[..., 1::2] & 0xF) << 4)).astype(np.uint8)


def unpack_i4(packed: np.ndarray) -> np.ndarray:
    p = np.ascontiguousarray(packed, np.uint8)
    lo = (p & 0xF).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo).astype(np.int8)
    hi = np.where(hi >= 8, hi - 16, hi).astype(np.int8)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def activations(m: int, k: int, seed: int, outlier_frac: float = 0.01,
                outlier_gain: float = 20.0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    n_out = int(np.floor(outlier_frac * k))
    if n_out:
        ch = rng.choice(k, size=n_out, replace=False)
        x[:, ch] *= np.float32(outlier_gain)
    return x


def convrot_weights(n: int, k: int, bits: int, seed: int) -> dict:
    rng = np.random.default_rng(seed + 7919)
    if bits == 8:
        w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        packed = None
    else:
        w = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
        packed = pack_i4(w)
    ws = rng.uniform(1e-3, 1e-2, size=n).astype(np.float32)
    return {"w_i8": w, "w_packed": packed, "w_scale": ws}


def convrot_linear(m: int, n: int, k: int, bits: int, seed: int) -> dict:
    """One ConvRot linear: x f32 [m][k], W int [n][k] (+ packed form for int4),
    w_scale f32 [n]."""
    out = {"x": activations(m, k, seed), "m": m, "n": n, "k": k, "bits": bits}
    out.update(convrot_weights(n, k, bits, seed))
    return out


def config0(seed: int = 1000) -> dict:
    """Single INT8 ConvRot linear, M=256, K=N=3072."""
    return convrot_linear(256, 3072, 3072, 8, seed)


def config1(seed: int = 1001, m: int = 4608) -> dict:
    """Single INT4 ConvRot linear at the DiT MLP shape, M=4608, K=3072, N=12288."""
    return convrot_linear(m, 12288, 3072, 4, seed)


def q8_0_weights(n: int, k: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed + 104729)
    nblk = k // 32
    out = np.empty((n, nblk, Q8_0_BLOCK_BYTES), np.uint8)
    d = rng.uniform(1e-3, 1e-2, size=(n, nblk)).astype(np.float16)
    out[:, :, 0:2] = d.view(np.uint8).reshape(n, nblk, 2)
    out[:, :, 2:] = rng.integers(-127, 128, size=(n, nblk, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(n, nblk * Q8_0_BLOCK_BYTES)


def q8_0_gemv(m: int, n: int, k: int, seed: int) -> dict:
    rng = np.random.default_rng(seed)
    return {"x": rng.standard_normal((m, k), dtype=np.float32),
            "w": q8_0_weights(n, k, seed), "m": m, "n": n, "k": k}


def config2(m: int = 1, down: bool = False, seed: int = 1002) -> dict:
    """LLM decode GEMV at Qwen-27B-like dims: K=5120 -> N=17408, or the
    down-projection K=17408 -> N=5120."""
    n, k = (5120, 17408) if down else (17408, 5120)
    return q8_0_gemv(m, n, k, seed + (1 if down else 0))


# DiT block of the synthetic model (configs 3 and 4): name, N, K.
DIT_HIDDEN = 3072
DIT_MLP = 12288
DIT_BLOCKS = 28
DIT_TOKENS = 4608
DIT_LINEARS = (
    ("wq", DIT_HIDDEN, DIT_HIDDEN),
    ("wk", DIT_HIDDEN, DIT_HIDDEN),
    ("wv", DIT_HIDDEN, DIT_HIDDEN),
    ("gate", DIT_HIDDEN, DIT_HIDDEN),
    ("wo", DIT_HIDDEN, DIT_HIDDEN),
    ("mlp_gate", DIT_MLP, DIT_HIDDEN),
    ("mlp_up", DIT_MLP, DIT_HIDDEN),
    ("mlp_down", DIT_HIDDEN, DIT_MLP),
)


def dit_block_weights(block: int, bits: int, seed: int = 1003, hidden: int = DIT_HIDDEN,
                      mlp: int = DIT_MLP) -> dict:
    """Random-init quantised weights of one transformer block (the eight
    quantised linears of src/models/dit.zig:594-664 at the synthetic dims)."""
    out = {}
    for i, (name, n, k) in enumerate(DIT_LINEARS):
        n = mlp if n == DIT_MLP else hidden
        k = mlp if k == DIT_MLP else hidden
        w = convrot_weights(n, k, bits, seed + 1000 * block + i)
        out[name] = {"w": w["w_packed"] if bits == 4 else w["w_i8"], "w_scale": w["w_scale"],
                     "n": n, "k": k, "bits": bits}
    return out


GGUF_BLOCK = {"q8_0": (32, 34), "q4_0": (32, 18), "q4_k": (256, 144), "q5_k": (256, 176), "q6_k": (256, 210),
              "iq4_nl": (32, 18)}


def gguf_weights(fmt: str, n: int, k: int, seed: int) -> np.ndarray:
    """Random block-quantised weight rows [n][row_bytes] with every block's f16 scale
    fields pinned to small finite values (random bit patterns include NaN/inf), the way the
    reference's device tests build theirs (src/gpu/cuda/backend.zig:3356-3377): d = 0.05,
    dmin = 0.02."""
    elems, nbytes = GGUF_BLOCK[fmt]
    rng = np.random.default_rng(seed + 7919)
    w = rng.integers(0, 256, size=(n, k // elems, nbytes), dtype=np.uint8)
    d16 = np.frombuffer(np.uint16(0x2A66).tobytes(), np.uint8)
    m16 = np.frombuffer(np.uint16(0x251F).tobytes(), np.uint8)
    if fmt in ("q8_0", "q4_0", "iq4_nl"):
        w[:, :, 0:2] = d16
    elif fmt in ("q4_k", "q5_k"):
        w[:, :, 0:2] = d16
        w[:, :, 2:4] = m16
    elif fmt == "q6_k":
        w[:, :, 208:210] = d16
    return w.reshape(n, -1)
