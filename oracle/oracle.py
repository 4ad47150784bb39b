"""ctypes/numpy front end of the CPU oracle (``libtpb_oracle.so``).

TEST INFRASTRUCTURE ONLY.  The oracle restates TensorPencil's CPU arithmetic
for the quantized-linear path (see ``tpb_oracle.h`` for the per-function
source citations).  Only the tests, the smoke check and the CPU-baseline legs
of the benchmark may import this module; the shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtpb_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "tpb_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE, "-B", "libtpb_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.tpo_f16_to_f32.restype = C.c_float
        _lib.tpo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.tpo_f32_to_f16.restype = C.c_uint16
        _lib.tpo_f32_to_f16.argtypes = [C.c_float]
        _lib.tpo_nibble_i4.restype = C.c_int8
        _lib.tpo_nibble_i4.argtypes = [C.c_uint8, C.c_int]
        _lib.tpo_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().tpo_num_threads())


# -- ConvRot ----------------------------------------------------------------

def rotate(x: np.ndarray) -> np.ndarray:
    out = _c(x, np.float32).copy()
    assert out.shape[-1] % 256 == 0
    rows = out.reshape(-1, out.shape[-1])
    for r in rows:
        lib().tpo_convrot_rotate(_p(r), C.c_size_t(r.size))
    return out


def hadamard256() -> np.ndarray:
    h = np.empty((256, 256), np.float32)
    lib().tpo_hadamard256(_p(h))
    return h


def nibble_i4(byte: int, idx: int) -> int:
    return int(lib().tpo_nibble_i4(byte, idx))


def unpack_i4(packed: np.ndarray, n_elems: int | None = None) -> np.ndarray:
    packed = _c(packed, np.uint8)
    n = packed.size * 2 if n_elems is None else n_elems
    out = np.empty(n, np.int8)
    lib().tpo_unpack_i4(_p(packed), C.c_size_t(n), _p(out))
    return out.reshape(packed.shape[:-1] + (packed.shape[-1] * 2,)) if n_elems is None else out


def pack_i4(vals: np.ndarray) -> np.ndarray:
    vals = _c(vals, np.int8)
    out = np.empty(vals.size // 2, np.uint8)
    lib().tpo_pack_i4(_p(vals), C.c_size_t(vals.size), _p(out))
    return out.reshape(vals.shape[:-1] + (vals.shape[-1] // 2,))


def i4_convrot_dequant(packed: np.ndarray, row_scale: np.ndarray, rows: int, cols: int) -> np.ndarray:
    packed = _c(packed, np.uint8)
    row_scale = _c(row_scale, np.float32)
    out = np.empty((rows, cols), np.float32)
    lib().tpo_i4_convrot_dequant(_p(packed), _p(row_scale), C.c_size_t(rows), C.c_size_t(cols), _p(out))
    return out


# -- integer-domain replica --------------------------------------------------

def convrot_prep(x: np.ndarray, bits: int = 8, want_rotated: bool = False):
    """Returns (q int8 [m][k], act_scale f32 [m]) and, if asked, the rotated rows."""
    x = _c(x, np.float32)
    m, k = x.shape
    q = np.empty((m, k), np.int8)
    s = np.empty(m, np.float32)
    xr = np.empty((m, k), np.float32) if want_rotated else None
    lib().tpo_convrot_prep(_p(x), C.c_size_t(m), C.c_size_t(k), C.c_int(bits), _p(q), _p(s),
                           _p(xr) if xr is not None else None)
    return (q, s, xr) if want_rotated else (q, s)


def igemm_s32(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    a = _c(a, np.int8)
    w = _c(w, np.int8)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2
    acc = np.empty((m, n), np.int32)
    lib().tpo_igemm_s32(_p(a), _p(w), C.c_size_t(m), C.c_size_t(n), C.c_size_t(k), _p(acc))
    return acc


def dequant_sim(acc: np.ndarray, act_scale: np.ndarray, w_scale: np.ndarray) -> np.ndarray:
    acc = _c(acc, np.int32)
    m, n = acc.shape
    y = np.empty((m, n), np.float64)
    lib().tpo_dequant_sim(_p(acc), _p(_c(act_scale, np.float32)), _p(_c(w_scale, np.float32)),
                          C.c_size_t(m), C.c_size_t(n), _p(y))
    return y


def linear_truth(xr: np.ndarray, w: np.ndarray, w_scale: np.ndarray) -> np.ndarray:
    xr = _c(xr, np.float32)
    w = _c(w, np.int8)
    m, k = xr.shape
    n = w.shape[0]
    y = np.empty((m, n), np.float64)
    lib().tpo_linear_truth(_p(xr), _p(w), _p(_c(w_scale, np.float32)), C.c_size_t(m),
                           C.c_size_t(n), C.c_size_t(k), _p(y))
    return y


def convrot_linear_sim(x: np.ndarray, w_i8: np.ndarray, w_scale: np.ndarray, bits: int = 8):
    """Whole replica: returns (q, act_scale, acc_s32, y_f64)."""
    q, s = convrot_prep(x, bits)
    acc = igemm_s32(q, w_i8)
    return q, s, acc, dequant_sim(acc, s, w_scale)


# -- `--backend cpu` float path ----------------------------------------------

def linear_cpu_backend(x: np.ndarray, w: np.ndarray, w_bits: int, row_scale: np.ndarray,
                       n: int, k: int, convrot: int = 256, bias=None, nthreads: int = 0,
                       path: str = "auto") -> np.ndarray:
    """The reference's `--backend cpu` linear.  path: "auto" dispatches on the row count as
    matmul.zig:152 does (m < 16: small-m path, else packed); "small" / "packed" force one."""
    x = _c(x, np.float32)
    m = x.shape[0]
    w = _c(w, np.int8 if w_bits == 8 else np.uint8)
    y = np.empty((m, n), np.float32)
    b = _c(bias, np.float32) if bias is not None else None
    fn = {"auto": lib().tpo_linear_cpu_backend, "small": lib().tpo_linear_cpu_small_m,
          "packed": lib().tpo_linear_cpu_packed}[path]
    fn(_p(x), C.c_size_t(m), _p(w), C.c_int(w_bits), _p(_c(row_scale, np.float32)), C.c_size_t(n),
       C.c_size_t(k), C.c_int(convrot), _p(b) if b is not None else None, _p(y), C.c_int(nthreads))
    return y


# -- GGUF Q8_0 ----------------------------------------------------------------

Q8_0_BLOCK_BYTES = 34


def f16_to_f32(h: int) -> float:
    return float(lib().tpo_f16_to_f32(h))


def q8_0_pack(qs: np.ndarray, d_f16: np.ndarray) -> np.ndarray:
    """Assemble Q8_0 rows: qs int8 [n][k], d float16 [n][k/32] -> uint8 [n][k/32*34]."""
    qs = _c(qs, np.int8)
    n, k = qs.shape
    nblk = k // 32
    d16 = _c(d_f16, np.float16).reshape(n, nblk)
    out = np.empty((n, nblk, 34), np.uint8)
    out[:, :, 0:2] = d16.view(np.uint8).reshape(n, nblk, 2)
    out[:, :, 2:] = qs.view(np.uint8).reshape(n, nblk, 32)
    return out.reshape(n, nblk * 34)


def q8_0_dequant_row(blocks: np.ndarray, k: int) -> np.ndarray:
    blocks = _c(blocks, np.uint8)
    out = np.empty(k, np.float32)
    lib().tpo_q8_0_dequant_row(_p(blocks), C.c_size_t(k), _p(out))
    return out


def q8_1_quantize(x: np.ndarray, tie_mode: int = 0):
    x = _c(x, np.float32)
    n = x.size
    d = np.empty(n // 32, np.float32)
    qs = np.empty(n, np.int8)
    lib().tpo_q8_1_quantize(_p(x), C.c_size_t(n), C.c_int(tie_mode), _p(d), _p(qs))
    return d, qs.reshape(x.shape)


def q8_0_gemv_f64(w: np.ndarray, n: int, k: int, x: np.ndarray, scale: float = 1.0) -> np.ndarray:
    w = _c(w, np.uint8)
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), np.float32)
    lib().tpo_q8_0_gemv_f64(_p(w), C.c_size_t(n), C.c_size_t(k), _p(x), C.c_size_t(m),
                            C.c_float(scale), _p(y))
    return y


def q8_0_gemv_q8(w: np.ndarray, n: int, k: int, x: np.ndarray, scale: float = 1.0,
                 tie_mode: int = 0) -> np.ndarray:
    w = _c(w, np.uint8)
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), np.float32)
    lib().tpo_q8_0_gemv_q8(_p(w), C.c_size_t(n), C.c_size_t(k), _p(x), C.c_size_t(m),
                           C.c_float(scale), C.c_int(tie_mode), _p(y))
    return y


def q8_0_block_sumi(w: np.ndarray, n: int, k: int, xq: np.ndarray) -> np.ndarray:
    w = _c(w, np.uint8)
    xq = _c(xq, np.int8).reshape(-1, k)
    m = xq.shape[0]
    out = np.empty((m, n, k // 32), np.int32)
    lib().tpo_q8_0_block_sumi(_p(w), C.c_size_t(n), C.c_size_t(k), _p(xq), C.c_size_t(m), _p(out))
    return out


# -- elementwise neighbours of the linears (producers of the prep input, gated residual) --

def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().tpo_silu_mul(_p(gate), _p(up), C.c_size_t(gate.size), _p(out))
    return out


def sigmoid_mul(dst: np.ndarray, gate: np.ndarray) -> np.ndarray:
    dst, gate = _c(dst, np.float32), _c(gate, np.float32)
    out = np.empty_like(dst)
    lib().tpo_sigmoid_mul(_p(dst), _p(gate), C.c_size_t(dst.size), _p(out))
    return out


def rms_mod(x: np.ndarray, premul: np.ndarray, shift: np.ndarray, eps: float) -> np.ndarray:
    x = _c(x, np.float32)
    rows, dim = x.shape
    premul, shift = _c(premul, np.float32), _c(shift, np.float32)
    assert premul.size == dim and shift.size == dim
    out = np.empty_like(x)
    lib().tpo_rms_mod(_p(x), C.c_size_t(rows), C.c_size_t(dim), _p(premul), _p(shift), C.c_float(eps), _p(out))
    return out


def gated_add(x: np.ndarray, delta: np.ndarray, gate: np.ndarray) -> np.ndarray:
    x, delta, gate = _c(x, np.float32), _c(delta, np.float32), _c(gate, np.float32)
    rows, dim = x.shape
    assert gate.size == dim
    out = np.empty_like(x)
    lib().tpo_gated_add(_p(x), _p(delta), _p(gate), C.c_size_t(rows), C.c_size_t(dim), _p(out))
    return out


# -- other GGUF block formats ---------------------------------------------------------------

GGUF_FMT = {"q8_0": 0, "q4_0": 1, "q4_k": 2, "q5_k": 3, "q6_k": 4, "iq4_nl": 5}


def gguf_row_bytes(fmt: str, k: int) -> int:
    lib().tpo_gguf_row_bytes.restype = C.c_size_t
    return int(lib().tpo_gguf_row_bytes(GGUF_FMT[fmt], C.c_size_t(k)))


def gguf_dequant_row(fmt: str, row: np.ndarray, k: int) -> np.ndarray:
    row = _c(row, np.uint8)
    out = np.empty(k, np.float32)
    lib().tpo_gguf_dequant_row(GGUF_FMT[fmt], _p(row), C.c_size_t(k), _p(out))
    return out


def gguf_gemv_q8(fmt: str, w: np.ndarray, n: int, k: int, x: np.ndarray, scale: float = 1.0) -> np.ndarray:
    """y[m][n]: dequantised weight rows times q8_1-dequantised activations, f64 accumulation."""
    w = _c(w, np.uint8)
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), np.float32)
    lib().tpo_gguf_gemv_q8(GGUF_FMT[fmt], _p(w), C.c_size_t(n), C.c_size_t(k), _p(x), C.c_size_t(m),
                           C.c_float(scale), _p(y))
    return y


# -- attention of the DiT block ---------------------------------------------------------------

def qk_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """x [..., hd] normalised per last-dim row, times w[hd]."""
    x = _c(x, np.float32)
    hd = x.shape[-1]
    out = np.empty_like(x)
    lib().tpo_qk_norm(_p(x), C.c_size_t(x.size // hd), C.c_size_t(hd), _p(_c(w, np.float32)), C.c_float(eps), _p(out))
    return out


def flux_freqs(positions: np.ndarray, axes_dim, theta: float):
    positions = _c(positions, np.float32).reshape(-1, len(axes_dim))
    seq = positions.shape[0]
    half = sum(d // 2 for d in axes_dim)
    cos, sin = np.empty((seq, half), np.float32), np.empty((seq, half), np.float32)
    ad = (C.c_int * len(axes_dim))(*axes_dim)
    lib().tpo_flux_freqs(_p(positions), C.c_size_t(seq), ad, C.c_int(len(axes_dim)), C.c_double(theta), _p(cos), _p(sin))
    return cos, sin


def rope_interleaved(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, heads: int, hd: int) -> np.ndarray:
    out = _c(x, np.float32).copy()
    seq = out.size // (heads * hd)
    lib().tpo_rope_interleaved(_p(out), _p(_c(cos, np.float32)), _p(_c(sin, np.float32)), C.c_size_t(seq),
                               C.c_size_t(heads), C.c_size_t(hd))
    return out


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, heads: int, kv_heads: int, hd: int,
              scale: float = None) -> np.ndarray:
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    seq_q, seq_kv = q.size // (heads * hd), k.size // (kv_heads * hd)
    out = np.empty((seq_q, heads * hd), np.float32)
    lib().tpo_attention(_p(q), _p(k), _p(v), C.c_size_t(seq_q), C.c_size_t(seq_kv), C.c_size_t(heads),
                        C.c_size_t(kv_heads), C.c_size_t(hd), C.c_float(scale if scale is not None else hd ** -0.5),
                        _p(out))
    return out
