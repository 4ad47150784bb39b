"""Host-side mirror of TensorPencil's ``cuda.Backend`` op surface for the
quantized-linear path (src/gpu/cuda/backend.zig:196), on top of the C ABI of
``libtpb200.so``.

Method names, argument meaning and the hidden prep -> GEMM state follow the
reference so its orchestrators' call sequences carry over unchanged:

    opI8Prep / opI8Gemm / opI4Prep / opI4Gemm      backend.zig:2454-2573
    opGemvQuant / opGemvQuantizeX / opGemvQuantQ8N backend.zig:1660-1735
    prefetchWeight / cachedWeight                  backend.zig:689, :1376-1429
    tensorCreate / tensorUpload / tensorDownload   backend.zig:740, :1257-1269
    beginBatch / endBatch                          backend.zig:1449-1455

Device buffers are ``torch`` CUDA tensors (the reference's ``DeviceBuffer`` is a
raw device pointer + size); weights arrive as host ``numpy`` arrays, as the
reference passes mmap'd checkpoint slices, and are resolved to device copies
through a cache keyed by the host address.

Nothing here computes on the CPU: every op raises if the CUDA library or a
device is missing.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import TPB_BF16, TPB_F16, TPB_F32, TPB_OK, TPB_S32, TpbError

_TORCH_TO_TPB = {torch.float32: TPB_F32, torch.bfloat16: TPB_BF16, torch.float16: TPB_F16,
                 torch.int32: TPB_S32}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Backend:
    """One device, one compute stream (the caller's current torch stream)."""

    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("tensorpencil_b200.Backend needs a CUDA device; there is no CPU path")
        self.lib = _lib.load()
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        torch.cuda.init()
        torch.zeros(1, device=self.device)  # make sure the primary context exists
        h = C.c_void_p()
        rc = self.lib.tpb_create(C.byref(h), device)
        if rc != TPB_OK:
            raise TpbError(rc, self.lib.tpb_status_string(rc).decode())
        self.h = h
        # prep -> GEMM state (backend.zig:336-341)
        self.i8_x: Optional[torch.Tensor] = None
        self.i8_scale: Optional[torch.Tensor] = None
        self.i8_sum: Optional[torch.Tensor] = None
        self.i8_m = 0
        self.i8_cols = 0
        self.i8_bits = 0
        # q8_1 activation scratch of the GEMV path (backend.zig:1691)
        self.q8_act: Optional[torch.Tensor] = None
        # host-pointer-keyed weight cache (backend.zig:1376-1378)
        self._wcache: Dict[Tuple[int, int], Tuple[torch.Tensor, np.ndarray]] = {}
        self.launches = 0  # kernels launched through this backend (bench accounting)
        self._w4_reserved = 0  # elements of int4-expansion scratch reserved in the library

    # -- plumbing -----------------------------------------------------------------
    def close(self):
        if getattr(self, "h", None):
            torch.cuda.synchronize(self.device)
            self.lib.tpb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, rc: int):
        if rc != TPB_OK:
            raise TpbError(rc, self.lib.tpb_last_error(self.h).decode())

    def status_poll(self) -> int:
        """Synchronises and raises TpbError(TPB_ERR_TIMEOUT) if a bounded
        device-side wait gave up."""
        detail = C.c_uint32(0)
        rc = self.lib.tpb_status_poll(self.h, self._stream(), C.byref(detail))
        self._check(rc)
        return int(detail.value)

    def sm_count(self) -> int:
        return int(self.lib.tpb_device_sm_count(self.h))

    # -- tensors (backend.zig:740, :1257-1269) ---------------------------------------
    def tensorCreate(self, nbytes: int) -> torch.Tensor:
        return torch.empty(nbytes, dtype=torch.uint8, device=self.device)

    def tensorUpload(self, dst: torch.Tensor, host: np.ndarray):
        src = torch.from_numpy(np.ascontiguousarray(host)).view(torch.uint8).reshape(-1)
        dst.view(torch.uint8).reshape(-1)[: src.numel()].copy_(src, non_blocking=True)

    def tensorDownload(self, src: torch.Tensor) -> np.ndarray:
        return src.detach().cpu().numpy()

    def beginBatch(self):
        pass

    def endBatch(self):
        torch.cuda.current_stream(self.device).synchronize()

    def cachedWeight(self, host: np.ndarray) -> torch.Tensor:
        """Device copy of a host weight slice, keyed by its address and size."""
        key = (host.__array_interface__["data"][0], host.nbytes)
        hit = self._wcache.get(key)
        if hit is not None:
            return hit[0]
        dev = torch.from_numpy(np.ascontiguousarray(host)).to(self.device, non_blocking=False)
        self._wcache[key] = (dev, host)  # keep the host array alive: the key is its address
        return dev

    def prefetchWeight(self, host: np.ndarray):
        self.cachedWeight(host)

    def dropWeights(self):
        self._wcache.clear()

    def reserveW4(self, n: int, k: int):
        """Sizes the library's int4-expansion scratch for weights of up to n x k elements
        (tpb_convrot_w4_reserve: the one place that allocates; the GEMM entries never do).
        The mirror calls it on first sight of a larger int4 weight, as the reference grows
        its scratch (backend.zig:2457-2470); a host that captures graphs calls it up front."""
        if n * k > self._w4_reserved:
            self._check(self.lib.tpb_convrot_w4_reserve(self.h, n, k))
            self._w4_reserved = n * k

    # -- ConvRot linear ---------------------------------------------------------------
    def _prep(self, x: torch.Tensor, m: int, cols: int, bits: int):
        assert x.is_cuda and x.is_contiguous()
        if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise TypeError("prep input must be f32, f16 or bf16")
        assert x.numel() >= m * cols
        if self.i8_x is None or self.i8_x.numel() < m * cols:
            self.i8_x = torch.empty(max(m * cols, 1), dtype=torch.int8, device=self.device)
        if self.i8_scale is None or self.i8_scale.numel() < m:
            self.i8_scale = torch.empty(max(m, 1), dtype=torch.float32, device=self.device)
            self.i8_sum = torch.empty(max(m, 1), dtype=torch.int32, device=self.device)
        rc = self.lib.tpb_convrot_prep(self.h, self._stream(), x.data_ptr(), _TORCH_TO_TPB[x.dtype],
                                       m, cols, bits, self.i8_x.data_ptr(),
                                       self.i8_scale.data_ptr(), self.i8_sum.data_ptr())
        self._check(rc)
        self.launches += 1
        self.i8_m, self.i8_cols, self.i8_bits = m, cols, bits

    def opI8Prep(self, x: torch.Tensor, m: int, cols: int, in_f16: bool = False):
        """Rotate + per-row quantise x[m][cols] into the backend's prepped
        activation (backend.zig:2454-2480).  ``in_f16`` is implied by x.dtype."""
        self._prep(x, m, cols, 8)

    def opI4Prep(self, x: torch.Tensor, m: int, cols: int):
        """int4 (W4A4) analogue of opI8Prep (backend.zig:2532-2553)."""
        self._prep(x, m, cols, 4)

    # -- elementwise neighbours and the prep with them fused in ---------------------------
    def _prep_fused(self, op: int, a: torch.Tensor, b: Optional[torch.Tensor], premul: Optional[torch.Tensor],
                    shift: Optional[torch.Tensor], eps: float, m: int, cols: int, bits: int):
        assert a.is_cuda and a.is_contiguous() and a.dtype in (torch.float32, torch.bfloat16)
        assert b is None or (b.dtype == a.dtype and b.is_contiguous())
        if self.i8_x is None or self.i8_x.numel() < m * cols:
            self.i8_x = torch.empty(max(m * cols, 1), dtype=torch.int8, device=self.device)
        if self.i8_scale is None or self.i8_scale.numel() < m:
            self.i8_scale = torch.empty(max(m, 1), dtype=torch.float32, device=self.device)
            self.i8_sum = torch.empty(max(m, 1), dtype=torch.int32, device=self.device)
        rc = self.lib.tpb_convrot_prep_fused(self.h, self._stream(), op, a.data_ptr(), _ptr(b), _ptr(premul),
                                             _ptr(shift), eps, _TORCH_TO_TPB[a.dtype], m, cols, bits,
                                             self.i8_x.data_ptr(), self.i8_scale.data_ptr(), self.i8_sum.data_ptr())
        self._check(rc)
        self.launches += 1
        self.i8_m, self.i8_cols, self.i8_bits = m, cols, bits

    def prepSiluMul(self, gate: torch.Tensor, up: torch.Tensor, m: int, cols: int, bits: int = 8):
        """siluMul + op{I8,I4}Prep in one kernel: the prepped activation is
        rotate+quantise(silu(gate) * up) (dit_cuda.zig:513-514 without the round trip)."""
        self._prep_fused(1, gate, up, None, None, 0.0, m, cols, bits)

    def prepSigmoidMul(self, a: torch.Tensor, gate: torch.Tensor, m: int, cols: int, bits: int = 8):
        """sigmoidMul + prep in one kernel (dit_cuda.zig:490-491)."""
        self._prep_fused(2, a, gate, None, None, 0.0, m, cols, bits)

    def prepRmsMod(self, x: torch.Tensor, mod: torch.Tensor, rows: int, dim: int, premul_off: int, shift_off: int,
                   eps: float, bits: int = 8):
        """rmsMod + prep in one kernel (dit_cuda.zig:473-474, :499-500); ``mod`` is
        the reference's modulation buffer, offsets in elements."""
        self._prep_fused(3, x, None, mod[premul_off:premul_off + dim], mod[shift_off:shift_off + dim], eps,
                         rows, dim, bits)

    @staticmethod
    def _check_f32_out(name: str, t: torch.Tensor, total: int):
        """The stand-alone elementwise ops write f32: a narrower or shorter tensor behind
        the output pointer would be overrun on the device, so refuse it here."""
        if t.dtype != torch.float32:
            raise TypeError(f"{name}: the output tensor must be float32 (got {t.dtype}); "
                            "pass a separate f32 output for bf16 inputs")
        if not t.is_contiguous() or t.numel() < total:
            raise ValueError(f"{name}: the output tensor must be contiguous and hold {total} elements")

    @staticmethod
    def _check_in(name: str, t: torch.Tensor, total: int):
        if t.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"{name}: inputs must be float32 or bfloat16 (got {t.dtype})")
        if not t.is_contiguous() or t.numel() < total:
            raise ValueError(f"{name}: input tensors must be contiguous and hold {total} elements")

    def siluMul(self, a: torch.Tensor, b: torch.Tensor, total: int, out: Optional[torch.Tensor] = None):
        """out = silu(a) * b; in place on ``a`` (backend.zig:3310-3315) unless ``out`` is given.
        The result is f32, so the in-place form needs f32 inputs."""
        out = a if out is None else out
        self._check_f32_out("siluMul", out, total)
        self._check_in("siluMul", a, total)
        self._check_in("siluMul", b, total)
        if a.dtype != b.dtype:
            raise TypeError("siluMul: both inputs must have the same dtype")
        self._check(self.lib.tpb_silu_mul(self.h, self._stream(), a.data_ptr(), b.data_ptr(), _TORCH_TO_TPB[a.dtype],
                                          out.data_ptr(), total))
        self.launches += 1

    def sigmoidMul(self, a: torch.Tensor, b: torch.Tensor, total: int, out: Optional[torch.Tensor] = None):
        """out = a * sigmoid(b); in place on ``a`` (backend.zig:3294-3299) unless ``out`` is given."""
        out = a if out is None else out
        self._check_f32_out("sigmoidMul", out, total)
        self._check_in("sigmoidMul", a, total)
        self._check_in("sigmoidMul", b, total)
        if a.dtype != b.dtype:
            raise TypeError("sigmoidMul: both inputs must have the same dtype")
        self._check(self.lib.tpb_sigmoid_mul(self.h, self._stream(), a.data_ptr(), b.data_ptr(),
                                             _TORCH_TO_TPB[a.dtype], out.data_ptr(), total))
        self.launches += 1

    def rmsMod(self, x: torch.Tensor, out: torch.Tensor, mod: torch.Tensor, rows: int, dim: int, premul_off: int,
               shift_off: int, eps: float):
        """out = x * inv_rms(x) * mod[premul_off + c] + mod[shift_off + c] (backend.zig:2738-2760)."""
        self._check_f32_out("rmsMod", out, rows * dim)
        self._check_in("rmsMod", x, rows * dim)
        self._check(self.lib.tpb_rms_mod(self.h, self._stream(), x.data_ptr(), _TORCH_TO_TPB[x.dtype], out.data_ptr(),
                                         mod[premul_off:].data_ptr(), mod[shift_off:].data_ptr(), eps, rows, dim))
        self.launches += 1

    def gatedAdd(self, a: torch.Tensor, b: torch.Tensor, mod: torch.Tensor, total: int, dim: int, gate_off: int):
        """a[row][c] += mod[gate_off + c] * b[row][c] (backend.zig:3342-3347); a is f32."""
        self._check_f32_out("gatedAdd", a, total)
        self._check_in("gatedAdd", b, total)
        self._check(self.lib.tpb_gated_add(self.h, self._stream(), a.data_ptr(), b.data_ptr(), _TORCH_TO_TPB[b.dtype],
                                           mod[gate_off:].data_ptr(), total // dim, dim))
        self.launches += 1

    # -- attention (qk-norm + RoPE + softmax attention) ------------------------------------
    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_norm: torch.Tensor, k_norm: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, heads: int, kv_heads: int, head_dim: int = 128,
                  eps: float = 1e-5, scale: Optional[float] = None, out_dtype=torch.bfloat16,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """qkNorm + rope on q and k, then attn (dit_cuda.zig:479-489) in two library calls.
        q [seq][heads*hd], k / v [seq][kv_heads*hd] (f32 or bf16); cos / sin [seq][hd/2]."""
        seq = q.shape[0]
        assert q.dtype == k.dtype == v.dtype and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
        key = (seq, heads, kv_heads)
        if getattr(self, "_attn_key", None) != key:
            self._attn_qb = torch.empty((heads, seq, head_dim), dtype=torch.bfloat16, device=self.device)
            self._attn_kb = torch.empty((kv_heads, seq, head_dim), dtype=torch.bfloat16, device=self.device)
            self._attn_vt = torch.empty(self.lib.tpb_attn_vt_elems(seq, kv_heads), dtype=torch.bfloat16, device=self.device)
            self._attn_key = key
        self._check(self.lib.tpb_attn_prepare(self.h, self._stream(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                              _TORCH_TO_TPB[q.dtype], q_norm.data_ptr(), k_norm.data_ptr(), eps,
                                              cos.data_ptr(), sin.data_ptr(), seq, heads, kv_heads, head_dim,
                                              self._attn_qb.data_ptr(), self._attn_kb.data_ptr(), self._attn_vt.data_ptr()))
        if out is None:
            out = torch.empty((seq, heads * head_dim), dtype=out_dtype, device=self.device)
        self._check(self.lib.tpb_attention(self.h, self._stream(), out.data_ptr(), _TORCH_TO_TPB[out.dtype],
                                           self._attn_qb.data_ptr(), self._attn_kb.data_ptr(), self._attn_vt.data_ptr(),
                                           seq, seq, heads, kv_heads, head_dim,
                                           float(scale if scale is not None else head_dim ** -0.5)))
        self.launches += 4
        return out

    def _gemm(self, y: torch.Tensor, w_bytes: np.ndarray, weight_scale: np.ndarray, rows: int,
              w_bits: int, ldy: Optional[int] = None):
        assert self.i8_bits == w_bits, "opI{8,4}Gemm must follow the matching prep"
        w_dev = self.cachedWeight(w_bytes) if isinstance(w_bytes, np.ndarray) else w_bytes
        ws_dev = self.cachedWeight(weight_scale) if isinstance(weight_scale, np.ndarray) else weight_scale
        ydt = _TORCH_TO_TPB[y.dtype]
        if w_bits == 4:
            self.reserveW4(rows, self.i8_cols)
        rc = self.lib.tpb_convrot_gemm(self.h, self._stream(), y.data_ptr(), ydt,
                                       ldy if ldy is not None else rows,
                                       self.i8_x.data_ptr(), self.i8_scale.data_ptr(),
                                       self.i8_sum.data_ptr() if w_bits == 4 else None,
                                       w_dev.data_ptr(), w_bits, _ptr(ws_dev),
                                       self.i8_m, rows, self.i8_cols)
        self._check(rc)
        self.launches += 2 if w_bits == 4 else 1

    def gemmGatedAdd(self, x: torch.Tensor, w_bytes, weight_scale, rows: int, mod: torch.Tensor, gate_off: int,
                     w_bits: int = 8):
        """opI{8,4}Gemm + gatedAdd in one kernel: x[m][rows] += mod[gate_off + c] * linear(prepped)
        (dit_cuda.zig:492-493, :515-516).  x is f32, updated in place."""
        assert self.i8_bits == w_bits and x.dtype == torch.float32 and x.is_contiguous()
        w_dev = self.cachedWeight(w_bytes) if isinstance(w_bytes, np.ndarray) else w_bytes
        ws_dev = self.cachedWeight(weight_scale) if isinstance(weight_scale, np.ndarray) else weight_scale
        if w_bits == 4:
            self.reserveW4(rows, self.i8_cols)
        rc = self.lib.tpb_convrot_gemm_gated_add(self.h, self._stream(), x.data_ptr(), rows, mod[gate_off:].data_ptr(),
                                                 self.i8_x.data_ptr(), self.i8_scale.data_ptr(),
                                                 self.i8_sum.data_ptr() if w_bits == 4 else None, w_dev.data_ptr(),
                                                 w_bits, _ptr(ws_dev), self.i8_m, rows, self.i8_cols)
        self._check(rc)
        self.launches += 2 if w_bits == 4 else 1

    def gemmSiluPair(self, y: torch.Tensor, w_gate, gate_scale, w_up, up_scale, rows: int, w_bits: int = 8):
        """mlp.gate GEMM + mlp.up GEMM + siluMul in one kernel: y[m][rows] = silu(linear_gate(prepped)) *
        linear_up(prepped) (dit_cuda.zig:508-513).  y is f32 or bf16."""
        assert self.i8_bits == w_bits and y.dtype in (torch.float32, torch.bfloat16) and y.stride(-1) == 1
        dev = [self.cachedWeight(a) if isinstance(a, np.ndarray) else a for a in (w_gate, gate_scale, w_up, up_scale)]
        if w_bits == 4:
            self.reserveW4(2 * rows, self.i8_cols)
        rc = self.lib.tpb_convrot_gemm_silu_pair(self.h, self._stream(), y.data_ptr(), _TORCH_TO_TPB[y.dtype], y.stride(0),
                                                 self.i8_x.data_ptr(), self.i8_scale.data_ptr(),
                                                 self.i8_sum.data_ptr() if w_bits == 4 else None,
                                                 dev[0].data_ptr(), _ptr(dev[1]), dev[2].data_ptr(), _ptr(dev[3]),
                                                 w_bits, self.i8_m, rows, self.i8_cols)
        self._check(rc)
        self.launches += 3 if w_bits == 4 else 1

    def gemmGroup(self, ys, weights, scales, rows: int, w_bits: int = 8):
        """Up to four op{I8,I4}Gemm calls on the same prepped activations in one launch (q, k, v and gate of a DiT
        block, dit_cuda.zig:473-478): ys[g][m][rows] = linear_g(prepped), bit-identical to the separate calls.  The
        outputs share dtype (f32 or bf16) and row stride."""
        n = len(ys)
        assert 1 <= n <= 4 and len(weights) == n and len(scales) == n and self.i8_bits == w_bits
        assert all(y.dtype == ys[0].dtype and y.stride(-1) == 1 and y.stride(0) == ys[0].stride(0) for y in ys)
        w_dev = [self.cachedWeight(a) if isinstance(a, np.ndarray) else a for a in weights]
        s_dev = [self.cachedWeight(a) if isinstance(a, np.ndarray) else a for a in scales]
        if w_bits == 4:
            self.reserveW4(n * rows, self.i8_cols)
        arr = C.c_void_p * n
        rc = self.lib.tpb_convrot_gemm_group(self.h, self._stream(), n, arr(*[y.data_ptr() for y in ys]),
                                             _TORCH_TO_TPB[ys[0].dtype], ys[0].stride(0), self.i8_x.data_ptr(),
                                             self.i8_scale.data_ptr(), self.i8_sum.data_ptr() if w_bits == 4 else None,
                                             arr(*[w.data_ptr() for w in w_dev]), arr(*[_ptr(a) for a in s_dev]),
                                             w_bits, self.i8_m, rows, self.i8_cols)
        self._check(rc)
        self.launches += n + 1 if w_bits == 4 else 1

    def opI8Gemm(self, y: torch.Tensor, w_bytes, weight_scale, rows: int, c_h16: bool = False):
        """y[m][rows] = prepped @ W^T * act_scale[row] * weight_scale[col]
        (backend.zig:2484-2501).  The output type is y.dtype (f32 or bf16; int32
        stores the raw accumulators)."""
        self._gemm(y, w_bytes, weight_scale, rows, 8)

    def opI4Gemm(self, y: torch.Tensor, w_bytes, weight_scale, rows: int):
        """int4 GEMM + fused rescale against the last opI4Prep; ``w_bytes`` is the
        packed weight [rows][cols/2] (backend.zig:2558-2573)."""
        self._gemm(y, w_bytes, weight_scale, rows, 4)

    # -- Q8_0 GEMV ------------------------------------------------------------------------
    def opGemvQuantizeX(self, x: torch.Tensor, cols: int):
        """Quantise f32 activations (cols = total element count, a multiple of
        32) into the shared q8 scratch: f32 d[cols/32] then int8 qs[cols]
        (backend.zig:1687-1695)."""
        assert x.dtype == torch.float32 and x.is_cuda and cols % 32 == 0
        need = cols // 32 * 4 + cols
        if self.q8_act is None or self.q8_act.numel() < need:
            self.q8_act = torch.empty(need, dtype=torch.uint8, device=self.device)
        self._q8_total = cols
        rc = self.lib.tpb_q8_1_quantize(self.h, self._stream(), x.data_ptr(), cols, self.q8_act.data_ptr())
        self._check(rc)
        self.launches += 1

    def opGemvQuantQ8N(self, dt: str, y: torch.Tensor, w_bytes, scale: float, rows: int, cols: int,
                       ng: int, row_off: int, n_total: int):
        """Grouped dp4a GEMV: y[i][rows] = scale * (W @ x_hat[row_off+i]) for i < ng <= 8
        against the activations staged by ONE opGemvQuantizeX(x, n_total*cols)
        (backend.zig:1719-1735)."""
        from ._lib import GGUF_FMT
        if dt not in GGUF_FMT:
            raise NotImplementedError(f"GEMV weight format {dt!r} is not implemented (q8_0, q4_0, q4_k, q5_k, q6_k, iq4_nl are)")
        assert self.q8_act is not None and self._q8_total == n_total * cols
        w_dev = self.cachedWeight(w_bytes) if isinstance(w_bytes, np.ndarray) else w_bytes
        rc = self.lib.tpb_gguf_gemv_q8n(self.h, self._stream(), GGUF_FMT[dt], y.data_ptr(), w_dev.data_ptr(),
                                        float(scale), rows, cols, self.q8_act.data_ptr(), ng,
                                        row_off, n_total)
        self._check(rc)
        self.launches += 1

    def opGemvQuant(self, dt: str, y: torch.Tensor, x: torch.Tensor, w_bytes, scale: float, rows: int,
                    cols: int):
        """M = 1 GEMV in f32 arithmetic on un-quantised x (backend.zig:1660-1681)."""
        if dt != "q8_0":
            raise NotImplementedError(f"GEMV weight format {dt!r} is outside this library's scope")
        w_dev = self.cachedWeight(w_bytes) if isinstance(w_bytes, np.ndarray) else w_bytes
        rc = self.lib.tpb_q8_0_gemv_f32(self.h, self._stream(), y.data_ptr(), x.data_ptr(),
                                        w_dev.data_ptr(), float(scale), rows, cols)
        self._check(rc)
        self.launches += 1

    # -- composites the harness uses -----------------------------------------------------
    def convrot_linear(self, x: torch.Tensor, w, w_scale, n: int, bits: int,
                       out_dtype=torch.float32, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """prep + GEMM for one linear through the one-call entry point; x is [m][k] on the
        device.  ``y`` may be passed in to avoid the allocation."""
        m, k = x.shape
        if y is None:
            y = torch.empty((m, n), dtype=out_dtype, device=self.device)
        assert x.is_cuda and x.is_contiguous()
        if isinstance(w, np.ndarray):
            w = self.cachedWeight(w)
        if isinstance(w_scale, np.ndarray):
            w_scale = self.cachedWeight(w_scale)
        if self.i8_x is None or self.i8_x.numel() < m * k:
            self.i8_x = torch.empty(max(m * k, 1), dtype=torch.int8, device=self.device)
        if self.i8_scale is None or self.i8_scale.numel() < m:
            self.i8_scale = torch.empty(max(m, 1), dtype=torch.float32, device=self.device)
            self.i8_sum = torch.empty(max(m, 1), dtype=torch.int32, device=self.device)
        if bits == 4:
            self.reserveW4(n, k)
        rc = self.lib.tpb_convrot_linear(self.h, self._stream(), y.data_ptr(), _TORCH_TO_TPB[y.dtype], n,
                                         x.data_ptr(), _TORCH_TO_TPB[x.dtype], self.i8_x.data_ptr(),
                                         self.i8_scale.data_ptr(), self.i8_sum.data_ptr(), w.data_ptr(), bits,
                                         _ptr(w_scale), m, n, k)
        self._check(rc)
        self.launches += 3 if bits == 4 else 2
        self.i8_m, self.i8_cols, self.i8_bits = m, k, bits
        return y

    def convrot_linear_host(self, x_host: torch.Tensor, w, w_scale, n: int, bits: int,
                            y_host: torch.Tensor, chunk_rows: int = 512, copy_only: bool = False):
        """The same linear with HOST activations and a HOST result (pinned
        tensors) -- the shape of a call from a host-resident orchestrator
        (tensorUpload / op / tensorDownload, src/models/dit_cuda.zig:430-433, :527).
        Weights stay in the device-side weight cache as in the reference.

        The rows are independent, so the call is pipelined in chunks of
        ``chunk_rows``: chunk i+1 uploads on one side stream while chunk i is
        prepped and multiplied on the current stream and chunk i-1 downloads on a
        second side stream (PCIe is full duplex).  An INT4 weight is widened once
        per call, not once per chunk.  On return everything is enqueued and the
        current stream waits for the last download.

        ``copy_only`` runs the same uploads and downloads over the same buffers, streams and
        events with no kernel between them: the floor the host link sets for this call."""
        m, k = x_host.shape
        key = (m, k, n, x_host.dtype, y_host.dtype)
        if getattr(self, "_host_io_key", None) != key:
            self._host_x = torch.empty((m, k), dtype=x_host.dtype, device=self.device)
            self._host_y = torch.empty((m, n), dtype=y_host.dtype, device=self.device)
            self._host_io_key = key
        if getattr(self, "_s_in", None) is None:
            self._s_in = torch.cuda.Stream(device=self.device)
            self._s_out = torch.cuda.Stream(device=self.device)
        cur = torch.cuda.current_stream(self.device)
        w8 = w
        if bits == 4 and not copy_only:
            if getattr(self, "_host_w8", None) is None or self._host_w8.numel() < n * k:
                self._host_w8 = torch.empty(n * k, dtype=torch.int8, device=self.device)
            self._check(self.lib.tpb_convrot_w4_expand(self.h, self._stream(), w.data_ptr(), n, k,
                                                       self._host_w8.data_ptr()))
            self.launches += 1
            w8 = self._host_w8
        bounds = [(r0, min(r0 + chunk_rows, m)) for r0 in range(0, m, chunk_rows)]
        self._s_in.wait_stream(cur)            # earlier work on the staging buffers is done
        uploaded = []
        with torch.cuda.stream(self._s_in):
            for r0, r1 in bounds:
                self._host_x[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._s_in)
                uploaded.append(ev)
        ydt = _TORCH_TO_TPB[y_host.dtype]
        for (r0, r1), ev in zip(bounds, uploaded):
            cur.wait_event(ev)
            if not copy_only:
                self._prep(self._host_x[r0:r1], r1 - r0, k, bits)
                rc = self.lib.tpb_convrot_gemm(self.h, self._stream(), self._host_y[r0:r1].data_ptr(), ydt, n,
                                               self.i8_x.data_ptr(), self.i8_scale.data_ptr(), None,
                                               w8.data_ptr(), 8, _ptr(w_scale), r1 - r0, n, k)
                self._check(rc)
                self.launches += 1
            done = torch.cuda.Event()
            done.record(cur)
            self._s_out.wait_event(done)
            with torch.cuda.stream(self._s_out):
                y_host[r0:r1].copy_(self._host_y[r0:r1], non_blocking=True)
        cur.wait_stream(self._s_out)

    def q8_0_linear(self, x: torch.Tensor, w, n: int, k: int, scale: float = 1.0) -> torch.Tensor:
        """Decode linear the way the reference's steppers dispatch it
        (src/models/qwen3_cuda.zig:1497-1517): quantise all rows once, then one
        grouped GEMV per 8 activation rows."""
        m = x.shape[0]
        y = torch.empty((m, n), dtype=torch.float32, device=self.device)
        self.opGemvQuantizeX(x, m * k)
        for r0 in range(0, m, 8):
            ng = min(8, m - r0)
            self.opGemvQuantQ8N("q8_0", y[r0:], w, scale, n, k, ng, r0, m)
        return y
