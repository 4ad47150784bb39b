"""On-disk checkpoint formats for the quantized-linear path, and a budgeted device
weight cache: what turns the synthetic harness into something that loads files.

* ``SafeTensors``: the safetensors container (8-byte little-endian header length, JSON
  header, raw tensor bytes), memory-mapped, read-only -- src/core/safetensors.zig.
* ``load_convrot_weight``: the reference's ConvRot weight resolution on top of it
  (src/models/dit.zig:690-722): int4 weights are nibble-packed ``[rows][cols/2]`` bytes
  stored as ``U8`` (the reference's converter) or ``I8`` (ComfyUI's W4A4 converter); a real
  int8 weight is ``I8`` at the full ``[rows][cols]``: int4 is told from int8 by the halved
  column count, not by dtype alone; either comes with a per-output-row ``<name>_scale``.
* ``Gguf``: the GGUF container (magic, version 2 or 3, typed metadata, tensor table with
  ggml type ids, data section aligned to ``general.alignment``) -- src/core/gguf.zig:1-60,
  :200-295.  Dimensions are stored fastest-first and are reversed into row-major order.
* ``WeightCache``: device copies of host weights under a byte budget with LRU eviction
  and pinning -- the policy side of Backend.cachedWeight / ``--vram-budget``
  (src/gpu/cuda/backend.zig:1376-1445, src/pipeline.zig:603-652).

Errors carry the reference's error names (MissingTensor, ShapeMismatch, InvalidHeader, ...).
"""
from __future__ import annotations

import json
import mmap
import struct
from collections import OrderedDict
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np


class FormatError(ValueError):
    """``name`` is the reference's error tag (error.MissingTensor and so on)."""

    def __init__(self, name: str, detail: str = ""):
        super().__init__(f"{name}: {detail}" if detail else name)
        self.name = name


# ---------------------------------------------------------------------------------------
# safetensors
# ---------------------------------------------------------------------------------------

_ST_DTYPES = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2), "I8": (np.int8, 1),
              "U8": (np.uint8, 1), "I32": (np.int32, 4), "I64": (np.int64, 8), "F8_E4M3": (np.uint8, 1)}


@dataclass
class TensorView:
    name: str
    dtype: str                 # the container's dtype tag ("I8", "Q4_K", ...)
    shape: Tuple[int, ...]     # row-major
    data: np.ndarray           # uint8 view into the mapping

    def elem_count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def to_f32(self) -> np.ndarray:
        """toF32Alloc: f32 / f16 / bf16 tensors as float32."""
        if self.dtype == "F32":
            return self.data.view(np.float32).copy().reshape(self.shape)
        if self.dtype == "F16":
            return self.data.view(np.float16).astype(np.float32).reshape(self.shape)
        if self.dtype == "BF16":
            return (self.data.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(self.shape)
        raise FormatError("UnsupportedDType", f"{self.name}: {self.dtype} has no f32 view")


class SafeTensors:
    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise FormatError("FileTooSmall")
        (hlen,) = struct.unpack_from("<Q", self._mm, 0)
        if hlen > len(self._mm) - 8:
            raise FormatError("InvalidHeader", "header length exceeds the file")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise FormatError("InvalidHeader", str(e))
        self.metadata = header.pop("__metadata__", {})
        payload = np.frombuffer(self._mm, dtype=np.uint8, offset=8 + hlen)
        self.tensors: Dict[str, TensorView] = {}
        for name, info in header.items():
            dt = info.get("dtype")
            shape = tuple(info.get("shape", ()))
            lo, hi = info.get("data_offsets", (0, 0))
            if dt not in _ST_DTYPES:
                raise FormatError("UnsupportedDType", f"{name}: {dt}")
            if any((not isinstance(s, int)) or s < 0 for s in shape):
                raise FormatError("InvalidShape", name)
            n = 1
            for s in shape:
                n *= s
            if not (0 <= lo <= hi <= payload.size) or hi - lo != n * _ST_DTYPES[dt][1]:
                raise FormatError("InvalidOffsets", name)
            self.tensors[name] = TensorView(name, dt, shape, payload[lo:hi])

    def get(self, name: str) -> Optional[TensorView]:
        return self.tensors.get(name)

    def close(self):
        self.tensors = {}
        try:
            self._mm.close()
        except BufferError:      # views still alive: the mapping goes with them
            pass
        self._f.close()


CONVROT_GROUP = 256   # src/ops/convrot.zig


@dataclass
class ConvRotWeight:
    w: np.ndarray            # int8 [rows][cols] (bits 8) or packed uint8 [rows][cols/2] (bits 4)
    row_scale: np.ndarray    # f32 [rows]
    bits: int
    rows: int
    cols: int


def load_convrot_weight(st: SafeTensors, name: str, rows: int, cols: int, prefix: str = "") -> ConvRotWeight:
    """Loader.mat for an int8/int4 ConvRot weight (src/models/dit.zig:690-722)."""
    view = st.get(prefix + name)
    if view is None:
        raise FormatError("MissingTensor", prefix + name)
    shape = view.shape
    halved = len(shape) == 2 and shape[0] == rows and cols % 2 == 0 and shape[1] == cols // 2
    is_i4 = view.dtype == "U8" or (view.dtype == "I8" and halved)
    if not is_i4 and view.dtype != "I8":
        raise FormatError("UnsupportedCheckpoint", f"{name}: {view.dtype} is not a ConvRot weight")
    stored_cols = cols // 2 if is_i4 else cols
    if is_i4 and cols % 2 != 0:
        raise FormatError("ShapeMismatch", name)
    if len(shape) != 2 or shape[0] != rows or shape[1] != stored_cols:
        raise FormatError("ShapeMismatch", f"{name}: {shape} for [{rows}][{cols}]")
    sv = st.get(prefix + name + "_scale")
    if sv is None:
        raise FormatError("MissingTensor", prefix + name + "_scale")
    if sv.elem_count() != rows:
        raise FormatError("ShapeMismatch", name + "_scale")
    if cols % CONVROT_GROUP != 0:
        raise FormatError("ShapeMismatch", f"{name}: cols {cols} is not a multiple of {CONVROT_GROUP}")
    scale = np.ascontiguousarray(sv.to_f32().reshape(rows))
    if is_i4:
        w = view.data.reshape(rows, cols // 2)
    else:
        w = view.data.view(np.int8).reshape(rows, cols)
    return ConvRotWeight(w, scale, 4 if is_i4 else 8, rows, cols)


def write_safetensors(path: str, tensors: Dict[str, Tuple[str, np.ndarray]], metadata: Optional[dict] = None):
    """Writes ``{name: (dtype tag, array)}``: test fixtures and converted checkpoints."""
    header, blobs, off = {}, [], 0
    for name, (dt, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


# ---------------------------------------------------------------------------------------
# GGUF
# ---------------------------------------------------------------------------------------

# ggml type id -> (tag, elements per block, bytes per block)   (src/core/gguf.zig:40-56)
GGML_TYPES = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 8: ("Q8_0", 32, 34), 12: ("Q4_K", 256, 144),
              13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 16: ("I8", 1, 1), 20: ("IQ4_NL", 32, 18),
              26: ("I32", 1, 4), 30: ("BF16", 1, 2)}
GGML_ID = {v[0]: k for k, v in GGML_TYPES.items()}
# tag -> the GEMV format name of this library
GGUF_GEMV_FORMAT = {"Q8_0": "q8_0", "Q4_0": "q4_0", "Q4_K": "q4_k", "Q5_K": "q5_k", "Q6_K": "q6_k", "IQ4_NL": "iq4_nl"}

_KV_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        n = struct.calcsize(fmt)
        if len(self.buf) - self.pos < n:
            raise FormatError("InvalidHeader", "truncated")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += n
        return v

    def string(self):
        n = self.take("<Q")
        if n > len(self.buf) - self.pos:
            raise FormatError("InvalidHeader", "string runs past the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, t):
        if t in _KV_SCALAR:
            return self.take(_KV_SCALAR[t])
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.take("<I"), self.take("<Q")
            if et == 9:
                raise FormatError("InvalidHeader", "nested arrays")
            return [self.value(et) for _ in range(n)]
        raise FormatError("InvalidHeader", f"kv type {t}")



# llama.cpp tensor names -> the HF-style names the model loaders ask for (src/core/gguf.zig:396-480).
# One table for the Qwen / llama family; Gemma's "sandwich" norms rename three entries (there
# ffn_norm is the norm BEFORE the feed-forward block) and Gemma 4 adds a per-layer output scale.
_LAYER_SUFFIX = {
    "attn_norm.weight": "input_layernorm.weight",
    "post_attention_norm.weight": "post_attention_layernorm.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight",
    "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
    "attn_output.weight": "self_attn.o_proj.weight",
}
_LAYER_SUFFIX.update({f"attn_{p}.weight": f"self_attn.{p}_proj.weight" for p in "qkv"})
_LAYER_SUFFIX.update({f"attn_{p}_norm.weight": f"self_attn.{p}_norm.weight" for p in "qk"})
_GEMMA_SUFFIX = dict(_LAYER_SUFFIX, **{"ffn_norm.weight": "pre_feedforward_layernorm.weight",
                                       "post_ffw_norm.weight": "post_feedforward_layernorm.weight"})
_ARCH_SUFFIX = {"gemma3": _GEMMA_SUFFIX, "gemma4": dict(_GEMMA_SUFFIX, **{"layer_output_scale.weight": "out_scale.weight"})}
_TOP_LEVEL = {"token_embd.weight": "embed_tokens.weight", "output_norm.weight": "norm.weight", "output.weight": "lm_head.weight"}


def canonical_name(raw: str, arch: str = "") -> str:
    """``blk.<n>.<suffix>`` -> ``layers.<n>.<HF suffix>`` (suffixes without an entry keep their
    llama.cpp spelling under ``layers.<n>.``); the three top-level names; anything else, HF names
    included, passes through (gguf.zig:454-480)."""
    if raw in _TOP_LEVEL:
        return _TOP_LEVEL[raw]
    if raw.startswith("blk."):
        layer, dot, suffix = raw[4:].partition(".")
        if not dot or not layer.isascii() or not layer.isdigit():
            return raw
        return f"layers.{layer}.{_ARCH_SUFFIX.get(arch, _LAYER_SUFFIX).get(suffix, suffix)}"
    return raw


class Gguf:
    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 24:
            raise FormatError("FileTooSmall")
        r = _Reader(self._mm)
        if bytes(self._mm[0:4]) != b"GGUF":
            raise FormatError("InvalidMagic")
        r.pos = 4
        self.version = r.take("<I")
        if self.version not in (2, 3):
            raise FormatError("UnsupportedVersion", str(self.version))
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        self.alignment = int(self.metadata.get("general.alignment", 32))
        infos = []
        for _ in range(n_tensors):
            name = r.string()
            nd = r.take("<I")
            if nd > 8:
                raise FormatError("InvalidShape", name)
            dims = [r.take("<Q") for _ in range(nd)]
            tid, off = r.take("<I"), r.take("<Q")
            if tid not in GGML_TYPES:
                raise FormatError("UnsupportedTensorType", f"{name}: ggml type {tid}")
            if off % self.alignment != 0:
                raise FormatError("InvalidOffsets", name)
            infos.append((name, tuple(reversed(dims)), tid, off))      # row-major shape
        data_start = (r.pos + self.alignment - 1) // self.alignment * self.alignment
        payload = np.frombuffer(self._mm, dtype=np.uint8, offset=min(data_start, len(self._mm)))
        self.tensors: Dict[str, TensorView] = {}
        self._canonical: Optional[Dict[str, TensorView]] = None
        for name, shape, tid, off in infos:
            tag, be, bb = GGML_TYPES[tid]
            if name in self.tensors:
                raise FormatError("DuplicateTensor", name)
            n = 1
            for s in shape:
                n *= s
            if shape and shape[-1] % be != 0:
                raise FormatError("InvalidShape", f"{name}: last dim {shape[-1]} is not a multiple of {be}")
            nbytes = n // be * bb
            if off + nbytes > payload.size:
                raise FormatError("InvalidOffsets", name)
            self.tensors[name] = TensorView(name, tag, shape, payload[off:off + nbytes])

    def get(self, name: str) -> Optional[TensorView]:
        """By the name in the file or, as the reference's reader stores them (gguf.zig:256), by the
        canonical HF-style name for the file's ``general.architecture``."""
        v = self.tensors.get(name)
        if v is None:
            if self._canonical is None:
                arch = str(self.metadata.get("general.architecture", ""))
                self._canonical = {canonical_name(n, arch): t for n, t in self.tensors.items()}
            v = self._canonical.get(name)
        return v

    def close(self):
        self.tensors = {}
        self._canonical = None
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def write_gguf(path: str, tensors: Dict[str, Tuple[str, Tuple[int, ...], np.ndarray]],
               metadata: Optional[Dict[str, object]] = None, alignment: int = 32, version: int = 3):
    """Writes ``{name: (type tag, row-major shape, raw bytes as uint8)}`` (fixtures)."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    kv = dict(metadata or {})
    if alignment != 32:
        kv["general.alignment"] = alignment
    out = [b"GGUF", struct.pack("<I", version), struct.pack("<QQ", len(tensors), len(kv))]
    for k, v in kv.items():
        out.append(s(k))
        if isinstance(v, bool):
            out.append(struct.pack("<I?", 7, v))
        elif isinstance(v, int):
            out.append(struct.pack("<II", 4, v))
        elif isinstance(v, float):
            out.append(struct.pack("<If", 6, v))
        elif isinstance(v, str):
            out.append(struct.pack("<I", 8) + s(v))
        elif isinstance(v, list):
            out.append(struct.pack("<IIQ", 9, 4, len(v)) + b"".join(struct.pack("<I", int(e)) for e in v))
        else:
            raise TypeError(type(v))
    off, blobs = 0, []
    for name, (tag, shape, raw) in tensors.items():
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        out.append(s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape)) +
                   struct.pack("<IQ", GGML_ID[tag], off))
        blobs.append((off, raw.tobytes()))
        off = (off + raw.size + alignment - 1) // alignment * alignment
    head = b"".join(out)
    pad = -len(head) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        pos = 0
        for o, raw in blobs:
            f.write(b"\0" * (o - pos))
            f.write(raw)
            pos = o + len(raw)


# ---------------------------------------------------------------------------------------
# device weight cache under a budget
# ---------------------------------------------------------------------------------------

class WeightCache:
    """Device copies of host weights keyed by host address, at most ``budget`` bytes:
    least-recently-used entries that are not pinned are dropped to make room
    (cachedWeight + the vram budget, src/gpu/cuda/backend.zig:1376-1445).  ``upload`` maps a
    host array to a device object with ``nbytes``-sized cost (``Backend.cachedWeight`` on a
    GPU, anything on the CPU in tests)."""

    def __init__(self, upload: Callable[[np.ndarray], object], budget: int):
        self.upload, self.budget = upload, budget
        self._lru: "OrderedDict[int, Tuple[object, int, np.ndarray]]" = OrderedDict()
        self._pinned: Dict[int, int] = {}
        self.bytes = 0
        self.hits = self.misses = self.evictions = 0

    @staticmethod
    def _key(host: np.ndarray) -> int:
        return host.__array_interface__["data"][0]

    def get(self, host: np.ndarray, pin: bool = False):
        k = self._key(host)
        ent = self._lru.get(k)
        if ent is not None and ent[1] == host.nbytes:
            self._lru.move_to_end(k)
            self.hits += 1
        else:
            if ent is not None:
                self._drop(k)
            self.misses += 1
            self._make_room(host.nbytes)
            ent = (self.upload(host), host.nbytes, host)     # keeps the host array alive while cached
            self._lru[k] = ent
            self.bytes += host.nbytes
        if pin:
            self._pinned[k] = self._pinned.get(k, 0) + 1
        return ent[0]

    def unpin(self, host: np.ndarray):
        k = self._key(host)
        if self._pinned.get(k, 0) <= 1:
            self._pinned.pop(k, None)
        else:
            self._pinned[k] -= 1

    def _drop(self, k: int):
        _, n, _ = self._lru.pop(k)
        self.bytes -= n
        self._pinned.pop(k, None)

    def _make_room(self, need: int):
        if need > self.budget:
            raise MemoryError(f"DeviceOutOfMemory: weight of {need} bytes exceeds the budget of {self.budget}")
        for k in list(self._lru):
            if self.bytes + need <= self.budget:
                break
            if k in self._pinned:
                continue
            self._drop(k)
            self.evictions += 1
        if self.bytes + need > self.budget:
            raise MemoryError("DeviceOutOfMemory: pinned weights leave no room under the budget")

    def drop_all(self):
        self._lru.clear()
        self._pinned.clear()
        self.bytes = 0
