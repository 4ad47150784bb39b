"""Weight streaming on top of the C ABI's ``tpb_stream_*`` entry points: the
host-side counterpart of the reference's ``prefetchBlock`` /
``cachedWeight`` flow (src/models/dit_cuda.zig:322-334, :462-470;
src/gpu/cuda/backend.zig:689-736, :1376-1429).

A *layer* is the set of arrays one transformer block needs (packed weights and
their scales); its arrays are packed once into one pinned host image so a layer
moves with a single host-to-device copy.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ._lib import TPB_OK, TpbError

_ALIGN = 256


class _DevView:
    """Exposes a raw device address to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape: Tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


def packed_size(arrays: Sequence[np.ndarray]) -> int:
    off = 0
    for a in arrays:
        off = (off + _ALIGN - 1) // _ALIGN * _ALIGN + a.nbytes
    return off


class Streamer:
    def __init__(self, backend, budget_bytes: int, slot_bytes: int, n_slots: int):
        self.be = backend
        self.lib = backend.lib
        s = C.c_void_p()
        rc = self.lib.tpb_stream_open(backend.h, budget_bytes, slot_bytes, n_slots, C.byref(s))
        backend._check(rc)
        self.s = s
        self._images: Dict[int, Tuple[int, int]] = {}            # layer -> (pinned ptr, bytes)
        self._layout: Dict[int, List[Tuple[int, tuple, str]]] = {}  # layer -> [(offset, shape, typestr)]

    def _check(self, rc: int):
        if rc != TPB_OK:
            raise TpbError(rc, self.lib.tpb_last_error(self.be.h).decode())

    def register(self, layer_id: int, arrays: Sequence[np.ndarray]):
        total = packed_size(arrays)
        p = C.c_void_p()
        self._check(self.lib.tpb_host_alloc(self.be.h, total, C.byref(p)))
        img = (C.c_uint8 * total).from_address(p.value)
        view = np.frombuffer(img, dtype=np.uint8)
        layout = []
        off = 0
        for a in arrays:
            a = np.ascontiguousarray(a)
            off = (off + _ALIGN - 1) // _ALIGN * _ALIGN
            view[off:off + a.nbytes] = a.view(np.uint8).reshape(-1)
            layout.append((off, tuple(a.shape), a.dtype.str))
            off += a.nbytes
        rc = self.lib.tpb_stream_register(self.s, layer_id, p, total)
        if rc != TPB_OK:
            self.lib.tpb_host_free(self.be.h, p)
            self._check(rc)
        old = self._images.get(layer_id)
        if old:
            self.lib.tpb_host_free(self.be.h, C.c_void_p(old[0]))
        self._images[layer_id] = (p.value, total)
        self._layout[layer_id] = layout

    def prefetch(self, layer_id: int):
        self._check(self.lib.tpb_stream_prefetch(self.s, layer_id))

    def acquire(self, layer_id: int) -> List[torch.Tensor]:
        """Makes the current stream wait for the layer's copy and returns device
        views of its arrays (valid until release)."""
        dev = C.c_void_p()
        self._check(self.lib.tpb_stream_acquire(self.s, layer_id, self.be._stream(), C.byref(dev)))
        return [torch.as_tensor(_DevView(dev.value + off, shape, ts), device=self.be.device)
                for off, shape, ts in self._layout[layer_id]]

    def release(self, layer_id: int):
        self._check(self.lib.tpb_stream_release(self.s, layer_id, self.be._stream()))

    def bytes_copied(self) -> int:
        return int(self.lib.tpb_stream_bytes_copied(self.s))

    def close(self):
        if self.s:
            self.lib.tpb_stream_close(self.s)
            self.s = None
            for p, _ in self._images.values():
                self.lib.tpb_host_free(self.be.h, C.c_void_p(p))
            self._images.clear()
