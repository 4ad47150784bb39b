"""Weight streaming on top of the C ABI's ``tpb_stream_*`` entry points: the
host-side counterpart of the reference's ``prefetchBlock`` /
``cachedWeight`` flow (src/models/dit_cuda.zig:322-334, :462-470;
src/gpu/cuda/backend.zig:689-736, :1376-1429).

A *layer* is the set of arrays one transformer block needs (packed weights and
their scales); its arrays are packed once into one pinned host image so a layer
moves with a single host-to-device copy.

With ``group`` (a torch.distributed process group, one rank per GPU of a node, every
rank holding the same layers) the ranks share the host link: a rank copies only its
1/world piece of a layer through PCIe and the pieces are exchanged over NVLink by an
in-place all-gather on the transfer stream, so a layer crosses the host link once per
node instead of once per GPU.  Every rank must prefetch the same layers in the same order.
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


def slot_size(image_bytes: int, world: int = 1) -> int:
    """Slot size for images of `image_bytes`: with `world` ranks sharing the link a slot holds
    `world` equal pieces rounded up to 256 bytes (tpb_stream_piece_bytes)."""
    if world <= 1:
        return image_bytes
    piece = (image_bytes + world - 1) // world
    return (piece + 255) // 256 * 256 * world


class Streamer:
    def __init__(self, backend, budget_bytes: int, slot_bytes: int, n_slots: int, group=None):
        self.be = backend
        self.lib = backend.lib
        self.group = group
        self.world = 1
        self.rank = 0
        if group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        s = C.c_void_p()
        rc = self.lib.tpb_stream_open(backend.h, budget_bytes, slot_bytes, n_slots, C.byref(s))
        backend._check(rc)
        self.s = s
        self._xfer = None
        if self.world > 1:
            self._xfer = torch.cuda.ExternalStream(int(self.lib.tpb_stream_transfer_stream(self.s)), device=backend.device)
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
        if self.world == 1:
            self._check(self.lib.tpb_stream_prefetch(self.s, layer_id))
            return
        import torch.distributed as dist
        dev = C.c_void_p()
        self._check(self.lib.tpb_stream_prefetch_part(self.s, layer_id, self.rank, self.world, C.byref(dev)))
        if not dev.value:
            return      # resident or on its way, on every rank alike
        piece = int(self.lib.tpb_stream_piece_bytes(self._images[layer_id][1], self.world))
        slot = torch.as_tensor(_DevView(dev.value, (self.world * piece,), "|u1"), device=self.be.device)
        with torch.cuda.stream(self._xfer):
            # in place: this rank's piece already sits at its offset
            dist.all_gather_into_tensor(slot, slot[self.rank * piece:(self.rank + 1) * piece], group=self.group)
        self._check(self.lib.tpb_stream_commit(self.s, layer_id))

    def acquire(self, layer_id: int) -> List[torch.Tensor]:
        """Makes the current stream wait for the layer's copy and returns device
        views of its arrays (valid until release)."""
        if self.world > 1:
            self.prefetch(layer_id)     # no-op when the layer is resident or on its way
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
