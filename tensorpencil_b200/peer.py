"""Peer-mapped output buffers for the N-split GEMM whose epilogue performs the
all-gather itself (``tpb_convrot_gemm_allgather``).

One process per GPU.  Every rank allocates one buffer through the library
(``tpb_peer_alloc``: device memory + a 64-byte IPC handle), the handles travel
through ``torch.distributed.all_gather_object`` (host plumbing), and every rank maps
the others' buffers (``tpb_peer_open``).  The first 256 bytes of a buffer hold the
barrier flags; the payload (the full row-major y) starts at ``PAYLOAD_OFFSET``.

The reference is single-GPU (src/gpu/cuda/context.zig:111); nothing here has a
reference counterpart.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib
from .offload import _DevView

PAYLOAD_OFFSET = 256
_TYPESTR = {torch.float32: "<f4", torch.bfloat16: None, torch.int32: "<i4"}


class PeerBuffers:
    """One buffer of ``payload_bytes`` per rank, mapped on every rank."""

    def __init__(self, be, payload_bytes: int, group: Optional[dist.ProcessGroup] = None):
        self.be, self.lib, self.group = be, be.lib, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        self.payload_bytes = payload_bytes
        p = C.c_void_p()
        handle = C.create_string_buffer(64)
        be._check(self.lib.tpb_peer_alloc(be.h, PAYLOAD_OFFSET + payload_bytes, C.byref(p), handle))
        self.local = p.value
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.bases: List[int] = []
        self._opened: List[int] = []
        for r in range(self.world):
            if r == self.rank:
                self.bases.append(self.local)
                continue
            q = C.c_void_p()
            hb = C.create_string_buffer(handles[r], 64)
            be._check(self.lib.tpb_peer_open(be.h, hb, C.byref(q)))
            self.bases.append(q.value)
            self._opened.append(q.value)
        self.epoch = 0
        self._flags = (C.c_void_p * self.world)(*self.bases)
        self._ys = (C.c_void_p * self.world)(*[b + PAYLOAD_OFFSET for b in self.bases])
        dist.barrier(group=group)   # everyone has mapped everyone before any kernel writes

    def tensor(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """This rank's payload as a torch tensor (no copy)."""
        n = 1
        for s in shape:
            n *= s
        if dtype == torch.bfloat16:
            t = torch.as_tensor(_DevView(self.local + PAYLOAD_OFFSET, (n,), "<i2"), device=self.be.device)
            return t.view(torch.bfloat16).view(*shape)
        t = torch.as_tensor(_DevView(self.local + PAYLOAD_OFFSET, (n,), _TYPESTR[dtype]), device=self.be.device)
        return t.view(*shape)

    def barrier(self, timeout_ms: int = 2000):
        """Device-side barrier over all ranks on the current stream: what every rank
        wrote (into any rank's buffer) before it is visible to kernels launched after
        it.  Bounded wait; a timeout shows up in ``Backend.status_poll``."""
        self.epoch += 1
        self.be._check(self.lib.tpb_peer_barrier(self.be.h, self.be._stream(), self._flags, self.world, self.rank,
                                                 self.epoch, timeout_ms))
        self.be.launches += 1

    def gemm_allgather(self, w_shard: torch.Tensor, w_scale_shard: torch.Tensor, n_shard: int, w_bits: int,
                       y_dtype: torch.dtype = torch.float32, ldy: Optional[int] = None):
        """GEMM of the backend's prepped activations against this rank's weight rows;
        the epilogue writes columns [rank*n_shard, (rank+1)*n_shard) of every rank's y.
        Call ``barrier()`` before reading y and before the next overwrite."""
        be = self.be
        assert be.i8_bits == w_bits, "must follow the matching prep"
        if w_bits == 4:
            be.reserveW4(n_shard, be.i8_cols)
        ld = ldy if ldy is not None else n_shard * self.world
        esz = 2 if y_dtype == torch.bfloat16 else 4
        if be.i8_m * ld * esz > self.payload_bytes:
            raise ValueError("output does not fit the peer buffer")
        ydt = {torch.float32: _lib.TPB_F32, torch.bfloat16: _lib.TPB_BF16, torch.int32: _lib.TPB_S32}[y_dtype]
        rc = self.lib.tpb_convrot_gemm_allgather(
            be.h, be._stream(), self._ys, self.world, self.rank, ydt, ld, be.i8_x.data_ptr(),
            be.i8_scale.data_ptr(), be.i8_sum.data_ptr() if w_bits == 4 else None, w_shard.data_ptr(), w_bits,
            w_scale_shard.data_ptr() if w_scale_shard is not None else None, be.i8_m, n_shard, be.i8_cols)
        be._check(rc)
        be.launches += 2 if w_bits == 4 else 1

    def gemm_allgather_blocked(self, w_shard: torch.Tensor, w_scale_shard: torch.Tensor, n_shard: int, w_bits: int,
                               y_dtype: torch.dtype = torch.float32):
        """As gemm_allgather, but every rank's shard lands as one contiguous [m][n_shard]
        block: the gathered result is column-blocked [rank][m][n_shard] (``nsplit.assemble``
        turns a [1][world][m][n_shard] view of it into row-major)."""
        be = self.be
        assert be.i8_bits == w_bits, "must follow the matching prep"
        if w_bits == 4:
            be.reserveW4(n_shard, be.i8_cols)
        esz = 2 if y_dtype == torch.bfloat16 else 4
        block = be.i8_m * n_shard * esz
        if block * self.world > self.payload_bytes:
            raise ValueError("output does not fit the peer buffer")
        ydt = {torch.float32: _lib.TPB_F32, torch.bfloat16: _lib.TPB_BF16, torch.int32: _lib.TPB_S32}[y_dtype]
        off = PAYLOAD_OFFSET + self.rank * block
        peers = [b + off for r, b in enumerate(self.bases) if r != self.rank]
        arr = (C.c_void_p * max(1, len(peers)))(*peers)
        rc = self.lib.tpb_convrot_gemm_multi(
            be.h, be._stream(), self.local + off, arr, len(peers), ydt, n_shard, be.i8_x.data_ptr(),
            be.i8_scale.data_ptr(), be.i8_sum.data_ptr() if w_bits == 4 else None, w_shard.data_ptr(), w_bits,
            w_scale_shard.data_ptr() if w_scale_shard is not None else None, be.i8_m, n_shard, be.i8_cols)
        be._check(rc)
        be.launches += 2 if w_bits == 4 else 1

    def close(self):
        if self.local is None:
            return
        torch.cuda.synchronize(self.be.device)
        dist.barrier(group=self.group)      # nobody is still writing into a buffer about to go away
        for q in self._opened:
            self.lib.tpb_peer_close(self.be.h, q)
        self._opened = []
        dist.barrier(group=self.group)
        self.lib.tpb_peer_free(self.be.h, self.local)
        self.local = None


class MulticastBuffers:
    """The same role as PeerBuffers, on torch's symmetric memory: one allocation per rank,
    every rank's copy reachable through the peers' ordinary addresses AND through one
    NVSwitch multicast address, so the GEMM epilogue can send each output tile once
    (``tpb_convrot_gemm_allgather_mc``).  ``available`` is False where the platform has no
    multicast support (no NVSwitch); nothing else is usable then."""

    def __init__(self, be, payload_bytes: int, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.be, self.lib = be, be.lib
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.payload_bytes = payload_bytes
        self._buf = symm_mem.empty(PAYLOAD_OFFSET + payload_bytes, dtype=torch.uint8, device=be.device)
        self._buf.zero_()
        torch.cuda.synchronize(be.device)
        self._hdl = symm_mem.rendezvous(self._buf, self.group)
        self.bases = [int(p) for p in self._hdl.buffer_ptrs]
        self.mc_base = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        self.available = self.mc_base != 0
        self.local = self.bases[self.rank]
        self.epoch = 0
        self._flags = (C.c_void_p * self.world)(*self.bases)
        dist.barrier(group=group)

    tensor = PeerBuffers.tensor
    barrier = PeerBuffers.barrier

    def gemm_allgather(self, w_shard: torch.Tensor, w_scale_shard: torch.Tensor, n_shard: int, w_bits: int,
                       y_dtype: torch.dtype = torch.float32, ldy: Optional[int] = None):
        """As PeerBuffers.gemm_allgather, one multimem store per element instead of world-1
        peer stores plus a local one."""
        be = self.be
        if not self.available:
            raise RuntimeError("no multicast support on this platform")
        assert be.i8_bits == w_bits, "must follow the matching prep"
        if w_bits == 4:
            be.reserveW4(n_shard, be.i8_cols)
        ld = ldy if ldy is not None else n_shard * self.world
        esz = 2 if y_dtype == torch.bfloat16 else 4
        if be.i8_m * ld * esz > self.payload_bytes:
            raise ValueError("output does not fit the buffer")
        ydt = {torch.float32: _lib.TPB_F32, torch.bfloat16: _lib.TPB_BF16, torch.int32: _lib.TPB_S32}[y_dtype]
        rc = self.lib.tpb_convrot_gemm_allgather_mc(
            be.h, be._stream(), self.mc_base + PAYLOAD_OFFSET, self.local + PAYLOAD_OFFSET, self.world, self.rank,
            ydt, ld, be.i8_x.data_ptr(), be.i8_scale.data_ptr(), be.i8_sum.data_ptr() if w_bits == 4 else None,
            w_shard.data_ptr(), w_bits, w_scale_shard.data_ptr() if w_scale_shard is not None else None,
            be.i8_m, n_shard, be.i8_cols)
        be._check(rc)
        be.launches += 2 if w_bits == 4 else 1

    def close(self):
        if self._buf is None:
            return
        torch.cuda.synchronize(self.be.device)
        dist.barrier(group=self.group)      # nobody is still writing into a buffer about to go away
        self._hdl = None
        self._buf = None
        dist.barrier(group=self.group)
