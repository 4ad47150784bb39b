"""World-size-2 test of the N-split GEMM + all-gather host logic on CPU (gloo).
The shard computation is the CPU checker's integer replica, so the test covers
the sharding, the chunked asynchronous gather and the reassembly; the GPU path
plugs the CUDA GEMM into the same function."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, chunks, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import oracle
    from tensorpencil_b200 import nsplit, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 24, 128, 512
        c = synth.convrot_linear(m, n, k, 8, seed=77)           # same data on every rank
        q, s = oracle.convrot_prep(c["x"], 8)                  # prep is replicated
        full = (oracle.igemm_s32(q, c["w_i8"]).astype(np.float32) * s[:, None]) * c["w_scale"][None, :]

        def compute_shard(lo, hi):
            acc = oracle.igemm_s32(q, c["w_i8"][lo:hi])        # this rank only touches its weight rows
            return torch.from_numpy((acc.astype(np.float32) * s[:, None]) * c["w_scale"][None, lo:hi])

        lo, hi = nsplit.shard_bounds(n, world, rank, 16 * chunks)
        assert (lo, hi) == (rank * n // world, (rank + 1) * n // world)
        g = nsplit.nsplit_gemm_allgather(compute_shard, m, n, chunks=chunks)
        y = nsplit.assemble(g).numpy()
        ok = np.array_equal(y.view(np.uint32), full.view(np.uint32))
        # column-blocked layout: g[chunk][rank] is that rank's piece
        piece = n // world // chunks
        ok = ok and np.array_equal(g[0, 1].numpy(), full[:, n // world:n // world + piece])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 2])
def test_nsplit_allgather_bit_identical_to_single(chunks):
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, chunks, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_bounds_rejects_uneven_splits():
    from tensorpencil_b200 import nsplit
    with pytest.raises(ValueError):
        nsplit.shard_bounds(100, 3, 0)
    with pytest.raises(ValueError):
        nsplit.shard_bounds(96, 4, 0, multiple=16)   # 24 per rank is not a multiple of 16
    assert nsplit.shard_bounds(12288, 8, 3) == (4608, 6144)
