"""Two-GPU checks (skipped on a single-GPU box): replicas give the same answer on
every device, the N-split GEMM is bit-identical to one GPU both with the NCCL
all-gather and with the all-gather fused into the GEMM epilogue (peer stores), and a
streamed block stack whose ranks share the host link (every rank copies half of each
block, the halves are exchanged over NVLink) equals the resident run bit for bit."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    from tensorpencil_b200 import nsplit, synth
    from tensorpencil_b200.backend import Backend
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        be = Backend(rank)
        m, n, k = 512, 2048, 1024
        c = synth.convrot_linear(m, n, k, 8, seed=5)
        x = torch.from_numpy(c["x"]).cuda()
        w = torch.from_numpy(c["w_i8"]).cuda()
        ws = torch.from_numpy(c["w_scale"]).cuda()
        y_full = be.convrot_linear(x, w, ws, n, 8)               # replica: the whole linear on this GPU
        lo, hi = nsplit.shard_bounds(n, world, rank, 32)

        def compute(a, b):
            y = torch.empty((m, b - a), dtype=torch.float32, device="cuda")
            be.opI8Gemm(y, w[a:b], ws[a:b], b - a)               # prep state is still the one of convrot_linear
            return y

        g = nsplit.nsplit_gemm_allgather(compute, m, n, chunks=2)
        same_split = bool(torch.equal(nsplit.assemble(g), y_full))
        # replicas agree across devices
        ref = y_full.clone()
        dist.broadcast(ref, src=0)
        same_replica = bool(torch.equal(ref, y_full))
        # the same split with the exchange done by the GEMM's own epilogue over NVLink
        from tensorpencil_b200.peer import PeerBuffers
        pb = PeerBuffers(be, m * n * 4)
        same_fused = True
        for dt in (torch.float32, torch.bfloat16):
            y_one = torch.empty((m, n), dtype=dt, device="cuda")
            be.opI8Gemm(y_one, w, ws, n)
            pb.barrier()                       # nobody still reads the previous contents
            pb.gemm_allgather(w[lo:hi], ws[lo:hi], hi - lo, 8, y_dtype=dt)
            pb.barrier()                       # every rank's columns have landed everywhere
            same_fused = same_fused and bool(torch.equal(pb.tensor((m, n), dt), y_one))
        be.status_poll()
        pb.close()
        # and with one multicast store per element, where the platform has NVSwitch multicast
        from tensorpencil_b200.peer import MulticastBuffers
        mb = MulticastBuffers(be, m * n * 4)
        if mb.available:
            for dt in (torch.float32, torch.bfloat16):
                y_one = torch.empty((m, n), dtype=dt, device="cuda")
                be.opI8Gemm(y_one, w, ws, n)
                mb.barrier()
                mb.gemm_allgather(w[lo:hi], ws[lo:hi], hi - lo, 8, y_dtype=dt)
                mb.barrier()
                same_fused = same_fused and bool(torch.equal(mb.tensor((m, n), dt), y_one))
            be.status_poll()
        mb.close()
        ret[rank] = (same_split, same_replica, same_fused)
        be.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_replicas_and_nsplit():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}


def _stream_worker(rank, world, port, ret):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    from tensorpencil_b200 import harness, synth
    from tensorpencil_b200.backend import Backend
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        be = Backend(rank)
        blocks, hid, mlp, tokens = 5, 512, 1024, 300
        res = harness.DitWeights(be, 4, blocks=blocks, hidden=hid, mlp=mlp, seed=77)
        probe = harness.DitWeights(be, 4, blocks=1, hidden=hid, mlp=mlp, seed=77, stream_budget=1 << 28)
        slot = probe.block_bytes
        probe.close()
        # two slots (plus the rounding the pieces need) for five blocks: slots are reused within a step
        st = harness.DitWeights(be, 4, blocks=blocks, hidden=hid, mlp=mlp, seed=77, stream_budget=2 * slot + 4096,
                                stream_group=dist.group.WORLD)
        mod = harness.dit_modulation(be, blocks, hid, seed=6)
        x0 = synth.activations(tokens, hid, seed=50 + rank)      # the ranks work on different latents
        outs = []
        for w in (res, st, st):                                  # the second streamed step reuses slots
            x = torch.from_numpy(x0.copy()).cuda()
            outs.append(harness.dit_step_linears(be, w, x, mode="fused", mod=mod, mlp_tile=tokens).clone())
            be.status_poll()
        copied = st.streamer.bytes_copied()
        ret[rank] = (bool(torch.equal(outs[0], outs[1])), bool(torch.equal(outs[0], outs[2])),
                     # every rank pulled about half of the ten block images through its own link
                     0.4 * 2 * blocks * slot <= copied <= 0.6 * 2 * blocks * slot)
        st.close()
        res.close()
        be.close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_streaming_with_a_shared_host_link():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_stream_worker, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}
