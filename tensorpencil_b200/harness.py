"""Drivers that replay the reference's call sequences over the quantized-linear
ops: one DiT step's block stack (resident or weight-streamed, one latent or a batch
of independent latents), and helpers for the decode GEMV benchmark.  Used by
``bench.py`` and the tests.

The DiT driver follows ``dit_cuda.forward`` (src/models/dit_cuda.zig:464-517): per
block one prep feeds wq/wk/wv/gate, one prep feeds wo, and the MLP runs in row
tiles (``mlp_tile``, :36-39): prep -> gate, up -> (SiLU * up) -> prep -> down.
Everything between the linears runs through this library too: RMS norm +
modulation, the sigmoid and SiLU gates and the gated residuals as the reference's
stand-alone ops (mode "unfused") or folded into the prep kernels and GEMM
epilogues (mode "fused"); qk-norm, RoPE and softmax attention when ``attn`` is
given.  Without ``attn`` the value projection stands in for the attention output,
which leaves every row independent (what the full-size parity tests rely on).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from . import synth
from .offload import Streamer, packed_size, slot_size

MLP_TILE = 2048  # src/models/dit_cuda.zig:39


class DitWeights:
    """Random-init quantised weights of the synthetic DiT, on the device
    (resident) or as per-block pinned host images behind a Streamer."""

    def __init__(self, be, bits: int, blocks: int = synth.DIT_BLOCKS, hidden: int = synth.DIT_HIDDEN,
                 mlp: int = synth.DIT_MLP, seed: int = 1003, stream_budget: Optional[int] = None,
                 distinct_blocks: Optional[int] = None, stream_group=None):
        self.be, self.bits, self.blocks, self.hidden, self.mlp = be, bits, blocks, hidden, mlp
        self.names = [n for n, _, _ in synth.DIT_LINEARS]
        # Generating 28 distinct blocks of random weights on the host takes a while and
        # says nothing more about speed than a few: blocks cycle through `distinct` sets.
        distinct = blocks if distinct_blocks is None else min(blocks, distinct_blocks)
        host = [self._random_block(b, seed) for b in range(distinct)]
        self.shapes = {n: (host[0][n]["n"], host[0][n]["k"]) for n in self.names}
        self.streamer: Optional[Streamer] = None
        if stream_budget is None:
            self.dev: List[Dict[str, tuple]] = []
            for b in range(blocks):
                hb = host[b % distinct]
                # every block owns its own device copy, so a step reads 28 blocks' worth of weights
                self.dev.append({n: (hb[n]["w"].clone() if b >= distinct else hb[n]["w"],
                                     hb[n]["w_scale"]) for n in self.names})
        else:
            host = [{n: {"w": hb[n]["w"].cpu().numpy(), "w_scale": hb[n]["w_scale"].cpu().numpy()} for n in self.names}
                    for hb in host]
            arrays0 = [a for n in self.names for a in (host[0][n]["w"], host[0][n]["w_scale"])]
            world = 1
            if stream_group is not None:
                import torch.distributed as dist
                world = dist.get_world_size(stream_group)
            slot = slot_size(packed_size(arrays0), world)
            n_slots = max(2, min(4, stream_budget // slot))
            if n_slots * slot > stream_budget:
                raise ValueError(f"budget {stream_budget} cannot hold two blocks of {slot} bytes")
            # stream_group: the ranks of a node that hold these same weights share the host link
            self.streamer = Streamer(be, stream_budget, slot, n_slots, group=stream_group)
            for b in range(blocks):
                hb = host[b % distinct]
                self.streamer.register(b, [a for n in self.names for a in (hb[n]["w"], hb[n]["w_scale"])])
            self.block_bytes = slot

    def _random_block(self, b: int, seed: int) -> Dict[str, dict]:
        """Random-init weights of one block, drawn on the device (same value ranges as
        synth.dit_block_weights: int8 in [-127,127] or packed int4 nibbles, scales
        ~U(1e-3,1e-2))."""
        out = {}
        g = torch.Generator(device=self.be.device).manual_seed(seed + 1000 * b)
        for name, n, k in synth.DIT_LINEARS:
            n = self.mlp if n == synth.DIT_MLP else self.hidden
            k = self.mlp if k == synth.DIT_MLP else self.hidden
            if self.bits == 8:
                wt = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=self.be.device, generator=g)
            else:
                wt = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=self.be.device, generator=g)
            ws = torch.rand(n, device=self.be.device, generator=g) * 9e-3 + 1e-3
            out[name] = {"w": wt, "w_scale": ws, "n": n, "k": k}
        return out

    def close(self):
        if self.streamer is not None:
            self.streamer.close()


def dit_modulation(be, blocks: int, hidden: int, seed: int = 7) -> torch.Tensor:
    """The per-block AdaLN vectors the step reads: for block b, six rows of `hidden` at
    offset b*6*hidden -- pre-attention premul and shift, attention gate, pre-MLP premul and
    shift, MLP gate (src/models/dit_cuda.zig:471-516).  premul = 1 + small, the rest small."""
    g = torch.Generator(device=be.device).manual_seed(seed)
    mod = (torch.rand(blocks * 6 * hidden, device=be.device, generator=g) - 0.5) * 0.2
    mod = mod.view(blocks, 6, hidden)
    mod[:, 0] += 1.0
    mod[:, 3] += 1.0
    return mod.reshape(-1).contiguous()


def dit_step_linears(be, w: DitWeights, x: torch.Tensor, out_dtype=torch.float32,
                     mlp_tile: int = MLP_TILE, mode: str = "linears",
                     mod: Optional[torch.Tensor] = None, eps: float = 1e-5,
                     attn: Optional[dict] = None, latents: int = 1, mlp_pair: bool = False,
                     qkvg_group: bool = False) -> torch.Tensor:
    """One step of the block stack on x [latents * tokens][hidden] (f32, updated in place).

    mode:
      "linears"  prep + GEMM only; the linears read whatever their input buffers hold
                 (the time of the quantized-linear kernels alone);
      "unfused"  the reference's sequence: rmsMod, prep, GEMMs, sigmoidMul, prep, GEMM,
                 gatedAdd, and per MLP tile rmsMod, prep, GEMMs, siluMul, prep, GEMM,
                 gatedAdd -- every elementwise op its own kernel (f32 only);
      "fused"    the same data flow with rmsMod / sigmoidMul / siluMul folded into the
                 prep kernels and gatedAdd folded into the wo / mlp.down GEMM epilogues;
                 with out_dtype=bf16 the q/k/v/gate and MLP gate/up outputs stay bf16.
    attn: None -> v stands in for the attention output (the linears and their elementwise
    neighbours alone); a dict {q_norm, k_norm, cos, sin, heads} -> qk-norm + RoPE + softmax
    attention run between the projections and the sigmoid gate (dit_cuda.zig:479-489),
    modes "unfused" and "fused".

    latents: x stacks this many independent latents of equal token count along the rows.
    Every op but attention is row-wise, so a block's linears run ONCE over all rows -- with
    streamed weights each block's image crosses PCIe once per step for the whole batch
    (the block is acquired, used by every latent, then released); attention runs per latent.

    mlp_tile: rows per MLP tile.  The reference tiles by 2048 rows to fit a 24 GB card;
    with 180 GB of HBM the whole batch can go through at once.

    mlp_pair (mode "fused"): the MLP's gate and up projections run as one launch whose epilogue
    applies the SiLU gate (Backend.gemmSiluPair), followed by a plain prep, instead of two GEMMs and
    the SiLU-gated prep.  qkvg_group: the q, k, v and gate projections of a block in one launch
    (Backend.gemmGroup) instead of four."""
    bits, hid, mlp = w.bits, w.hidden, w.mlp
    prep = be.opI8Prep if bits == 8 else be.opI4Prep
    gemm = (lambda y, wt, n: be.opI8Gemm(y, wt[0], wt[1], n)) if bits == 8 else \
           (lambda y, wt, n: be.opI4Gemm(y, wt[0], wt[1], n))
    m = x.shape[0]
    dev = be.device
    if mode not in ("linears", "unfused", "fused"):
        raise ValueError(f"unknown mode {mode!r}")
    if mode == "unfused" and out_dtype != torch.float32:
        raise ValueError("the unfused sequence is f32 only")
    if mode in ("unfused", "fused") and mod is None:
        raise ValueError("mode needs the modulation vectors (dit_modulation)")
    if latents < 1 or m % latents:
        raise ValueError("x must stack `latents` latents of equal token count")
    tokens = m // latents
    mlp_tile = min(mlp_tile, m)
    q = torch.empty((m, hid), dtype=out_dtype, device=dev)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    g = torch.empty_like(q)
    o = torch.empty_like(q)
    t1 = torch.empty((m, hid), dtype=torch.float32, device=dev) if mode == "unfused" else None
    tile_gate = torch.empty((mlp_tile, mlp), dtype=out_dtype, device=dev)
    tile_up = torch.empty_like(tile_gate)
    tile_down = torch.empty((mlp_tile, hid), dtype=out_dtype, device=dev) if mode != "fused" else None
    attn_buf = torch.zeros((m, hid), dtype=torch.float32, device=dev) if mode == "linears" else None
    act_buf = torch.zeros((mlp_tile, mlp), dtype=torch.float32, device=dev) if mode == "linears" else None
    st = w.streamer
    if st is not None:
        st.prefetch(0)
    for b in range(w.blocks):
        if st is not None:
            views = st.acquire(b)
            wb = {n: (views[2 * i], views[2 * i + 1]) for i, n in enumerate(w.names)}
            if b + 1 < w.blocks:
                st.prefetch(b + 1)          # prefetchBlock(b+1), dit_cuda.zig:470
        else:
            wb = w.dev[b]
        mb = b * 6 * hid
        # --- attention: one prep, four GEMMs (dit_cuda.zig:473-478) ---
        if mode == "fused":
            be.prepRmsMod(x, mod, m, hid, mb, mb + hid, eps, bits)
        elif mode == "unfused":
            be.rmsMod(x, t1, mod, m, hid, mb, mb + hid, eps)
            prep(t1, m, hid)
        else:
            prep(x, m, hid)
        if qkvg_group:
            # the four projections of one prep in one launch (bit-identical to the four calls)
            be.gemmGroup([q, k, v, g], [wb[n][0] for n in ("wq", "wk", "wv", "gate")],
                         [wb[n][1] for n in ("wq", "wk", "wv", "gate")], hid, bits)
        else:
            gemm(q, wb["wq"], hid)
            gemm(k, wb["wk"], hid)
            gemm(v, wb["wv"], hid)
            gemm(g, wb["gate"], hid)
        a = v                                              # without attn: v stands in for its output
        if attn is not None and mode != "linears":
            for l in range(latents):
                r = slice(l * tokens, (l + 1) * tokens)
                be.attention(q[r], k[r], v[r], attn["q_norm"], attn["k_norm"], attn["cos"], attn["sin"],
                             attn["heads"], attn["heads"], out_dtype=out_dtype, out=o[r])
            a = o
        if mode == "fused":
            be.prepSigmoidMul(a, g, m, hid, bits)
        elif mode == "unfused":
            be.sigmoidMul(a, g, m * hid)
            prep(a, m, hid)
        else:
            prep(attn_buf, m, hid)
        if mode == "fused":
            be.gemmGatedAdd(x, wb["wo"][0], wb["wo"][1], hid, mod, mb + 2 * hid, bits)   # GEMM + gated residual
        else:
            gemm(o, wb["wo"], hid)
        if mode == "unfused":
            be.gatedAdd(x, o, mod, m * hid, hid, mb + 2 * hid)
        # --- MLP in row tiles (dit_cuda.zig:495-516) ---
        for t0 in range(0, m, mlp_tile):
            rows = min(mlp_tile, m - t0)
            xt = x[t0:t0 + rows]
            if mode == "fused":
                be.prepRmsMod(xt, mod, rows, hid, mb + 3 * hid, mb + 4 * hid, eps, bits)
            elif mode == "unfused":
                be.rmsMod(xt, t1, mod, rows, hid, mb + 3 * hid, mb + 4 * hid, eps)
                prep(t1, rows, hid)
            else:
                prep(xt, rows, hid)
            if mode == "fused" and mlp_pair:
                # gate and up projections with the SiLU gate in the GEMM's epilogue, then a plain prep
                be.gemmSiluPair(tile_gate[:rows], wb["mlp_gate"][0], wb["mlp_gate"][1], wb["mlp_up"][0], wb["mlp_up"][1],
                                mlp, bits)
                prep(tile_gate[:rows], rows, mlp)
            else:
                gemm(tile_gate, wb["mlp_gate"], mlp)
                gemm(tile_up, wb["mlp_up"], mlp)
            if mode == "fused" and mlp_pair:
                pass
            elif mode == "fused":
                be.prepSiluMul(tile_gate, tile_up, rows, mlp, bits)
            elif mode == "unfused":
                be.siluMul(tile_gate, tile_up, rows * mlp)
                prep(tile_gate, rows, mlp)
            else:
                prep(act_buf, rows, mlp)
            if mode == "fused":
                be.gemmGatedAdd(xt, wb["mlp_down"][0], wb["mlp_down"][1], hid, mod, mb + 5 * hid, bits)
            else:
                gemm(tile_down, wb["mlp_down"], hid)
            if mode == "unfused":
                be.gatedAdd(xt, tile_down, mod, rows * hid, hid, mb + 5 * hid)
        if st is not None:
            st.release(b)
    return x


def attention_inputs(seq: int, heads: int, kv_heads: int, device, dtype=torch.bfloat16, seed: int = 5):
    """Synthetic q, k, v ([seq][heads*128]), unit-ish norm weights and the FLUX cos / sin tables
    ([seq][64], axes 32/48/48 over a 3-axis position id: src/ops/rope.zig:26-60) on the device."""
    g = torch.Generator(device=device).manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, device=device, generator=g)
    q, k, v = rnd(seq, heads * 128).to(dtype), rnd(seq, kv_heads * 128).to(dtype), rnd(seq, kv_heads * 128).to(dtype)
    qn, kn = 1.0 + 0.1 * rnd(128), 1.0 + 0.1 * rnd(128)
    idx = torch.arange(seq, device=device, dtype=torch.float32)
    pos = torch.stack([torch.zeros_like(idx), torch.div(idx, 64, rounding_mode="floor"), idx % 64], dim=1)
    ang = []
    for a, d in enumerate((32, 48, 48)):
        freq = 10000.0 ** (-torch.arange(0, d, 2, device=device, dtype=torch.float32) / d)
        ang.append(pos[:, a:a + 1] * freq[None, :])
    ang = torch.cat(ang, dim=1)                            # [seq][64]
    return q, k, v, qn.contiguous(), kn.contiguous(), torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


def dit_linear_ops(tokens: int, blocks: int, hidden: int, mlp: int) -> float:
    """2*M*N*K summed over the eight linears of every block."""
    per_block = 5 * 2.0 * tokens * hidden * hidden + 3 * 2.0 * tokens * mlp * hidden
    return per_block * blocks


def rotating_q8_weights(n: int, k: int, copies: int, device) -> List[torch.Tensor]:
    """`copies` distinct Q8_0 weight buffers with sane f16 scales, generated on the
    device (the GEMV benchmark cycles through them so every launch streams from HBM)."""
    nb = k // 32
    out = []
    for i in range(copies):
        g = torch.Generator(device=device).manual_seed(1002 + i)
        w = torch.randint(0, 256, (n, nb, 34), dtype=torch.uint8, device=device, generator=g)
        w[:, :, 0] = 0x66
        w[:, :, 1] = 0x1e  # f16 0x1e66 ~ 6.2e-3
        out.append(w.reshape(n, nb * 34))
    return out
