"""One ConvRot GEMM split along N across ranks, output shards exchanged with an
all-gather (NCCL over NVLink on GPUs, gloo in the CPU tests).

The reference is single-GPU (src/gpu/cuda/context.zig:111), so this has no
reference behaviour to match beyond "the same numbers as one GPU".  It is the
one place in the quantized-linear path with a real exchange step:

    rank r holds W[r*N/g : (r+1)*N/g, :] and the matching w_scale slice;
    every rank holds the full quantised activations (prep is replicated: it is
    cheap and keeps the GEMM inputs local);
    each rank computes y[:, shard] = (acc * act_scale[:, None]) * w_scale[shard];
    the shards are gathered.

Splitting along N never changes an output element: its int32 accumulator sums
over all of K on one rank and the epilogue is elementwise, so the gathered result
is bit-identical to the single-GPU one.  (A K split would need a reduction and
would change the float rounding order; it is not offered.)

Layout.  Row-major [M][N/g] shards do not concatenate into row-major [M][N], so
the gathered tensor is column-blocked: ``out[r]`` is rank r's [M][N/g] block, i.e.
``y[:, r*N/g:(r+1)*N/g] == out[r]``.  ``assemble`` returns the row-major view for
callers that need it (one extra pass over the output).

No kernel here reads another GPU's memory: the collective deposits remote shards
in local memory before anything touches them.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """Columns [lo, hi) of rank `rank`: equal shards, N/world a multiple of `multiple`
    (the GEMM needs n % 16 == 0 per shard)."""
    if n % world != 0 or (n // world) % multiple != 0:
        raise ValueError(f"N={n} does not split into {world} shards that are multiples of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def nsplit_gemm_allgather(compute_shard: Callable[[int, int], torch.Tensor], m: int, n: int,
                          group: Optional[dist.ProcessGroup] = None, chunks: int = 1,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Runs ``compute_shard(lo, hi) -> [m][hi-lo]`` for this rank's columns and
    all-gathers the shards into ``out[world][m][n/world]``.

    ``chunks`` > 1 splits the shard's columns into that many pieces and starts each
    piece's all-gather (async) while the next piece is being computed, so the
    transfer overlaps the GEMM.  With chunks the gathered layout is
    ``out[world][chunks][m][n/world/chunks]`` flattened into the same buffer; use
    ``assemble`` to get row-major [m][n]."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = shard_bounds(n, world, rank, 16 * chunks)
    per = hi - lo
    piece = per // chunks
    handles = []
    result = None
    for c in range(chunks):
        y_piece = compute_shard(lo + c * piece, lo + (c + 1) * piece)
        if y_piece.shape != (m, piece):
            raise ValueError(f"compute_shard returned {tuple(y_piece.shape)}, expected {(m, piece)}")
        y_piece = y_piece.contiguous()
        if result is None:
            result = out if out is not None else torch.empty((chunks, world, m, piece), dtype=y_piece.dtype,
                                                             device=y_piece.device)
            result = result.view(chunks, world, m, piece)
        # output as the flat concatenation [world*m][piece]: accepted by both nccl and gloo
        handles.append(dist.all_gather_into_tensor(result[c].view(world * m, piece), y_piece, group=group,
                                                   async_op=True))
    for h in handles:
        h.wait()
    return result


def assemble(gathered: torch.Tensor) -> torch.Tensor:
    """[chunks][world][m][piece] -> row-major [m][world*chunks*piece] with columns in
    their original order (rank-major, then chunk, then column)."""
    chunks, world, m, piece = gathered.shape
    return gathered.permute(2, 1, 0, 3).reshape(m, world * chunks * piece)
