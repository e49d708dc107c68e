"""Row sharding of one logical tensor across the GPUs of a box.

Every operation of this backend is row independent, so a [R, F] tensor is cut
into per-rank row ranges on 16-row band boundaries: each shard is then a
self-contained tiled tensor (no tile is shared between ranks) and needs no
communication; broadcast operands (scale, bias) are replicated. The one
exchange is the whole-tensor sum of squares: every rank contributes one FP32
partial, the partials are all-gathered and added in rank order on every rank,
so the result does not depend on a collective's internal reduction order.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np

BAND = 16


def shard_rows(rows: int, world: int, rank: int) -> tuple[int, int]:
    """(first_row, row_count) of `rank`: whole 16-row bands, as even as possible.

    The last band may be partial; ranks beyond the number of bands get no rows.
    """
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world)")
    if rows <= 0:
        raise ValueError("rows must be positive")
    bands = (rows + BAND - 1) // BAND
    base, extra = divmod(bands, world)
    first_band = rank * base + min(rank, extra)
    count_bands = base + (1 if rank < extra else 0)
    first = first_band * BAND
    last = min(rows, (first_band + count_bands) * BAND)
    return first, max(0, last - first)


def combine_partials(partials: Sequence[float]) -> np.float32:
    """Adds per-rank FP32 partial sums in rank order, each step rounded to FP32."""
    total = np.float32(0.0)
    for value in partials:
        total = np.float32(total + np.float32(value))
    return total


def all_gather_sum(local, group=None):
    """All-gathers one FP32 partial per rank and folds them in rank order.

    `local` is a one-element float32 torch tensor on the device the process
    group communicates from (CUDA for NCCL, CPU for gloo). Returns a 0-dim
    float32 tensor, bit-identical on every rank.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    gathered = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(gathered, local, group=group)
    total = torch.zeros((), dtype=torch.float32, device=local.device)
    for part in gathered:
        total = total + part.reshape(())
    return total
