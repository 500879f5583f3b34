"""Sharding of the path across GPUs: contiguous ranges of (batch x head) slices.

Every kernel of the path works on one (batch, head) slice at a time and no
result of one slice feeds another (dK/dV are summed over q-blocks of the same
slice only), so ranks need no collective on the data path: each rank runs the
three API calls on its own slices.  These helpers only compute who owns what.
"""

from __future__ import annotations

from typing import Tuple

import torch


def slice_range(num_slices: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the flattened (batch*head) slices owned by `rank`;
    ranges are contiguous, disjoint, cover everything and differ in size by at
    most one."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(num_slices, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_heads(x: torch.Tensor, num_heads: int, rank: int, world: int):
    """View of x [B, N, H*D] holding this rank's heads, plus the head count.

    Heads must divide evenly.  The view is strided (no copy): the kernels
    address [b][n][h][d] through explicit strides."""
    if num_heads % world != 0:
        raise ValueError(f"num_heads ({num_heads}) must be divisible by the world size ({world})")
    C = x.shape[-1]
    D = C // num_heads
    per = num_heads // world
    return x[:, :, rank * per * D:(rank + 1) * per * D], per
