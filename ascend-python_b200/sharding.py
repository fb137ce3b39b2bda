"""Host-side helpers for the row-parallel (K-sharded) matmul + allreduce.

Rank r of a world of W holds the K slice ``[bounds[r], bounds[r+1])`` of the
activations' columns and of the weight's rows; partial products are summed by
allreduce.  Shards are as even as possible and, when K allows, aligned to 128
so that every shard keeps the 16-byte row pitch the TMA path needs.
"""
from __future__ import annotations

from typing import List, Tuple


def k_shard_bounds(K: int, world_size: int, align: int = 128) -> List[int]:
    """Boundaries b[0]=0 <= ... <= b[W]=K of the K shards."""
    if world_size < 1:
        raise ValueError(f"world_size should be greater than 0, but the actual value is {world_size}")
    if K < 0:
        raise ValueError("K must be non-negative")
    if K % (world_size * align) == 0:
        step = K // world_size
        return [r * step for r in range(world_size + 1)]
    units = K // align
    if units >= world_size:
        base, extra = divmod(units, world_size)
        bounds, pos = [0], 0
        for r in range(world_size):
            pos += (base + (1 if r < extra else 0)) * align
            bounds.append(pos)
        bounds[-1] = K  # the remainder below one alignment unit goes to the last rank
        return bounds
    base, extra = divmod(K, world_size)
    bounds, pos = [0], 0
    for r in range(world_size):
        pos += base + (1 if r < extra else 0)
        bounds.append(pos)
    return bounds


def shard_row_parallel(x, w, world_size: int, rank: int, align: int = 128) -> Tuple:
    """(x[:, k0:k1], w[k0:k1, :]) of `rank`; x is [M,K], w is [K,N]."""
    b = k_shard_bounds(x.shape[-1], world_size, align)
    k0, k1 = b[rank], b[rank + 1]
    return x[..., k0:k1], w[k0:k1, :]
