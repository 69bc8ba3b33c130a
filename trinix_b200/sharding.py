"""Batch sharding for the data-parallel forward: independent units, no collective.

Every op on the path is independent across rows / sequences, so rank r of W simply owns a
contiguous slice of the leading (batch or row) dimension.
"""
from __future__ import annotations

from typing import Tuple


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of the n units owned by `rank`; sizes differ by at most one, earlier ranks
    take the remainder. Raises on an invalid rank."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} for world size {world}")
    if n < 0:
        raise ValueError("n must be >= 0")
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard(t, rank: int, world: int, dim: int = 0):
    """Slice of tensor `t` along `dim` owned by `rank`."""
    lo, hi = shard_bounds(t.shape[dim], rank, world)
    return t.narrow(dim, lo, hi - lo)
