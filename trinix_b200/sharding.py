"""Batch sharding for the data-parallel forward: independent units, no collective.

Every op on the path is independent across rows / sequences, so rank r of W simply owns a
contiguous slice of the leading (batch or row) dimension. The only communication a sharded run
needs is outside the data path: the maximum over ranks of a measured time, and an untimed
gather that checks "the shards side by side equal the unsharded result, bit for bit".
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple, Union

import torch


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


def max_over_ranks(values: Union[float, Sequence[float]], device="cpu"):
    """Element-wise maximum over all ranks of one or several numbers (e.g. measured times): the
    figure a data-parallel job is judged by. Without an initialised process group the values
    come back unchanged."""
    import torch.distributed as dist
    single = not isinstance(values, (list, tuple))
    t = torch.tensor([values] if single else list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = [float(v) for v in t.tolist()]
    return out[0] if single else out


def gather_shards(local: torch.Tensor, n: int, world: int) -> torch.Tensor:
    """All ranks' dim-0 shards of an n-unit result, concatenated in rank order on every rank
    (ragged shards are padded to the largest for the exchange and trimmed afterwards)."""
    import torch.distributed as dist
    if world == 1:
        return local
    sizes = [hi - lo for lo, hi in (shard_bounds(n, r, world) for r in range(world))]
    big = max(sizes)
    pad = torch.zeros((big,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]].copy_(local)
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], dim=0)


def cross_rank_identical(fn: Callable, full_inputs: Sequence[torch.Tensor], rank: int,
                         world: int) -> bool:
    """Does the batch-sharded run reproduce the unsharded one bit for bit?

    Every rank holds the same `full_inputs` (commonly seeded); tensors among them whose leading
    dim equals the batch size n = full_inputs[0].shape[0] are sharded, the rest (weights, tables)
    are replicated. Rank r applies `fn` to its shard; the outputs (a tensor or a tuple of tensors
    with leading dim = shard size) are gathered — the one communication, outside any timed
    region — and compared with `fn(*full_inputs)`. The verdict of all ranks is AND-ed."""
    import torch.distributed as dist
    n = full_inputs[0].shape[0]
    mine = [shard(t, rank, world) if (t.dim() > 0 and t.shape[0] == n) else t
            for t in full_inputs]
    outs = fn(*mine)
    outs = outs if isinstance(outs, (tuple, list)) else (outs,)
    gathered = [gather_shards(o.contiguous(), n, world) for o in outs]
    want = fn(*full_inputs)
    want = want if isinstance(want, (tuple, list)) else (want,)
    ok = all(g.shape == w.shape and torch.equal(g, w) for g, w in zip(gathered, want))
    flag = torch.tensor([1 if ok else 0], device=gathered[0].device)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(int(flag.item()))
