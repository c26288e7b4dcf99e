"""Slot sharding across the GPUs of one box.

Every ``(slot, head)`` tile of a decode step is independent, and the steps of
one slot are sequential, so the state pool is partitioned **by slot**: rank
``r`` of ``G`` owns a contiguous block of every layer's pool and the matching
rows of the activations.  Nothing crosses ranks on the data path; a process
group is only used to agree on timings (max over ranks) and to gather outputs
for reporting.
"""

from __future__ import annotations

from typing import Tuple

import torch


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """``[lo, hi)`` of ``n`` items owned by ``rank``: contiguous, disjoint,
    covering, sizes differing by at most one (the first ``n % world`` ranks get
    the extra item)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_requests(state_indices: torch.Tensor, num_slots: int, world: int, rank: int):
    """Split a global batch of slot ids over ranks by slot ownership.

    Slot 0 is the padding id and belongs to nobody; real slots ``1..num_slots-1``
    are block-partitioned.  Returns ``(rows, local_ids)``: the positions in the
    global batch that this rank serves, and their slot ids re-based into this
    rank's local pool (local id 0 stays the padding slot).  Padding requests
    (id <= 0) are served by rank 0 so that every output row is written once."""
    ids = state_indices.to(torch.int64)
    lo, hi = shard_range(num_slots - 1, world, rank)
    lo, hi = lo + 1, hi + 1
    mine = (ids >= lo) & (ids < hi)
    if rank == 0:
        mine = mine | (ids <= 0)
    rows = torch.nonzero(mine, as_tuple=False).flatten()
    local = ids[rows]
    local = torch.where(local > 0, local - lo + 1, torch.zeros_like(local))
    return rows, local.to(torch.int32)


def local_pool_slots(num_slots: int, world: int, rank: int) -> int:
    """Slots a rank must allocate: its share of the real slots plus padding slot 0."""
    lo, hi = shard_range(num_slots - 1, world, rank)
    return hi - lo + 1


def max_over_ranks(seconds: float, device=None) -> float:
    """Slowest rank's elapsed time (identity without a process group)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return seconds
    t = torch.tensor([seconds], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_rows(local_rows: torch.Tensor, local_out: torch.Tensor, total_rows: int):
    """Reassemble per-rank output rows into the global batch order on every
    rank (reporting only; not on the data path)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        out = local_out.new_zeros((total_rows,) + tuple(local_out.shape[1:]))
        out[local_rows] = local_out
        return out
    world = dist.get_world_size()
    rows_list = [None] * world
    outs_list = [None] * world
    dist.all_gather_object(rows_list, local_rows.cpu())
    dist.all_gather_object(outs_list, local_out.cpu())
    out = outs_list[0].new_zeros((total_rows,) + tuple(local_out.shape[1:]))
    for r, o in zip(rows_list, outs_list):
        out[r] = o
    return out
