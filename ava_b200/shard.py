"""Sharding of independent sequences over ranks (one process per GPU).

Every row of a state is independent of the others (reference: design-tests/nn/gpu/src/state.rs:13-15; `select` and
`cat` are row operations), and the weights are read-only, so the step needs no data-path collective: rank r holds a
contiguous block of the sequences with its own copy of the weights.  The only communication is for measurement (a
barrier and a max over ranks of the device time) and for gathering outputs on the host when a caller wants them.
"""
from __future__ import annotations


def block(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """[first, last) of the rows rank `rank` owns: contiguous blocks, sizes differing by at most one."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(total_rows, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def owner(total_rows: int, world: int, row: int) -> int:
    """The rank that owns `row`."""
    for r in range(world):
        a, b = block(total_rows, world, r)
        if a <= row < b:
            return r
    raise ValueError("row out of range")


def max_over_ranks(value: float, dist=None, device=None) -> float:
    """The slowest rank's time: what a multi-GPU throughput is computed from."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def kv_owner(position: int, block: int, world: int) -> int:
    """The rank that keeps token `position` of one long sequence whose engram store is split by position: contiguous
    blocks of `block` positions, the tail (the decoded tokens) on the last rank."""
    return min(position // block, world - 1)
