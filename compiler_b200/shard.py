"""Partition of work over GPUs (and of rows over chunks).

The reference partitions program instances over 1/2/4/8 workers with a strided range and
proves exactly-once coverage (``strided_range`` / ``check_partition``,
a100c/plan/partition.py:26-59).  Across GPUs a contiguous block per rank is the better
shape -- one slab of HBM per device, no interleaving -- so ``block_range`` hands rank r the
r-th of ``world`` nearly equal contiguous blocks; ``check_partition`` keeps the reference's
guarantee: every item is owned by exactly one rank.
"""
from __future__ import annotations


def block_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) of rank's contiguous block; the first ``total % world`` ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if total < 0:
        raise ValueError("negative extent")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def column_range(total: int, rank: int, world: int, multiple: int = 8) -> tuple[int, int]:
    """Like ``block_range`` but every boundary is a multiple of ``multiple`` columns, so each
    shard's rows stay 16-byte aligned for TMA (8 x 2-byte elements)."""
    if total % multiple:
        raise ValueError(f"{total} columns are not a multiple of {multiple}")
    lo, hi = block_range(total // multiple, rank, world)
    return lo * multiple, hi * multiple


def strided_items(total: int, rank: int, world: int) -> range:
    """The reference's own policy: items rank, rank + world, ... (partition.py:26-34)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    return range(rank, total, world)


def row_chunks(rows: int, chunks: int) -> list[tuple[int, int]]:
    """Non-empty contiguous [lo, hi) chunks covering ``rows``."""
    chunks = max(1, min(chunks, rows)) if rows > 0 else 1
    return [r for r in (block_range(rows, c, chunks) for c in range(chunks)) if r[1] > r[0]]


def check_partition(total: int, world: int, policy=block_range) -> None:
    """Raise unless the ranks' shares cover 0..total-1 exactly once (partition.py:42-59)."""
    seen = [0] * total
    for rank in range(world):
        share = policy(total, rank, world)
        items = share if isinstance(share, range) else range(*share)
        for i in items:
            if not 0 <= i < total:
                raise AssertionError(f"rank {rank} owns out-of-range item {i}")
            seen[i] += 1
    bad = [i for i, n in enumerate(seen) if n != 1]
    if bad:
        raise AssertionError(f"items not owned exactly once: {bad[:8]}")


def shard_rows_offset(rows_per_rank: int, rank: int) -> int:
    """Global index of a rank's first row when every rank holds ``rows_per_rank`` rows of an
    N-times-larger job (the ``row_offset`` the masked softmax needs)."""
    return rows_per_rank * rank
