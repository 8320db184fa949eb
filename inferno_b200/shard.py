"""Partition of the flattened batch*head axis over ranks.

Attention is independent per (batch, head): outputs and gradients of one head depend only on
that head's Q, K, V and dO.  Multi-GPU runs therefore give each rank a contiguous range of the
B*H heads -- a contiguous slab of every dense [B,H,T,D] tensor -- and need no collective inside
the attention path.  (The reference is single-process and single-GPU; it has no counterpart.)
"""
from __future__ import annotations


def shard_range(total_heads: int, rank: int, world_size: int) -> range:
    """Contiguous range of heads owned by ``rank``; sizes differ by at most one."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world_size")
    base, extra = divmod(total_heads, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_sizes(total_heads: int, world_size: int):
    return [len(shard_range(total_heads, r, world_size)) for r in range(world_size)]
