"""Partition of the (batch x head) space across GPUs.

The attention kernels' unit of work is one (batch, head) pair (the reference's grid unit,
quant_flash_attn.py:187) and the quantizer's is one token row (asymmetric_quant.py:132); units are
independent, so multi-GPU runs give every rank a contiguous, equal slice of the flattened B*H
axis and need no collective on the data path.
"""
from __future__ import annotations


def shard_bounds(n_units: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous [start, end) of `n_units` for `rank`; the first n_units % world_size ranks get
    one extra unit.  Every unit belongs to exactly one rank."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(n_units, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def head_slice(t, world_size: int, rank: int):
    """View of a (B,H,S,D) tensor as (n_local_heads, 1... ) is layout dependent, so this returns
    the rank's slice of the tensor flattened over (B*H): shape (1, n_local, S, D)."""
    B, H = t.shape[0], t.shape[1]
    s, e = shard_bounds(B * H, world_size, rank)
    return t.reshape(1, B * H, *t.shape[2:])[:, s:e]
