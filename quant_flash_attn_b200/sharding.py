"""Partition of the (batch x head) space across GPUs.

The attention kernels' unit of work is one (batch, head) pair (the reference's grid unit,
quant_flash_attn.py:187) and the quantizer's is one token row (asymmetric_quant.py:132); units are
independent, so multi-GPU runs give every rank a contiguous, equal slice of the flattened B*H
axis and need no collective on the data path.  `all_gather_heads` is the one step AFTER the path that
needs the interconnect: when the heads of all ranks belong to one model layer, the layer's next
operator wants the whole (B,H,S,D) output on every rank.
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


def all_gather_heads(local, batch: int, heads: int, group=None):
    """Inverse of `head_slice` across a process group: every rank passes its (1, n_local, S, D) slice
    (n_local from `shard_bounds`) and receives the full (batch, heads, S, D) tensor.

    One `all_gather` over the group's backend (NCCL rides NVLink / NVSwitch between the GPUs of a node;
    gloo on CPU).  Slices may differ by one head between ranks, so the shorter ones are padded to the
    longest for the collective and trimmed afterwards.  Not part of the attention path: heads never
    exchange data while they are computed."""
    import torch
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = batch * heads
    spans = [shard_bounds(n, world, r) for r in range(world)]
    s, e = spans[rank]
    if local.shape[0] != 1 or local.shape[1] != e - s:
        raise ValueError(f"rank {rank} holds heads [{s}, {e}) but passed a tensor of shape {tuple(local.shape)}")
    longest = max(b - a for a, b in spans)
    send = local.contiguous()
    if e - s < longest:
        pad = torch.zeros((1, longest - (e - s), *local.shape[2:]), dtype=local.dtype, device=local.device)
        send = torch.cat([send, pad], dim=1)
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send, group=group)
    full = torch.cat([recv[r][:, : spans[r][1] - spans[r][0]] for r in range(world)], dim=1)
    return full.reshape(batch, heads, *local.shape[2:])

