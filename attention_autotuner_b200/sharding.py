"""(batch, head)-slice data parallelism over the GPUs of one node.

Every (b, h) slice of the three operators depends only on that slice's q, k, v (dO) and on the head's mask
or decay, so the slices are split into contiguous ranges, one per rank, and each rank runs the single-GPU
operator on its range. There is no collective on the data path. ``scatter_slices`` / ``gather_slices``
move inputs and outputs between rank 0 and the shards for validation only (NCCL on GPUs, gloo on CPU).
The reference has no multi-GPU code; this is the one decomposition the operators admit without a reduction.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def slice_range(rank: int, world: int, n_slices: int):
    """Contiguous range [lo, hi) of flattened slices s = b*H + h owned by ``rank``; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, rem = divmod(n_slices, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def heads_of(lo: int, hi: int, H: int):
    """Head index of every slice in [lo, hi) (for selecting the rows of a [H, ...] mask or decay)."""
    return torch.arange(lo, hi) % H


def flatten_bh(t: torch.Tensor) -> torch.Tensor:
    """[B, H, L, d] -> [B*H, L, d] view."""
    return t.reshape(t.shape[0] * t.shape[1], *t.shape[2:])


def scatter_slices(full: torch.Tensor | None, n_slices: int, tail_shape, dtype, device, src: int = 0):
    """Rank ``src`` holds ``full`` [n_slices, *tail]; every rank returns its [hi-lo, *tail] shard."""
    rank, world = dist.get_rank(), dist.get_world_size()
    lo, hi = slice_range(rank, world, n_slices)
    out = torch.empty((hi - lo, *tail_shape), dtype=dtype, device=device)
    if world == 1:
        out.copy_(full[lo:hi])
        return out
    if rank == src:
        for r in range(world):
            a, b = slice_range(r, world, n_slices)
            if r == src:
                out.copy_(full[a:b])
            elif b > a:
                dist.send(full[a:b].contiguous(), dst=r)
    elif hi > lo:
        dist.recv(out, src=src)
    return out


def gather_slices(shard: torch.Tensor, n_slices: int, dst: int = 0):
    """Inverse of scatter_slices: rank ``dst`` returns the [n_slices, *tail] tensor, the others None."""
    rank, world = dist.get_rank(), dist.get_world_size()
    if world == 1:
        return shard.clone()
    if rank == dst:
        full = torch.empty((n_slices, *shard.shape[1:]), dtype=shard.dtype, device=shard.device)
        for r in range(world):
            a, b = slice_range(r, world, n_slices)
            if r == dst:
                full[a:b].copy_(shard)
            elif b > a:
                dist.recv(full[a:b], src=r)
        return full
    if shard.shape[0] > 0:
        dist.send(shard.contiguous(), dst=dst)
    return None
