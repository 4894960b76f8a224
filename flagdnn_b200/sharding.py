"""Batch sharding of the convolution path across the GPUs of one node.

Every output image depends only on its own input image and the replicated
filter, bias and scale, so rank r of g simply owns a contiguous slice of the
batch: no halo, no exchange, no collective on the hot path.  The helpers here
compute the slices and, where a caller wants the whole activation on every
rank, gather it with torch.distributed (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def batch_slice(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the images rank ``rank`` of ``world`` owns; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's images of a batch-major tensor (a view, no copy)."""
    begin, end = batch_slice(x.shape[0], rank, world)
    return x[begin:end]


def gather_batch(y_local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """All ranks' output slices concatenated along the batch on every rank.

    Optional epilogue of a sharded run; slices may differ in size by one image,
    so every rank pads to the largest slice for the collective and trims after.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [batch_slice(n_total, r, world) for r in range(world)]
    largest = max(e - b for b, e in sizes)
    padded = y_local
    if y_local.shape[0] < largest:
        pad = torch.zeros((largest - y_local.shape[0], *y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
        padded = torch.cat([y_local, pad], dim=0)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[: e - b] for p, (b, e) in zip(parts, sizes)], dim=0)
