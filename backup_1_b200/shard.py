"""Sharding of the hot path over ranks (one process per GPU).

GEMM shards by row-blocks of A and C (B replicated); the convolution shards by images.  Every
rank computes its shard with the single-GPU entry points and no data-path collective; the
gathered result exists only when the caller asks for it (one all-gather of row-blocks /
images).  The reference has no multi-device code (DECX_cpu/DECX_CPU.cpp:9: "supports only
single GPU"); the partition rule below is this implementation's.
"""
from __future__ import annotations


def block_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block [first, last) of `total` units owned by `rank`; the first
    `total % world` ranks own one unit more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    base, extra = divmod(total, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def gemm_row_shard(M: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [first, last) of A and C that `rank` owns."""
    return block_range(M, world, rank)


def conv_batch_shard(batch: int, world: int, rank: int) -> tuple[int, int]:
    """Images [first, last) that `rank` owns."""
    return block_range(batch, world, rank)


def all_gather_blocks(local, total_units: int, group=None):
    """All-gather of per-rank blocks of unequal size along dim 0 (torch.distributed, any
    backend).  `local` holds this rank's units [first, last) of `total_units`.  Returns the
    full tensor [total_units, ...] on every rank."""
    import torch
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    first, last = block_range(total_units, world, rank)
    assert local.shape[0] == last - first
    sizes = [block_range(total_units, world, r) for r in range(world)]
    full = torch.empty((total_units,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if len({b - a for a, b in sizes}) == 1:
        dist.all_gather_into_tensor(full, local.contiguous(), group=group)
    else:
        # unequal blocks: gather blocks padded to the largest size, then keep the valid rows
        mx = max(b - a for a, b in sizes)
        padded = torch.zeros((mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded[: last - first] = local
        tmp = torch.empty((world * mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(tmp, padded, group=group)
        for r, (a, b) in enumerate(sizes):
            full[a:b] = tmp[r * mx: r * mx + (b - a)]
    return full
