"""(batch, head) sharding of a block-sparse problem over the GPUs of one box.

Every (z, h) pair of the path is an independent problem: dense tensors are
[Z, H, ., .], block-format tensors are [Z, nnz, block, block] with the blocks
of one head contiguous along nnz, and the layout carries one [Mb, Nb] slice
per head.  A problem is therefore split over ranks without any exchange step:
first along Z (every rank keeps the whole layout), then, when there are more
ranks than batch entries, along H (the rank takes a contiguous range of heads,
the matching layout slice and the matching range of blocks).

The only collective is the all-gather that reassembles outputs for
verification; it is never on a timed path.  The reference has no multi-GPU
code at all; this module has no counterpart there.
"""
from collections import namedtuple

import torch

Shard = namedtuple('Shard', 'z0 z1 h0 h1')


def plan(Z, H, world_size):
    """Splits Z x H into `world_size` shards.  Z is split first; if world_size
    exceeds Z, every batch entry is further split over heads.  Requires the
    split to be even (world_size | Z, or Z | world_size and (world_size/Z) | H)."""
    if world_size <= 0:
        raise ValueError('world_size must be positive')
    if Z % world_size == 0:
        per = Z // world_size
        return [Shard(r * per, (r + 1) * per, 0, H) for r in range(world_size)]
    if world_size % Z == 0 and H % (world_size // Z) == 0:
        parts = world_size // Z
        per = H // parts
        return [Shard(r // parts, r // parts + 1, (r % parts) * per, (r % parts + 1) * per) for r in range(world_size)]
    raise ValueError('cannot split Z=%d, H=%d evenly over %d ranks' % (Z, H, world_size))


def block_range(layout, h0, h1):
    """Range [b0, b1) of canonical block ids owned by heads [h0, h1)."""
    per_head = (layout != 0).sum((1, 2))
    b0 = int(per_head[:h0].sum())
    return b0, b0 + int(per_head[h0:h1].sum())


def slice_layout(layout, shard):
    return layout[shard.h0:shard.h1].contiguous()


def slice_dense(x, shard):
    """[Z, H, R, C] -> the shard's [z1-z0, h1-h0, R, C] view."""
    return x[shard.z0:shard.z1, shard.h0:shard.h1]


def slice_sparse(x, layout, shard):
    """[Z, nnz, block, block] -> the shard's batch entries and its heads' blocks."""
    b0, b1 = block_range(layout, shard.h0, shard.h1)
    return x[shard.z0:shard.z1, b0:b1]


def gather_dense(local, shards, Z, H, group=None):
    """All-gathers per-rank [z, h, R, C] results into the full [Z, H, R, C] tensor
    (verification only).  Works on any backend (NCCL on GPUs, gloo on CPU)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    out = torch.empty((Z, H) + tuple(local.shape[2:]), dtype=local.dtype, device=local.device)
    for part, s in zip(parts, shards):
        out[s.z0:s.z1, s.h0:s.h1] = part
    return out


def gather_sparse(local, layout, shards, Z, group=None):
    """All-gathers per-rank block-format results into the full [Z, nnz, block, block]
    tensor.  Shards that split heads own different numbers of blocks, so every
    rank pads to the largest shard before the collective."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    ranges = [block_range(layout, s.h0, s.h1) for s in shards]
    widest = max(b1 - b0 for b0, b1 in ranges)
    zmax = max(s.z1 - s.z0 for s in shards)
    padded = torch.zeros((zmax, widest) + tuple(local.shape[2:]), dtype=local.dtype, device=local.device)
    padded[:local.size(0), :local.size(1)] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    nnz = int((layout != 0).sum())
    out = torch.empty((Z, nnz) + tuple(local.shape[2:]), dtype=local.dtype, device=local.device)
    for part, s, (b0, b1) in zip(parts, shards, ranges):
        out[s.z0:s.z1, b0:b1] = part[:s.z1 - s.z0, :b1 - b0]
    return out
