"""Multi-GPU host logic: the path shards into independent (batch, head) units, so ranks never exchange data inside
a step. One process per GPU (torch.distributed; NCCL on GPUs, gloo in the CPU tests). The only collective is the
optional all-gather of the attention output for a consumer that needs every head on every rank (the boundary
where a head-sharded attention meets a replicated output projection).

The reference has no multi-device code at all (single device, batch-1 planning, docs/LIMITATIONS.md:15-32)."""
from __future__ import annotations


def shard_range(n_units, rank, world):
    """Contiguous, balanced split of n_units over `world` ranks: the first n_units % world ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank %d of %d" % (rank, world))
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_dim(t, dim, rank, world):
    """The rank's slice of tensor `t` along `dim` (a view, no copy)."""
    lo, hi = shard_range(t.shape[dim], rank, world)
    return t.narrow(dim, lo, hi - lo)


def gather_dim(local, dim, n_total, group=None):
    """All-gather ragged shards along `dim` back into the full tensor on every rank. Shards may differ by one unit,
    so they are padded to the largest shard for the collective and trimmed afterwards."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return local
    sizes = [shard_range(n_total, r, world) for r in range(world)]
    biggest = max(hi - lo for lo, hi in sizes)
    moved = local.movedim(dim, 0).contiguous()
    if moved.shape[0] < biggest:
        pad = torch.zeros((biggest - moved.shape[0],) + tuple(moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        moved = torch.cat([moved, pad], 0)
    out = [torch.empty_like(moved) for _ in range(world)]
    dist.all_gather(out, moved, group=group)
    full = torch.cat([o[: hi - lo] for o, (lo, hi) in zip(out, sizes)], 0)
    return full.movedim(0, dim).contiguous()
