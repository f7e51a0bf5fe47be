"""Multi-GPU plumbing for the hot path: one process per GPU, the (image, fixation) rows are independent,
so each rank takes a contiguous shard of the images (all fixations of an image stay on one GPU: the
image is read once), tables and weights are replicated, and there is no collective on the data path.
The one optional collective gathers final outputs (e.g. CLS embeddings) on every rank."""
import torch
import torch.distributed as dist

__all__ = ["shard_range", "shard_batch", "all_gather_rows"]


def shard_range(n, rank, world):
    """[lo, hi) of `n` items for `rank` of `world`: contiguous, sizes differ by at most one, earlier ranks
    take the larger shards."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(*tensors, rank=None, world=None):
    """Slice every tensor's leading (image) dimension to this rank's shard."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    lo, hi = shard_range(tensors[0].shape[0], rank, world)
    out = tuple(t[lo:hi] for t in tensors)
    return out if len(out) > 1 else out[0]


def all_gather_rows(y, total_rows=None, group=None):
    """Concatenate every rank's rows (dimension 0) in rank order on all ranks.  Shards may differ in size
    by one row (shard_range); they are padded to the largest shard for the collective and trimmed after.
    `total_rows` (sum over ranks) avoids the extra all-gather of shard sizes."""
    world = dist.get_world_size(group)
    if world == 1:
        return y
    rank = dist.get_rank(group)
    if total_rows is None:
        sizes = torch.zeros(world, dtype=torch.long, device=y.device)
        sizes[rank] = y.shape[0]
        dist.all_reduce(sizes, group=group)
        sizes = [int(s) for s in sizes.tolist()]
    else:
        sizes = [shard_range(total_rows, r, world)[1] - shard_range(total_rows, r, world)[0] for r in range(world)]
    big = max(sizes)
    if y.shape[0] < big:
        y = torch.cat([y, y.new_zeros((big - y.shape[0],) + tuple(y.shape[1:]))], 0)
    out = y.new_empty((world * big,) + tuple(y.shape[1:]))
    dist.all_gather_into_tensor(out, y.contiguous(), group=group)
    if all(s == big for s in sizes):
        return out
    return torch.cat([out[r * big: r * big + sizes[r]] for r in range(world)], 0)
