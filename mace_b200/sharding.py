"""Data-parallel sharding of an inference batch over the GPUs of one box.

Every operator on the path is independent across the batch dimension (Conv2D / depthwise /
pooling per image, FullyConnected per row, batched MatMul per batch entry), so the batch is
split into contiguous runs of images, one per rank, the weights are replicated, and the only
exchange is the final gather of the output rows.  One process per GPU; `dist` is
``torch.distributed`` with the NCCL backend on GPUs (gloo in the CPU tests).
"""
import numpy as np


def shard_bounds(batch, world, rank):
    """[begin, end) of the images rank `rank` of `world` processes: contiguous runs whose
    sizes differ by at most one (the first ``batch % world`` ranks get the extra image)."""
    if world < 1 or not (0 <= rank < world) or batch < 0:
        raise ValueError("bad shard request: batch=%d world=%d rank=%d" % (batch, world, rank))
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sizes(batch, world):
    return [shard_bounds(batch, world, r)[1] - shard_bounds(batch, world, r)[0] for r in range(world)]


def gather_rows(dist, local_rows, batch, device=None):
    """All ranks receive the [batch, ...] output assembled from every rank's rows (rank order =
    image order).  Shards may be ragged: rows are padded to the largest shard for the
    collective and trimmed afterwards.  `local_rows` is a numpy array; returns numpy."""
    import torch
    world, rank = dist.get_world_size(), dist.get_rank()
    sizes = shard_sizes(batch, world)
    if local_rows.shape[0] != sizes[rank]:
        raise ValueError("rank %d holds %d rows, its shard has %d" % (rank, local_rows.shape[0], sizes[rank]))
    width = max(sizes)
    padded = np.zeros((width,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype)
    padded[:sizes[rank]] = local_rows
    mine = torch.from_numpy(padded)
    if device is not None:
        mine = mine.to(device)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    out = [p.cpu().numpy()[:n] for p, n in zip(parts, sizes)]
    return np.concatenate(out, axis=0)
