"""Batch-dimension partitioner for one process per GPU.

Convolution over the batch has no cross-image state (the reference kernel already decomposes
its grid into (image, tile), Tetris/spconv2d_kernel.cu:74-76), so the multi-GPU path is plain
sharding: rank r of `world` owns the contiguous batch slice given by the C ABI's
tetris_batch_slice; there is no collective on the data path.  The only optional exchange is the
final gather of the per-rank outputs, done with torch.distributed (NCCL on GPUs, gloo on CPU).
"""
import torch
import torch.distributed as dist


def slice_bounds(batch_size, world, rank):
    """(begin, count): same arithmetic as tetris_batch_slice in the native library."""
    base, extra = divmod(batch_size, world)
    return rank * base + min(rank, extra), base + (1 if rank < extra else 0)


def shard_batch(x, world=None, rank=None):
    """The slice of a batch-major tensor that this rank owns (a view, no copy)."""
    world = dist.get_world_size() if world is None else world
    rank = dist.get_rank() if rank is None else rank
    begin, count = slice_bounds(x.shape[0], world, rank)
    return x[begin:begin + count]


def gather_shards(y_local, batch_size, world=None, rank=None):
    """All ranks receive the whole batch, shard outputs concatenated in rank order.

    Shards may differ by one image, so every rank pads its shard to the largest one before the
    all-gather and the padding is cut away afterwards.
    """
    world = dist.get_world_size() if world is None else world
    rank = dist.get_rank() if rank is None else rank
    counts = [slice_bounds(batch_size, world, r)[1] for r in range(world)]
    assert y_local.shape[0] == counts[rank], "shard has %d images, expected %d" % (y_local.shape[0], counts[rank])
    largest = max(counts)
    padded = y_local
    if y_local.shape[0] < largest:
        pad = torch.zeros((largest - y_local.shape[0],) + tuple(y_local.shape[1:]),
                          dtype=y_local.dtype, device=y_local.device)
        padded = torch.cat([y_local, pad], 0)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous())
    return torch.cat([p[:c] for p, c in zip(parts, counts)], 0)
