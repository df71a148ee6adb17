"""Data-parallel helpers: the path shards by batch, and the only exchange it needs is the sum of
the weight / bias gradients over the ranks (the reference is single-device; its per-batch loop,
package/ext_modules/src/nn/cuda/mapped_convolution_layer.cu:174-190, is what makes the weight
gradient the one cross-batch reduction)."""
import torch
import torch.distributed as dist


def shard_batch(batch, rank, world):
    """Contiguous slice [begin, end) of a batch of `batch` elements owned by `rank`."""
    base, rem = divmod(batch, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def allreduce_gradients(tensors, group=None):
    """Sum the given gradient tensors over all ranks with ONE collective: they are flattened into a
    single fp32 bucket, all-reduced, and copied back in place (in their own dtype).
    Returns the bucket (fp32, summed)."""
    tensors = [t for t in tensors if t is not None]
    if not tensors:
        return None
    bucket = torch.cat([t.detach().reshape(-1).float() for t in tensors])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for t in tensors:
        n = t.numel()
        t.detach().copy_(bucket[off:off + n].view_as(t))
        off += n
    return bucket
