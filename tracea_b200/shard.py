"""Batch sharding of a conv workload over the GPUs of one box.

Output pixel m = (n, ho, wo) depends on image n alone, so the path shards by image with no
exchange step: rank g of G owns images [g*N/G, (g+1)*N/G), weights and bias are replicated, and no
collective is issued on the data path. (The reference opens device 0 only,
src/runtime/manager/mod.rs:100; sharding is this library's addition.) torch.distributed is used by
callers for the start/stop barrier and the max-over-ranks of the timing, nothing else.
"""


def shard_range(n_images, rank, world_size):
    """Contiguous [begin, end) of the images rank `rank` owns. The first n_images % world_size ranks
    get one extra image, so every image is owned exactly once and shard sizes differ by at most one."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("rank %d out of range for world size %d" % (rank, world_size))
    if n_images < 0:
        raise ValueError("negative batch")
    base, extra = divmod(n_images, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sizes(n_images, world_size):
    return [b - a for a, b in (shard_range(n_images, r, world_size) for r in range(world_size))]


def max_over_ranks(value, group=None):
    """Max of a per-rank scalar (e.g. elapsed milliseconds) over the process group; the identity when
    torch.distributed is not initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sum_over_ranks(value, group=None):
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())
