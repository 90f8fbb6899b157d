"""Column sharding of the hot path across the GPUs of one node.

The dense feature matrix ``X [N, F]`` is cut into ``G`` contiguous column blocks, one per
rank; the compressed graph is replicated.  Propagation, mean, mean-backward and reconstruct
act on every column independently, so they run on the local block with no communication.
Only the LSH assignment needs whole rows: each rank projects its block onto its slice of the
hyperplanes and the partial projections are summed with ONE all-reduce (NCCL over NVLink on
GPUs, gloo in the CPU tests) before sign packing, after which every rank derives the same
bucket ids, counts and permutation.
"""
import torch
import torch.distributed as dist


def column_range(width, rank, world):
    """``(begin, end)`` of rank's block; blocks are ``ceil(width / world)`` wide, the last one
    takes what is left (the convention the CPU oracle's sharded projection uses)."""
    per = -(-int(width) // int(world))
    begin = min(rank * per, width)
    return begin, min(begin + per, width)


def shard_columns(x, rank, world):
    """This rank's contiguous column block of ``x`` as its own contiguous tensor."""
    begin, end = column_range(x.size(-1), rank, world)
    return x[..., begin:end].contiguous()


def shard_planes(planes, rank, world):
    """Rows of the ``[F, H]`` hyperplane matrix that belong to this rank's feature columns."""
    begin, end = column_range(planes.size(0), rank, world)
    return planes[begin:end].contiguous()


def allreduce_projection(partial, group=None):
    """Sum the ``[N, H]`` partial projections of all ranks in place (the path's one collective)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def gather_columns(local, group=None):
    """Concatenate every rank's column block (test / export helper, not on the hot path)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local, group=group)
    return torch.cat(parts, dim=-1)
