"""Batch sharding of the semiring products over the GPUs of one node.

Every batch element of every operator is independent (the reference maps batch to blockIdx.z,
matmul_cuda_kernel.cu:24), so the N-GPU path is: one process per GPU, rank r owns a contiguous
slice of the batch, forward and backward need no communication, and a collective appears only
if the caller wants the results of all shards in one place (`gather_batch`, an all-gather).
No kernel reads another GPU's memory.
"""
import torch
import torch.distributed as dist


def shard_bounds(batch, rank, world):
    """[lo, hi) of rank's contiguous batch slice; the first batch % world ranks get one more."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(x, rank=None, world=None, group=None):
    """This rank's slice (a view) of a tensor whose first dimension is the batch."""
    rank = dist.get_rank(group) if rank is None else rank
    world = dist.get_world_size(group) if world is None else world
    lo, hi = shard_bounds(x.shape[0], rank, world)
    return x[lo:hi]


def gather_batch(local, batch, group=None):
    """All-gather the per-rank results into the full (batch, ...) tensor on every rank."""
    world = dist.get_world_size(group)
    sizes = [hi - lo for lo, hi in (shard_bounds(batch, r, world) for r in range(world))]
    pad = max(sizes)
    buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
    buf[: local.shape[0]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf.contiguous(), group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], 0)


def sharded_apply(fn, *batched, group=None, gather=True):
    """fn on this rank's slice of every argument; optionally all-gather the result."""
    batch = batched[0].shape[0]
    local = fn(*[shard_batch(x, group=group) for x in batched])
    return gather_batch(local, batch, group) if gather else local
