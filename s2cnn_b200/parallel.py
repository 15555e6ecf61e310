"""Batch data parallelism for the spectral path: one process per GPU, each rank owns a slice of
the batch.  Forward needs no communication; a training step reduces the parameter gradients once.

The reference has no distributed code at all (no NCCL/MPI/DataParallel anywhere in its sources);
this is the minimal layer the path needs on an 8-GPU NVSwitch box.
"""
import torch
import torch.distributed as dist


def shard_range(n, rank, world):
    """Contiguous [start, stop) of `n` batch elements owned by `rank`; sizes differ by at most 1,
    every element is owned exactly once, empty ranges are allowed when world > n."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def allreduce_gradients(params, average=False, group=None):
    """Sum (or average) ``.grad`` of the given parameters over all ranks with ONE all-reduce of a
    flat bucket (the gradients of this path are small - a few MB - so latency, not bandwidth,
    decides; one launch instead of one per parameter).  The real-space ``kernel.grad``
    ([f_in, f_out, n_grid]) is reduced, not the ~14x larger spectral gradient: the kernel transform
    is linear, so the two orders commute.  No-op when torch.distributed is not initialised."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n
    return flat.numel()


def max_over_ranks(value, device="cpu", group=None):
    """Max of a python float over ranks (used for device-time reporting)."""
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
