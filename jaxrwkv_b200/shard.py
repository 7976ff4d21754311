"""Batch sharding of the WKV operator across the GPUs of one node.

The recurrence is independent per (batch, head) (src/jaxrwkv/rwkv7.py:324-325 vmaps the
per-head algebra), so ranks own contiguous slices of the batch and never exchange data on this
path.  ``torch.distributed`` is used only to agree on timing (barrier, max over ranks).
"""
import torch
import torch.distributed as dist


def shard_bounds(global_batch, rank, world):
    """Contiguous slice [start, stop) of the batch owned by ``rank``; sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(value, device=None):
    """Max of a Python float over all ranks (identity when no process group is initialised)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device=None):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
