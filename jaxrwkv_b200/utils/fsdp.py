"""ZeRO-3 style parameter sharding over one process group (NCCL over NVLink on the GPUs, gloo on CPU).

The counterpart of jaxrwkv's src/jaxrwkv/utils/fsdp.py with the same names and rules: a parameter
of at least ``min_weight_size`` elements is split along its largest axis divisible by the group size
(``shard_param``, fsdp.py:30-41), gathered on use with an all-gather whose backward is a
reduce-scatter divided by the group size (``gather_param``, fsdp.py:43-55), and the gradients of the
small replicated parameters are averaged (``sync_grads``, fsdp.py:60-64).  No collective touches
the WKV operator itself; these wrap the projections around it in a training step.
"""
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist


@dataclass
class Partitioned:
    v: torch.Tensor          # the local shard (or the whole tensor when idx == 0)
    idx: int                 # sharded axis as a negative index, 0 = replicated (fsdp.py:16)
    group: Optional[Any] = None

    def gathered(self):
        return gather_param(self)


def _size(group):
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group):
    return dist.get_rank(group) if dist.is_initialized() else 0


def shard_param(value, group=None, min_weight_size=2 ** 18):
    """Keep this rank's slice of ``value`` along the largest axis the group size divides (fsdp.py:30-41)."""
    n = _size(group)
    if value.numel() < min_weight_size or n == 1:
        return Partitioned(value, 0, group)
    for i in sorted(range(value.dim()), key=lambda a: -value.shape[a]):
        if value.shape[i] % n == 0:
            step = value.shape[i] // n
            r = _rank(group)
            return Partitioned(value.narrow(i, r * step, step).contiguous(), i - value.dim(), group)
    return Partitioned(value, 0, group)          # no divisible axis: stays replicated (fsdp.py:40-41)


class _GatherMeanGrads(torch.autograd.Function):
    """all-gather along ``axis``; the gradient is reduce-scattered and divided by the group size."""

    @staticmethod
    def forward(ctx, x, axis, group):
        ctx.axis, ctx.group = axis, group
        n = _size(group)
        xm = x.movedim(axis, 0).contiguous()
        out = torch.empty((n * xm.shape[0],) + tuple(xm.shape[1:]), dtype=x.dtype, device=x.device)
        if dist.get_backend(group) == "gloo":
            parts = list(out.chunk(n, 0))
            dist.all_gather(parts, xm, group=group)
        else:
            dist.all_gather_into_tensor(out, xm, group=group)
        return out.movedim(0, axis)

    @staticmethod
    def backward(ctx, g):
        n = _size(ctx.group)
        gm = g.movedim(ctx.axis, 0).contiguous()
        step = gm.shape[0] // n
        if dist.get_backend(ctx.group) == "gloo":       # gloo has no reduce-scatter: all-reduce and keep our slice
            dist.all_reduce(gm, group=ctx.group)
            mine = gm.narrow(0, _rank(ctx.group) * step, step).clone()
        else:
            mine = torch.empty((step,) + tuple(gm.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(mine, gm, group=ctx.group)
        return (mine / n).movedim(0, ctx.axis), None, None


def gather_param(value):
    if not isinstance(value, Partitioned):
        return value
    if value.idx == 0:
        return value.v
    return _GatherMeanGrads.apply(value.v, value.v.dim() + value.idx, value.group)


def _map(fn, tree):
    if isinstance(tree, dict):
        return {k: _map(fn, v) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(_map(fn, v) for v in tree)
    return fn(tree)


def gather_params(params):
    """Gather every Partitioned leaf of a (nested dict / list) parameter tree (fsdp.py:57-58)."""
    return _map(gather_param, params)


def sync_grads(value):
    """Average the gradient of a replicated leaf over the group; sharded leaves are already reduced."""
    if isinstance(value, Partitioned) and value.idx == 0 and value.v.grad is not None and _size(value.group) > 1:
        dist.all_reduce(value.v.grad, group=value.group)
        value.v.grad /= _size(value.group)
    return value


def sharded_to_cpu(params):
    """Full parameter tree on the host (fsdp.py:66-67): gathers the shards, then copies."""
    with torch.no_grad():
        return _map(lambda x: gather_param(x).cpu() if isinstance(x, Partitioned) else x, params)
