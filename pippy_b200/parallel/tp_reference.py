"""Plain ``torch.distributed`` statements of the tensor-parallel linears (CPU tests, and the oracle of the fused
kernels): all-gather then matmul, matmul then reduce-scatter, both differentiable."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(out, x.contiguous(), group=group)
        return torch.cat(out, dim=0)

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        parts = [p.contiguous() for p in g.chunk(world, dim=0)]
        out = torch.empty_like(parts[0])
        dist.reduce_scatter(out, parts, group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        parts = [p.contiguous() for p in x.chunk(world, dim=0)]
        out = torch.empty_like(parts[0])
        dist.reduce_scatter(out, parts, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        out = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(out, g.contiguous(), group=ctx.group)
        return torch.cat(out, dim=0), None


def column_parallel_reference(x_shard, weight, group):
    x = _AllGatherRows.apply(x_shard, group) if group is not None and dist.get_world_size(group) > 1 else x_shard
    return F.linear(x, weight)


def row_parallel_reference(x, weight, residual_shard, group):
    y = F.linear(x, weight)
    if group is not None and dist.get_world_size(group) > 1:
        y = _ReduceScatterRows.apply(y, group)
    return y if residual_shard is None else y + residual_shard
