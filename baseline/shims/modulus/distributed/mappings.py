"""Autograd-aware collectives over a named process group (identity / all-reduce / split / uneven all-gather)."""

import torch
import torch.distributed as dist

from .manager import DistributedManager
from .utils import compute_split_shapes


def _grp(name):
    m = DistributedManager()
    return m.group(name), m.group_size(name), m.group_rank(name)


def _all_reduce(x, name):
    g, n, _ = _grp(name)
    if n == 1:
        return x
    x = x.contiguous()
    dist.all_reduce(x, group=g)
    return x


def _split(x, dim, name):
    g, n, r = _grp(name)
    if n == 1:
        return x
    return torch.split(x, compute_split_shapes(x.shape[dim], n), dim=dim)[r].contiguous()


def _gather(x, dim, shapes, name):
    g, n, r = _grp(name)
    if n == 1:
        return x
    x = x.contiguous()
    if shapes is None:
        shapes = [x.shape[dim]] * n
    outs = []
    for s in shapes:
        shp = list(x.shape)
        shp[dim] = s
        outs.append(torch.empty(shp, dtype=x.dtype, device=x.device))
    if len(set(shapes)) == 1:
        dist.all_gather(outs, x, group=g)
    else:
        # uneven: pad to the largest shard, gather, trim
        big = max(shapes)
        pad = list(x.shape)
        pad[dim] = big
        xp = x.new_zeros(pad)
        xp.narrow(dim, 0, x.shape[dim]).copy_(x)
        tmp = [torch.empty_like(xp) for _ in range(n)]
        dist.all_gather(tmp, xp, group=g)
        outs = [t.narrow(dim, 0, s) for t, s in zip(tmp, shapes)]
    return torch.cat(outs, dim=dim).contiguous()


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):
        ctx.name = name
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g, ctx.name), None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):
        return _all_reduce(x, name)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, name):
        ctx.dim, ctx.name = dim, name
        _, n, _ = _grp(name)
        ctx.shapes = compute_split_shapes(x.shape[dim], n)
        return _split(x, dim, name)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.dim, ctx.shapes, ctx.name), None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, shapes, name):
        ctx.dim, ctx.name = dim, name
        return _gather(x, dim, shapes, name)

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.dim, ctx.name), None, None, None


def copy_to_parallel_region(x, group):
    return _Copy.apply(x, group)


def reduce_from_parallel_region(x, group):
    return _Reduce.apply(x, group)


def scatter_to_parallel_region(x, dim, group):
    return _Scatter.apply(x, dim, group)


def gather_from_parallel_region(x, dim, shapes, group):
    return _Gather.apply(x, dim, shapes, group)
