"""Autograd-aware collectives between replicated and sharded regions of the model.

Contract of `modulus.distributed.mappings` as used by the reference (makani/mpu/layers.py:27-30,
makani/mpu/layer_norm.py:25, makani/utils/losses.py:28):

    copy_to_parallel_region(x, g)         forward identity            backward all-reduce(SUM)
    reduce_from_parallel_region(x, g)     forward all-reduce(SUM)     backward identity
    scatter_to_parallel_region(x, d, g)   forward keep local chunk    backward all-gather
    gather_from_parallel_region(x,d,s,g)  forward uneven all-gather   backward keep local chunk
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..utils import comm
from .helpers import all_gather_uneven, compute_split_shapes, split_tensor_along_dim


def _all_reduce(x: torch.Tensor, name: str) -> torch.Tensor:
    if comm.get_size(name) == 1:
        return x
    x = x.contiguous()
    if x.is_complex():
        dist.all_reduce(torch.view_as_real(x), group=comm.get_group(name))
    else:
        dist.all_reduce(x, group=comm.get_group(name))
    return x


def _split(x: torch.Tensor, dim: int, name: str) -> torch.Tensor:
    size = comm.get_size(name)
    if size == 1:
        return x
    return split_tensor_along_dim(x, dim, size)[comm.get_rank(name)].contiguous()


def _gather(x: torch.Tensor, dim: int, shapes: Optional[List[int]], name: str) -> torch.Tensor:
    size = comm.get_size(name)
    if size == 1:
        return x
    dim = dim % x.dim()
    if shapes is None:
        sz = torch.tensor([x.shape[dim]], dtype=torch.int64, device=x.device)
        all_sz = [torch.empty_like(sz) for _ in range(size)]
        dist.all_gather(all_sz, sz, group=comm.get_group(name))
        shapes = [int(s.item()) for s in all_sz]
    return all_gather_uneven(x, dim, list(shapes), comm.get_group(name))


class _CopyTo(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):
        ctx.name = name
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.clone(), ctx.name), None


class _ReduceFrom(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, name):
        return _all_reduce(x.clone(), name)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterTo(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, name):
        ctx.dim, ctx.name = dim, name
        ctx.shapes = compute_split_shapes(x.shape[dim], comm.get_size(name))
        return _split(x, dim, name)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.dim, ctx.shapes, ctx.name), None, None


class _GatherFrom(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, shapes, name):
        ctx.dim, ctx.name = dim, name
        return _gather(x, dim, shapes, name)

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.dim, ctx.name), None, None, None


def copy_to_parallel_region(x, name):
    return x if comm.get_size(name) == 1 else _CopyTo.apply(x, name)


def reduce_from_parallel_region(x, name):
    return x if comm.get_size(name) == 1 else _ReduceFrom.apply(x, name)


def scatter_to_parallel_region(x, dim, name):
    return x if comm.get_size(name) == 1 else _ScatterTo.apply(x, dim, name)


def gather_from_parallel_region(x, dim, shapes, name):
    return x if comm.get_size(name) == 1 else _GatherFrom.apply(x, dim, shapes, name)


# ------------------------------------------------------------------------------------------------ gradient reduction


class ReducedModule(torch.nn.Module):
    """What `init_gradient_reduction_hooks` returns: the model under `.module` (state-dict keys carry the `module.`
    prefix, as with DistributedDataParallel) plus a `GradReducer` that runs by itself at the end of every backward
    pass.  A plain training loop (`loss.backward(); optimizer.step(); optimizer.zero_grad()`) therefore needs no call
    into this framework, whichever `set_to_none` it uses."""

    def __init__(self, module: torch.nn.Module, bucket_mb: float = 25.0):
        super().__init__()
        from .grad_reduce import GradReducer

        self.module = module
        # no overlap: gradients that autograd allocated itself (after `zero_grad(set_to_none=True)`) are moved into the
        # reducer's flat buffer when backward ends, so the reduction cannot start before that
        self.reducer = GradReducer(module, bucket_mb=bucket_mb, overlap=False)
        self._views = [p.grad for p in self.reducer.params]
        self._queued = False
        for p in self.reducer.params:
            p.register_post_accumulate_grad_hook(self._on_grad)

    def _on_grad(self, _param):
        if not self._queued:
            self._queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish)

    def _finish(self):
        self._queued = False
        with torch.no_grad():
            for p, view in zip(self.reducer.params, self._views):
                if p.grad is None:
                    view.zero_()                 # unused in this pass: contributes nothing to the average
                elif p.grad.data_ptr() != view.data_ptr():
                    view.copy_(p.grad)
                p.grad = view
        self.reducer.reduce()

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)


def init_gradient_reduction_hooks(model, device_ids=None, output_device=None, bucket_cap_mb=25, broadcast_buffers=True,
                                  find_unused_parameters=False, gradient_as_bucket_view=True, static_graph=False):
    """Calling convention of makani/mpu/mappings.py:30-174: returns the model wrapped such that, after every backward
    pass, gradients are averaged over the `data` group and summed over the groups named in `param.is_shared_mp`.
    Without an initialised process group the model is returned unchanged.  The DDP-specific arguments are accepted and
    ignored: there are no buckets to tune and no buffers to broadcast (the trainer of this framework drives a
    `GradReducer` directly, with overlap; this entry point serves user loops written against the upstream function)."""
    if not dist.is_initialized():
        return model
    return ReducedModule(model, bucket_mb=float(bucket_cap_mb))
