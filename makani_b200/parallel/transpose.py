"""Distributed transposes: swap which tensor dimension is sharded over a process group.

`distributed_transpose(x, (dim0, dim1), dim1_split_sizes, group_name)` splits the local tensor along `dim0`
into near-equal (ceil) chunks, exchanges them all-to-all and concatenates what arrives along `dim1`, whose
per-rank extents are `dim1_split_sizes`; the backward pass is the reverse transpose.  Same contract as
torch-harmonics' `distributed_transpose_azimuth/polar` used at makani/mpu/layers.py:72-99.

This NCCL/gloo formulation is the portable path (CPU tests, baseline).  On NVLink machines the spectral
transforms read the peers' tiles directly from inside the GEMM kernels (`makani_b200.parallel.peer`).
"""

from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils import comm
from .helpers import compute_split_shapes, split_tensor_along_dim


def _all_to_all(recv, send, group, name):
    """all_to_all with a point-to-point fallback for backends without it (gloo)."""
    if dist.get_backend(group) != "gloo":
        dist.all_to_all(recv, send, group=group)
        return
    ranks = comm.get_group_ranks(name)
    me = comm.get_rank(name)
    recv[me].copy_(send[me])
    reqs = []
    for r, gr in enumerate(ranks):
        if r == me:
            continue
        reqs.append(dist.isend(send[r], dst=gr, group=group))
        reqs.append(dist.irecv(recv[r], src=gr, group=group))
    for q in reqs:
        q.wait()


def _transpose(x: torch.Tensor, dim0: int, dim1: int, dim1_split_sizes: Sequence[int], name: str):
    size = comm.get_size(name)
    group = comm.get_group(name)
    is_complex = x.is_complex()
    xr = torch.view_as_real(x) if is_complex else x
    dim0 = dim0 % x.dim()
    dim1 = dim1 % x.dim()
    send = [c.contiguous() for c in split_tensor_along_dim(xr, dim0, size)]
    dim0_sizes = compute_split_shapes(x.shape[dim0], size)
    my = comm.get_rank(name)
    recv = []
    for r in range(size):
        shp = list(send[my].shape)
        shp[dim1] = dim1_split_sizes[r]
        recv.append(torch.empty(shp, dtype=xr.dtype, device=xr.device))
    _all_to_all(recv, send, group, name)
    out = torch.cat(recv, dim=dim1)
    if is_complex:
        out = torch.view_as_complex(out)
    return out, dim0_sizes


class _DistributedTranspose(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dims, dim1_split_sizes, name):
        ctx.dims, ctx.name = dims, name
        out, ctx.dim0_sizes = _transpose(x, dims[0], dims[1], dim1_split_sizes, name)
        return out

    @staticmethod
    def backward(ctx, g):
        d0, d1 = ctx.dims
        gi, _ = _transpose(g.contiguous(), d1, d0, ctx.dim0_sizes, ctx.name)
        return gi, None, None, None


def distributed_transpose(x: torch.Tensor, dims: Tuple[int, int], dim1_split_sizes: Sequence[int], name: str):
    if comm.get_size(name) == 1:
        return x
    return _DistributedTranspose.apply(x, dims, list(dim1_split_sizes), name)


def distributed_transpose_azimuth(x, dims, dim1_split_sizes):
    return distributed_transpose(x, dims, dim1_split_sizes, "w")


def distributed_transpose_polar(x, dims, dim1_split_sizes):
    return distributed_transpose(x, dims, dim1_split_sizes, "h")
