"""Shape utilities and cold-path collectives for model-parallel tensors.

`compute_split_shapes` is the ceil-chunk rule every sharded dimension follows (e.g. 721 over 4 ranks ->
[181, 181, 181, 178]); the reference takes it from modulus (`modulus.distributed.utils.compute_split_shapes`,
used at makani/mpu/layers.py:26,61-64).  `gather_uneven` and `sync_params` mirror makani/mpu/helpers.py:33-103.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..utils import comm


def compute_split_shapes(size: int, num_chunks: int) -> List[int]:
    if num_chunks == 1:
        return [size]
    chunk = (size + num_chunks - 1) // num_chunks
    last = max(0, size - chunk * (num_chunks - 1))
    if last == 0:
        chunk = size // num_chunks
        last = size - chunk * (num_chunks - 1)
    return [chunk] * (num_chunks - 1) + [last]


def split_tensor_along_dim(tensor: torch.Tensor, dim: int, num_chunks: int):
    assert dim < tensor.dim()
    assert tensor.shape[dim] >= num_chunks, f"cannot split dim {dim} of size {tensor.shape[dim]} into {num_chunks} chunks"
    return list(torch.split(tensor, compute_split_shapes(tensor.shape[dim], num_chunks), dim=dim))


def get_memory_format(tensor: torch.Tensor):
    return torch.channels_last if tensor.is_contiguous(memory_format=torch.channels_last) else torch.contiguous_format


def all_gather_uneven(t: torch.Tensor, dim: int, sizes: List[int], group) -> torch.Tensor:
    """Concatenate along `dim` the tensors of all ranks, whose extents along `dim` are `sizes`.
    Shards are padded to the largest extent for the collective (every backend supports equal-size all_gather)."""
    dim = dim % t.dim()
    is_complex = t.is_complex()
    tr = torch.view_as_real(t) if is_complex else t
    tr = tr.contiguous()
    smax = max(sizes)
    if tr.shape[dim] < smax:
        pad_shape = list(tr.shape)
        pad_shape[dim] = smax - tr.shape[dim]
        tr = torch.cat([tr, torch.zeros(pad_shape, dtype=tr.dtype, device=tr.device)], dim=dim)
    outs = [torch.empty_like(tr) for _ in sizes]
    dist.all_gather(outs, tr, group=group)
    out = torch.cat([o.narrow(dim, 0, s) for o, s in zip(outs, sizes)], dim=dim)
    return torch.view_as_complex(out.contiguous()) if is_complex else out


def gather_uneven(tensor: torch.Tensor, dim: int, comm_name: str) -> torch.Tensor:
    """All-gather `tensor` along `dim` over group `comm_name` when ranks hold different extents along `dim`."""
    size = comm.get_size(comm_name)
    if size == 1:
        return tensor
    group = comm.get_group(comm_name)
    dim = dim % tensor.dim()
    my = torch.tensor([tensor.shape[dim]], dtype=torch.int64, device=tensor.device)
    sizes = [torch.empty_like(my) for _ in range(size)]
    dist.all_gather(sizes, my, group=group)
    return all_gather_uneven(tensor, dim, [int(s.item()) for s in sizes], group)


def sync_params(model: torch.nn.Module, mode: str = "broadcast") -> None:
    """Make replicated parameters identical: over `data`, and over every group named in `param.is_shared_mp`."""
    if not dist.is_initialized():
        return
    with torch.no_grad():
        for p in model.parameters():
            groups = ["data"] + list(getattr(p, "is_shared_mp", ["model"]))
            t = torch.view_as_real(p.data) if p.is_complex() else p.data
            for g in groups:
                if comm.get_size(g) <= 1:
                    continue
                if mode == "broadcast":
                    dist.broadcast(t, src=comm.get_root(g), group=comm.get_group(g))
                elif mode == "mean":
                    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=comm.get_group(g))
                    t.div_(comm.get_size(g))
                else:
                    raise ValueError(f"unknown sync mode {mode}")
