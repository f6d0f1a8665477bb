"""Distributed SHT stand-in: latitude split over the polar group, longitude over the azimuth group; each transform is
two local stages (longitude FFT, Legendre contraction) with split / `all_to_all` / cat transposes around them."""

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from ..legendre import precompute_legpoly
from ..sht import _grid

_POLAR_GROUP = None
_AZIMUTH_GROUP = None
_IS_INITIALIZED = False


def init(polar_process_group, azimuth_process_group):
    global _POLAR_GROUP, _AZIMUTH_GROUP, _IS_INITIALIZED
    _POLAR_GROUP, _AZIMUTH_GROUP, _IS_INITIALIZED = polar_process_group, azimuth_process_group, True


def is_initialized():
    return _IS_INITIALIZED


def polar_group():
    return _POLAR_GROUP


def azimuth_group():
    return _AZIMUTH_GROUP


def _size(g):
    return 1 if (g is None or not dist.is_initialized()) else dist.get_world_size(group=g)


def _rank(g):
    return 0 if (g is None or not dist.is_initialized()) else dist.get_rank(group=g)


def polar_group_size():
    return _size(_POLAR_GROUP)


def azimuth_group_size():
    return _size(_AZIMUTH_GROUP)


def polar_group_rank():
    return _rank(_POLAR_GROUP)


def azimuth_group_rank():
    return _rank(_AZIMUTH_GROUP)


def compute_split_shapes(size, num_chunks):
    if num_chunks == 1:
        return [size]
    chunk = (size + num_chunks - 1) // num_chunks
    last = max(0, size - chunk * (num_chunks - 1))
    if last == 0:
        chunk = size // num_chunks
        last = size - chunk * (num_chunks - 1)
    return [chunk] * (num_chunks - 1) + [last]


def split_tensor_along_dim(tensor, dim, num_chunks):
    return list(torch.split(tensor, compute_split_shapes(tensor.shape[dim], num_chunks), dim=dim))


def _transpose(tensor, dim0, dim1, dim1_split_sizes, group=None):
    comm_size = dist.get_world_size(group=group)
    comm_rank = dist.get_rank(group=group)
    dim0_split_sizes = compute_split_shapes(tensor.shape[dim0], comm_size)
    x_send = [y.contiguous() for y in torch.split(tensor, dim0_split_sizes, dim=dim0)]
    x_shape = list(x_send[comm_rank].shape)
    x_recv = []
    for n in dim1_split_sizes:
        x_shape[dim1] = n
        x_recv.append(torch.empty(x_shape, dtype=tensor.dtype, device=tensor.device))
    dist.all_to_all(x_recv, x_send, group=group)
    return x_recv, dim0_split_sizes


class distributed_transpose_azimuth(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dims, dim1_split_sizes):
        xlist, dim0_split_sizes = _transpose(x, dims[0], dims[1], dim1_split_sizes, group=azimuth_group())
        ctx.dims, ctx.dim0_split_sizes = dims, dim0_split_sizes
        return torch.cat(xlist, dim=dims[1])

    @staticmethod
    def backward(ctx, go):
        dims = ctx.dims
        gilist, _ = _transpose(go, dims[1], dims[0], ctx.dim0_split_sizes, group=azimuth_group())
        return torch.cat(gilist, dim=dims[0]), None, None


class distributed_transpose_polar(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dims, dim1_split_sizes):
        xlist, dim0_split_sizes = _transpose(x, dims[0], dims[1], dim1_split_sizes, group=polar_group())
        ctx.dims, ctx.dim0_split_sizes = dims, dim0_split_sizes
        return torch.cat(xlist, dim=dims[1])

    @staticmethod
    def backward(ctx, go):
        dims = ctx.dims
        gilist, _ = _transpose(go, dims[1], dims[0], ctx.dim0_split_sizes, group=polar_group())
        return torch.cat(gilist, dim=dims[0]), None, None


class _Base(nn.Module):
    def _setup(self, nlat, nlon, lmax, mmax, grid, norm, csphase):
        self.nlat, self.nlon, self.grid, self.norm, self.csphase = nlat, nlon, grid, norm, csphase
        t, w, default_lmax = _grid(grid, nlat)
        self.lmax = lmax or default_lmax
        self.mmax = mmax or nlon // 2 + 1
        self.comm_size_polar, self.comm_rank_polar = polar_group_size(), polar_group_rank()
        self.comm_size_azimuth, self.comm_rank_azimuth = azimuth_group_size(), azimuth_group_rank()
        self.lat_shapes = compute_split_shapes(self.nlat, self.comm_size_polar)
        self.lon_shapes = compute_split_shapes(self.nlon, self.comm_size_azimuth)
        self.l_shapes = compute_split_shapes(self.lmax, self.comm_size_polar)
        self.m_shapes = compute_split_shapes(self.mmax, self.comm_size_azimuth)
        return t, w

    def _local_m(self, table):
        return split_tensor_along_dim(table, dim=0, num_chunks=self.comm_size_azimuth)[self.comm_rank_azimuth].contiguous()

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon},\n lmax={self.lmax}, mmax={self.mmax},\n grid={self.grid}, csphase={self.csphase}"


class DistributedRealSHT(_Base):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="lobatto", norm="ortho", csphase=True):
        super().__init__()
        tq, w = self._setup(nlat, nlon, lmax, mmax, grid, norm, csphase)
        pct = torch.from_numpy(precompute_legpoly(self.mmax, self.lmax, tq, norm=norm, csphase=csphase))
        weights = torch.einsum("mlk,k->mlk", pct, torch.from_numpy(w.copy()))
        self.register_buffer("weights", self._local_m(weights), persistent=False)

    def forward(self, x):
        num_chans = x.shape[1]
        if self.comm_size_azimuth > 1:
            x = distributed_transpose_azimuth.apply(x, (1, -1), self.lon_shapes)
        x = 2.0 * torch.pi * torch.fft.rfft(x, n=self.nlon, dim=-1, norm="forward")
        x = x[..., : self.mmax]
        if self.comm_size_azimuth > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_azimuth)
            x = distributed_transpose_azimuth.apply(x, (-1, 1), chan_shapes)
        if self.comm_size_polar > 1:
            x = distributed_transpose_polar.apply(x, (1, -2), self.lat_shapes)
        x = torch.view_as_real(x)
        out_shape = list(x.size())
        out_shape[-3] = self.lmax
        xout = torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        xout[..., 0] = torch.einsum("...km,mlk->...lm", x[..., 0], self.weights.to(x.dtype))
        xout[..., 1] = torch.einsum("...km,mlk->...lm", x[..., 1], self.weights.to(x.dtype))
        x = torch.view_as_complex(xout)
        if self.comm_size_polar > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_polar)
            x = distributed_transpose_polar.apply(x, (-2, 1), chan_shapes)
        return x


class DistributedInverseRealSHT(_Base):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="lobatto", norm="ortho", csphase=True):
        super().__init__()
        t, _ = self._setup(nlat, nlon, lmax, mmax, grid, norm, csphase)
        pct = torch.from_numpy(precompute_legpoly(self.mmax, self.lmax, t, norm=norm, inverse=True, csphase=csphase))
        self.register_buffer("pct", self._local_m(pct), persistent=False)

    def forward(self, x):
        num_chans = x.shape[1]
        if self.comm_size_polar > 1:
            x = distributed_transpose_polar.apply(x, (1, -2), self.l_shapes)
        x = torch.view_as_real(x)
        rl = torch.einsum("...lm, mlk->...km", x[..., 0], self.pct.to(x.dtype))
        im = torch.einsum("...lm, mlk->...km", x[..., 1], self.pct.to(x.dtype))
        x = torch.view_as_complex(torch.stack((rl, im), -1).contiguous())
        if self.comm_size_polar > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_polar)
            x = distributed_transpose_polar.apply(x, (-2, 1), chan_shapes)
        if self.comm_size_azimuth > 1:
            x = distributed_transpose_azimuth.apply(x, (1, -1), self.m_shapes)
        x = torch.fft.irfft(x, n=self.nlon, dim=-1, norm="forward")
        if self.comm_size_azimuth > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_azimuth)
            x = distributed_transpose_azimuth.apply(x, (-1, 1), chan_shapes)
        return x
