"""3-D real FFT wrappers (depth, latitude, longitude) in local and spatially distributed form.

Contract: makani/mpu/fft3d.py:13-273 — `RealFFT3` / `InverseRealFFT3` (rfftn over the last three dims with
truncation to (ldmax, lhmax, lwmax) modes, keeping low and high frequencies of the two complex dimensions) and
`DistributedRealFFT3` / `DistributedInverseRealFFT3`, which shard (h, w) over the ("h", "w") groups and keep the
depth dimension local, using the same transpose choreography as the 2-D transform.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils import comm
from .helpers import compute_split_shapes
from .transpose import distributed_transpose_azimuth, distributed_transpose_polar


def _keep_low_high(x, n_keep, dim):
    hi, lo = math.ceil(n_keep / 2), math.floor(n_keep / 2)
    parts = [x.narrow(dim, 0, hi)]
    if lo > 0:
        parts.append(x.narrow(dim, x.shape[dim] - lo, lo))
    return torch.cat(parts, dim=dim)


def _pad_low_high(x, n_keep, n_full, dim):
    hi, lo = math.ceil(n_keep / 2), math.floor(n_keep / 2)
    shape = list(x.shape)
    shape[dim] = n_full - n_keep
    parts = [x.narrow(dim, 0, hi), torch.zeros(shape, dtype=x.dtype, device=x.device)]
    if lo > 0:
        parts.append(x.narrow(dim, x.shape[dim] - lo, lo))
    return torch.cat(parts, dim=dim)


class RealFFT3(nn.Module):
    def __init__(self, nd, nh, nw, ldmax=None, lhmax=None, lwmax=None):
        super().__init__()
        self.nd, self.nh, self.nw = nd, nh, nw
        self.ldmax = min(ldmax or nd, nd)
        self.lhmax = min(lhmax or nh, nh)
        self.lwmax = min(lwmax or nw // 2 + 1, nw // 2 + 1)

    def forward(self, x):
        y = torch.fft.rfftn(x, s=(self.nd, self.nh, self.nw), dim=(-3, -2, -1), norm="ortho")
        y = _keep_low_high(y, self.ldmax, -3)
        y = _keep_low_high(y, self.lhmax, -2)
        return y[..., : self.lwmax].contiguous()


class InverseRealFFT3(nn.Module):
    def __init__(self, nd, nh, nw, ldmax=None, lhmax=None, lwmax=None):
        super().__init__()
        self.nd, self.nh, self.nw = nd, nh, nw
        self.ldmax = min(ldmax or nd, nd)
        self.lhmax = min(lhmax or nh, nh)
        self.lwmax = min(lwmax or nw // 2 + 1, nw // 2 + 1)

    def forward(self, x):
        x = x[..., : self.lwmax]
        x = _pad_low_high(x, self.lhmax, self.nh, x.dim() - 2)
        x = _pad_low_high(x, self.ldmax, self.nd, x.dim() - 3)
        return torch.fft.irfftn(x, s=(self.nd, self.nh, self.nw), dim=(-3, -2, -1), norm="ortho")


class DistributedRealFFT3(nn.Module):
    """Input [B, C, D, H_loc, W_loc]; output [B, C, ldmax, lh_loc, lw_loc]."""

    def __init__(self, nd, nh, nw, ldmax=None, lhmax=None, lwmax=None):
        super().__init__()
        self.comm_size_h, self.comm_size_w = comm.get_size("h"), comm.get_size("w")
        self.nd, self.nh, self.nw = nd, nh, nw
        self.ldmax = min(ldmax or nd, nd)
        self.lhmax = min(lhmax or nh, nh)
        self.lwmax = min(lwmax or nw // 2 + 1, nw // 2 + 1)
        self.lat_shapes = compute_split_shapes(nh, self.comm_size_h)
        self.lon_shapes = compute_split_shapes(nw, self.comm_size_w)
        self.l_shapes = compute_split_shapes(self.lhmax, self.comm_size_h)
        self.m_shapes = compute_split_shapes(self.lwmax, self.comm_size_w)

    def forward(self, x):
        num_chans = x.shape[1]
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x, (1, -1), self.lon_shapes)
        x = torch.fft.rfft(x, n=self.nw, dim=-1, norm="ortho")[..., : self.lwmax]
        x = _keep_low_high(torch.fft.fft(x, n=self.nd, dim=-3, norm="ortho"), self.ldmax, x.dim() - 3)
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x.contiguous(), (-1, 1), compute_split_shapes(num_chans, self.comm_size_w))
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x, (1, -2), self.lat_shapes)
        x = _keep_low_high(torch.fft.fft(x, n=self.nh, dim=-2, norm="ortho"), self.lhmax, x.dim() - 2)
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x.contiguous(), (-2, 1), compute_split_shapes(num_chans, self.comm_size_h))
        return x


class DistributedInverseRealFFT3(nn.Module):
    def __init__(self, nd, nh, nw, ldmax=None, lhmax=None, lwmax=None):
        super().__init__()
        self.comm_size_h, self.comm_size_w = comm.get_size("h"), comm.get_size("w")
        self.nd, self.nh, self.nw = nd, nh, nw
        self.ldmax = min(ldmax or nd, nd)
        self.lhmax = min(lhmax or nh, nh)
        self.lwmax = min(lwmax or nw // 2 + 1, nw // 2 + 1)
        self.lat_shapes = compute_split_shapes(nh, self.comm_size_h)
        self.lon_shapes = compute_split_shapes(nw, self.comm_size_w)
        self.l_shapes = compute_split_shapes(self.lhmax, self.comm_size_h)
        self.m_shapes = compute_split_shapes(self.lwmax, self.comm_size_w)

    def forward(self, x):
        num_chans = x.shape[1]
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x, (1, -2), self.l_shapes)
        x = torch.fft.ifft(_pad_low_high(x, self.lhmax, self.nh, x.dim() - 2), n=self.nh, dim=-2, norm="ortho")
        if self.comm_size_h > 1:
            x = distributed_transpose_polar(x.contiguous(), (-2, 1), compute_split_shapes(num_chans, self.comm_size_h))
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x, (1, -1), self.m_shapes)
        x = torch.fft.ifft(_pad_low_high(x, self.ldmax, self.nd, x.dim() - 3), n=self.nd, dim=-3, norm="ortho")
        x = torch.fft.irfft(x, n=self.nw, dim=-1, norm="ortho")
        if self.comm_size_w > 1:
            x = distributed_transpose_azimuth(x.contiguous(), (-1, 1), compute_split_shapes(num_chans, self.comm_size_w))
        return x
