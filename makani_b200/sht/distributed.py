"""Spatially distributed spherical harmonic transforms (portable all-to-all formulation).

Grid data [B, C, nlat_loc, nlon_loc] is sharded in latitude over the polar group "h" and in longitude over the
azimuth group "w"; coefficients [B, C, l_loc, m_loc] are sharded l over "h" and m over "w".  Choreography
(the one torch-harmonics' DistributedRealSHT follows, mirrored in-tree by makani/mpu/layers.py:66-101 for
the FFT case): transpose(w): channels <-> longitude, DFT, truncate, transpose(w) back: m <-> channels,
transpose(h): channels <-> latitude, Legendre quadrature with this rank's m-slice of the table,
transpose(h) back: l <-> channels.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn as nn

from ..parallel.helpers import compute_split_shapes
from ..parallel.transpose import distributed_transpose_azimuth, distributed_transpose_polar
from ..utils import comm
from .legendre import legendre_table
from .quadrature import precompute_latitudes


class _DistBase(nn.Module):
    def __init__(self, nlat, nlon, lmax, mmax, grid, csphase):
        super().__init__()
        self.nlat, self.nlon, self.grid, self.csphase = nlat, nlon, grid, csphase
        self.lmax = lmax or (nlat - 1 if grid == "lobatto" else nlat)
        self.mmax = mmax or (nlon // 2 + 1)
        self.comm_size_polar = comm.get_size("h")
        self.comm_rank_polar = comm.get_rank("h")
        self.comm_size_azimuth = comm.get_size("w")
        self.comm_rank_azimuth = comm.get_rank("w")
        self.lat_shapes = compute_split_shapes(self.nlat, self.comm_size_polar)
        self.lon_shapes = compute_split_shapes(self.nlon, self.comm_size_azimuth)
        self.l_shapes = compute_split_shapes(self.lmax, self.comm_size_polar)
        self.m_shapes = compute_split_shapes(self.mmax, self.comm_size_azimuth)
        m0 = sum(self.m_shapes[: self.comm_rank_azimuth])
        self.m_slice = slice(m0, m0 + self.m_shapes[self.comm_rank_azimuth])

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon}, lmax={self.lmax}, mmax={self.mmax}, grid={self.grid}"


class DistributedRealSHT(_DistBase):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, csphase)
        theta, w = precompute_latitudes(nlat, grid)
        p = legendre_table(self.mmax, self.lmax, theta, csphase=csphase) * w[None, None, :]
        self.register_buffer("weights", torch.from_numpy(p[self.m_slice]).float().contiguous(), persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        num_chans = x.shape[1]
        if self.comm_size_azimuth > 1:
            x = distributed_transpose_azimuth(x, (1, -1), self.lon_shapes)
        x = 2.0 * np.pi * torch.fft.rfft(x, n=self.nlon, dim=-1, norm="forward")[..., : self.mmax]
        if self.comm_size_azimuth > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_azimuth)
            x = distributed_transpose_azimuth(x.contiguous(), (-1, 1), chan_shapes)
        if self.comm_size_polar > 1:
            x = distributed_transpose_polar(x, (1, -2), self.lat_shapes)
        w = self.weights.to(x.real.dtype)
        x = torch.complex(torch.einsum("...km,mlk->...lm", x.real, w), torch.einsum("...km,mlk->...lm", x.imag, w))
        if self.comm_size_polar > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_polar)
            x = distributed_transpose_polar(x.contiguous(), (-2, 1), chan_shapes)
        return x


class DistributedInverseRealSHT(_DistBase):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__(nlat, nlon, lmax, mmax, grid, csphase)
        theta, _ = precompute_latitudes(nlat, grid)
        p = legendre_table(self.mmax, self.lmax, theta, csphase=csphase)
        self.register_buffer("pct", torch.from_numpy(p[self.m_slice]).float().contiguous(), persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        num_chans = x.shape[1]
        if self.comm_size_polar > 1:
            x = distributed_transpose_polar(x, (1, -2), self.l_shapes)
        p = self.pct.to(x.real.dtype)
        x = torch.complex(torch.einsum("...lm,mlk->...km", x.real, p), torch.einsum("...lm,mlk->...km", x.imag, p))
        if self.comm_size_polar > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_polar)
            x = distributed_transpose_polar(x.contiguous(), (-2, 1), chan_shapes)
        if self.comm_size_azimuth > 1:
            x = distributed_transpose_azimuth(x, (1, -1), self.m_shapes)
        x = torch.fft.irfft(x, n=self.nlon, dim=-1, norm="forward")
        if self.comm_size_azimuth > 1:
            chan_shapes = compute_split_shapes(num_chans, self.comm_size_azimuth)
            x = distributed_transpose_azimuth(x.contiguous(), (-1, 1), chan_shapes)
        return x
