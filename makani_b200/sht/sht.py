"""Real spherical harmonic transforms (analysis / synthesis) and their spatially distributed variants.

`RealSHT` / `InverseRealSHT` reproduce the contract of the torch-harmonics objects the reference builds at
makani/models/networks/sfnonet.py:523-539 (attributes nlat, nlon, lmax, mmax, grid; complex output
[..., lmax, mmax]; "ortho" normalisation with Condon-Shortley phase; a forward and an inverse object may sit
on different grids with the same (lmax, mmax)).  This module is the exact-precision formulation (fp32/fp64
DFT + Legendre quadrature) used on CPU, for oracles and off the hot path; the bf16 tensor-core pipeline used
inside the SFNO blocks lives in `makani_b200.ops.spectral`.

`DistributedRealSHT` / `DistributedInverseRealSHT` shard latitude over the polar ("h") group and longitude
over the azimuth ("w") group, coefficients l over h and m over w (torch-harmonics' distributed SHT as used at
makani/models/networks/sfnonet.py:528-533), using the transposes of `makani_b200.parallel.transpose`.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn as nn

from .legendre import legendre_table
from .quadrature import precompute_latitudes


def _default_lmax(nlat: int, grid: str) -> int:
    return nlat - 1 if grid == "lobatto" else nlat


class RealSHT(nn.Module):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__()
        assert norm == "ortho", "only the orthonormal convention is used by the networks"
        self.nlat, self.nlon, self.grid, self.norm, self.csphase = nlat, nlon, grid, norm, csphase
        self.lmax = lmax or _default_lmax(nlat, grid)
        self.mmax = mmax or (nlon // 2 + 1)
        theta, w = precompute_latitudes(nlat, grid)
        p = legendre_table(self.mmax, self.lmax, theta, csphase=csphase)
        weights = torch.from_numpy(p * w[None, None, :])
        self.register_buffer("weights", weights.float(), persistent=False)

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon}, lmax={self.lmax}, mmax={self.mmax}, grid={self.grid}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        assert x.shape[-2] == self.nlat and x.shape[-1] == self.nlon
        xf = 2.0 * np.pi * torch.fft.rfft(x, dim=-1, norm="forward")[..., : self.mmax]
        w = self.weights.to(xf.real.dtype)
        re = torch.einsum("...km,mlk->...lm", xf.real, w)
        im = torch.einsum("...km,mlk->...lm", xf.imag, w)
        return torch.complex(re, im)


class InverseRealSHT(nn.Module):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="equiangular", norm="ortho", csphase=True):
        super().__init__()
        assert norm == "ortho"
        self.nlat, self.nlon, self.grid, self.norm, self.csphase = nlat, nlon, grid, norm, csphase
        self.lmax = lmax or _default_lmax(nlat, grid)
        self.mmax = mmax or (nlon // 2 + 1)
        theta, _ = precompute_latitudes(nlat, grid)
        p = legendre_table(self.mmax, self.lmax, theta, csphase=csphase)
        self.register_buffer("pct", torch.from_numpy(p).float(), persistent=False)

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon}, lmax={self.lmax}, mmax={self.mmax}, grid={self.grid}"

    def forward(self, c: torch.Tensor) -> torch.Tensor:
        assert c.shape[-2] == self.lmax and c.shape[-1] == self.mmax
        p = self.pct.to(c.real.dtype)
        re = torch.einsum("...lm,mlk->...km", c.real, p)
        im = torch.einsum("...lm,mlk->...km", c.imag, p)
        xf = torch.complex(re, im)
        return torch.fft.irfft(xf, n=self.nlon, dim=-1, norm="forward")
