"""Serial real SHT / inverse SHT modules (grid `[..., nlat, nlon]` <-> complex coefficients `[..., lmax, mmax]`)."""

import numpy as np
import torch
import torch.nn as nn

from .legendre import precompute_legpoly
from .quadrature import clenshaw_curtiss_weights, legendre_gauss_weights, lobatto_weights


def _grid(grid, nlat):
    if grid == "legendre-gauss":
        cost, w = legendre_gauss_weights(nlat, -1, 1)
        lmax = nlat
    elif grid == "lobatto":
        cost, w = lobatto_weights(nlat, -1, 1)
        lmax = nlat - 1
    elif grid == "equiangular":
        cost, w = clenshaw_curtiss_weights(nlat, -1, 1)
        lmax = nlat
    else:
        raise ValueError("Unknown quadrature mode")
    return np.flip(np.arccos(cost)), w, lmax


class RealSHT(nn.Module):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="lobatto", norm="ortho", csphase=True):
        super().__init__()
        self.nlat, self.nlon, self.grid, self.norm, self.csphase = nlat, nlon, grid, norm, csphase
        tq, w, default_lmax = _grid(grid, nlat)
        self.lmax = lmax or default_lmax
        self.mmax = mmax or self.nlon // 2 + 1
        pct = torch.from_numpy(precompute_legpoly(self.mmax, self.lmax, tq, norm=norm, csphase=csphase))
        weights = torch.einsum("mlk,k->mlk", pct, torch.from_numpy(w.copy()))
        self.register_buffer("weights", weights, persistent=False)

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon},\n lmax={self.lmax}, mmax={self.mmax},\n grid={self.grid}, csphase={self.csphase}"

    def forward(self, x):
        assert x.shape[-2] == self.nlat
        assert x.shape[-1] == self.nlon
        x = 2.0 * torch.pi * torch.fft.rfft(x, dim=-1, norm="forward")
        x = torch.view_as_real(x)
        out_shape = list(x.size())
        out_shape[-3] = self.lmax
        out_shape[-2] = self.mmax
        xout = torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        xout[..., 0] = torch.einsum("...km,mlk->...lm", x[..., : self.mmax, 0], self.weights.to(x.dtype))
        xout[..., 1] = torch.einsum("...km,mlk->...lm", x[..., : self.mmax, 1], self.weights.to(x.dtype))
        return torch.view_as_complex(xout)


class InverseRealSHT(nn.Module):
    def __init__(self, nlat, nlon, lmax=None, mmax=None, grid="lobatto", norm="ortho", csphase=True):
        super().__init__()
        self.nlat, self.nlon, self.grid, self.norm, self.csphase = nlat, nlon, grid, norm, csphase
        t, _, default_lmax = _grid(grid, nlat)
        self.lmax = lmax or default_lmax
        self.mmax = mmax or self.nlon // 2 + 1
        pct = torch.from_numpy(precompute_legpoly(self.mmax, self.lmax, t, norm=norm, inverse=True, csphase=csphase))
        self.register_buffer("pct", pct, persistent=False)

    def extra_repr(self):
        return f"nlat={self.nlat}, nlon={self.nlon},\n lmax={self.lmax}, mmax={self.mmax},\n grid={self.grid}, csphase={self.csphase}"

    def forward(self, x):
        assert x.shape[-2] == self.lmax
        assert x.shape[-1] == self.mmax
        x = torch.view_as_real(x)
        rl = torch.einsum("...lm, mlk->...km", x[..., 0], self.pct.to(x.dtype))
        im = torch.einsum("...lm, mlk->...km", x[..., 1], self.pct.to(x.dtype))
        x = torch.view_as_complex(torch.stack((rl, im), -1))
        return torch.fft.irfft(x, n=self.nlon, dim=-1, norm="forward")
