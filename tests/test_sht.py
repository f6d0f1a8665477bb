"""Spherical harmonic transform oracles: analytic identities of the fp64 formulation, and the GEMM-chain
formulation (run through the CPU emulation of the kernel addressing) against it."""

import math

import numpy as np
import pytest
import torch

from makani_b200.ops.spectral import SHTPlan, spectral_conv_dhconv
from makani_b200.sht import InverseRealSHT, RealSHT, legendre_table, precompute_latitudes
from makani_b200.sht.quadrature import clenshaw_curtiss_weights, legendre_gauss_weights, lobatto_weights


def _f64(nlat, nlon, lmax, mmax, grid):
    sht = RealSHT(nlat, nlon, lmax, mmax, grid)
    isht = InverseRealSHT(nlat, nlon, lmax, mmax, grid)
    th, w = precompute_latitudes(nlat, grid)
    p = legendre_table(mmax, lmax, th)
    sht.weights = torch.from_numpy(p * w[None, None, :])
    isht.pct = torch.from_numpy(p)
    return sht, isht, w


@pytest.mark.parametrize("rule,n", [(legendre_gauss_weights, 20), (clenshaw_curtiss_weights, 21), (lobatto_weights, 12)])
def test_quadrature_integrates_polynomials(rule, n):
    x, w = rule(n)
    assert abs(w.sum() - 2.0) < 1e-12
    assert abs((w * x ** 2).sum() - 2.0 / 3.0) < 1e-10
    assert abs((w * x ** 4).sum() - 2.0 / 5.0) < 1e-10
    assert np.all(np.diff(x) > 0)


@pytest.mark.parametrize("grid,nlat", [("legendre-gauss", 32), ("equiangular", 33)])
def test_sht_of_constant_and_roundtrip(grid, nlat):
    nlon, L, M = 64, 20, 21
    sht, isht, w = _f64(nlat, nlon, L, M, grid)
    c = sht(torch.ones(1, nlat, nlon, dtype=torch.float64))
    assert abs(c[0, 0, 0].real.item() - math.sqrt(4 * math.pi)) < 1e-10
    assert (c.abs().sum() - c[0, 0, 0].abs()).item() < 1e-10
    torch.manual_seed(0)
    cr = torch.randn(2, L, M, dtype=torch.complex128)
    l, m = torch.arange(L)[:, None], torch.arange(M)[None, :]
    cr = cr * (l >= m)
    cr[..., 0] = cr[..., 0].real + 0j
    x = isht(cr)
    if grid == "legendre-gauss":
        assert (sht(x) - cr).abs().max().item() < 1e-11
        qw = torch.from_numpy(w)[:, None] * (2 * math.pi / nlon)
        lhs = (x ** 2 * qw).sum(dim=(-1, -2))
        rhs = (cr[..., 0].abs() ** 2).sum(-1) + 2 * (cr[..., 1:].abs() ** 2).sum(dim=(-1, -2))
        assert torch.allclose(lhs, rhs, rtol=1e-10)


def test_longitude_rotation_multiplies_by_phase():
    nlat, nlon, L, M = 16, 32, 12, 13
    sht, isht, _ = _f64(nlat, nlon, L, M, "legendre-gauss")
    torch.manual_seed(1)
    x = torch.randn(1, nlat, nlon, dtype=torch.float64)
    c0 = sht(x)
    shift = 5
    c1 = sht(torch.roll(x, shifts=shift, dims=-1))
    m = torch.arange(M, dtype=torch.float64)
    phase = torch.exp(-1j * m * (2 * math.pi * shift / nlon))
    assert (c1 - c0 * phase).abs().max().item() < 1e-10


@pytest.mark.parametrize("B,C,Co", [(2, 4, 8), (1, 8, 4)])
def test_gemm_chain_matches_reference_forward_and_backward(B, C, Co):
    dt = torch.float64
    nlat, nlon, L, M = 33, 64, 16, 17
    nlat2, nlon2 = 16, 32
    pin = SHTPlan(nlat, nlon, L, M, "equiangular", "cpu", dt)
    pout = SHTPlan(nlat2, nlon2, L, M, "legendre-gauss", "cpu", dt)
    sht = RealSHT(nlat, nlon, L, M, "equiangular").double()
    isht = InverseRealSHT(nlat2, nlon2, L, M, "legendre-gauss").double()
    torch.manual_seed(2)
    x = torch.randn(B, C, nlat, nlon, dtype=dt, requires_grad=True)
    w = torch.randn(C, Co, L, dtype=torch.complex128, requires_grad=True)
    y, r = spectral_conv_dhconv(x, w, pin, pout, True)
    c = sht(x)
    yref = isht(torch.einsum("bixy,iox->boxy", c, w))
    rref = isht(c)
    assert (y - yref).abs().max().item() < 1e-5
    assert (r - rref).abs().max().item() < 1e-5
    gy, gr = torch.randn_like(yref), torch.randn_like(rref)
    gx, gw = torch.autograd.grad([y, r], [x, w], [gy, gr])
    gx2, gw2 = torch.autograd.grad([yref, rref], [x, w], [gy, gr])
    assert (gx - gx2).abs().max().item() < 1e-5
    assert (gw - gw2).abs().max().item() < 1e-4
