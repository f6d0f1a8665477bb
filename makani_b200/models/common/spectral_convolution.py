"""Spectral (Fourier / spherical-harmonic) convolution layers.

`SpectralConv` applies a learnable complex filter in the spectral domain of a transform pair
(forward on the input grid, inverse on the output grid) and returns `(y, residual)` where the residual is the
input re-gridded through `inverse(forward(x))` whenever the two grids differ.  Parameter names, shapes,
initialisation and sharding tags follow makani/models/common/spectral_convolution.py:43-148 (weight:
complex64 `[Cin, (Cout), l_loc(, m_loc)]`, std sqrt(gain/Cin), l = 0 row scaled by sqrt(2)).

Execution: for the per-degree ("dhconv") operator on CUDA bf16 input with local SHTs the whole layer runs as
the GEMM chain of `makani_b200.ops.spectral` (no cuFFT / cuBLAS); every other combination uses the exact
fp32 transform modules and einsum contractions.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ...ops import spectral as spectral_ops
from ...ops import spectral_dist as spectral_dist_ops
from ...sht import DistributedInverseRealSHT, DistributedRealSHT, InverseRealSHT, RealSHT
from ...utils import comm
from .activations import ComplexReLU
from .contractions import (compl_exp_mul2d_fwd, compl_exp_muladd2d_fwd, compl_mul2d_fwd, compl_muladd2d_fwd,
                           get_contract_fun)
from .factorizations import FactorizedWeight


def _grids_differ(fwd, inv) -> bool:
    diff = (fwd.nlat != inv.nlat) or (fwd.nlon != inv.nlon)
    if hasattr(fwd, "grid") and hasattr(inv, "grid"):
        diff = diff or (fwd.grid != inv.grid)
    return diff


def _local_modes(inverse_transform):
    if isinstance(inverse_transform, DistributedInverseRealSHT) or hasattr(inverse_transform, "l_shapes"):
        return (inverse_transform.l_shapes[comm.get_rank("h")], inverse_transform.m_shapes[comm.get_rank("w")],
                inverse_transform.lat_shapes[comm.get_rank("h")], inverse_transform.lon_shapes[comm.get_rank("w")])
    return inverse_transform.lmax, inverse_transform.mmax, inverse_transform.nlat, inverse_transform.nlon


class SpectralConv(nn.Module):
    def __init__(self, forward_transform, inverse_transform, in_channels, out_channels, operator_type="diagonal",
                 separable=False, bias=False, gain=1.0):
        super().__init__()
        self.forward_transform = forward_transform
        self.inverse_transform = inverse_transform
        self.in_channels, self.out_channels = in_channels, out_channels
        self.modes_lat, self.modes_lon = inverse_transform.lmax, inverse_transform.mmax
        self.scale_residual = _grids_differ(forward_transform, inverse_transform)
        self.operator_type, self.separable = operator_type, separable
        self.modes_lat_local, self.modes_lon_local, self.nlat_local, self.nlon_local = _local_modes(inverse_transform)

        shape = [in_channels] + ([] if separable else [out_channels])
        if operator_type == "diagonal":
            shape += [self.modes_lat_local, self.modes_lon_local]
        elif operator_type == "dhconv":
            shape += [self.modes_lat_local]
        else:
            raise ValueError(f"Unsupported operator type {operator_type}")
        scale = math.sqrt(gain / in_channels) * torch.ones(self.modes_lat_local, dtype=torch.complex64)
        scale[0] *= math.sqrt(2.0)
        if operator_type == "diagonal":
            scale = scale.unsqueeze(-1)
        self.weight = nn.Parameter(scale * torch.randn(*shape, dtype=torch.complex64))
        if operator_type == "dhconv":
            self.weight.is_shared_mp = ["matmul", "w"]
            self.weight.sharded_dims_mp = [None] * (len(shape) - 1) + ["h"]
        else:
            self.weight.is_shared_mp = ["matmul"]
            self.weight.sharded_dims_mp = [None] * (len(shape) - 2) + ["h", "w"]
        self._contract = get_contract_fun(operator_type, separable)

        if bias == "constant":
            self.bias = nn.Parameter(torch.zeros(1, out_channels, 1, 1))
        elif bias == "position":
            self.bias = nn.Parameter(torch.zeros(1, out_channels, self.nlat_local, self.nlon_local))
            self.bias.is_shared_mp = ["matmul"]
            self.bias.sharded_dims_mp = [None, None, "h", "w"]

    # ---- tensor-core path --------------------------------------------------------------------------
    def _fast_ok(self, x) -> bool:
        return (x.is_cuda and self.operator_type == "dhconv" and not self.separable
                and type(self.forward_transform) is RealSHT and type(self.inverse_transform) is InverseRealSHT
                and spectral_ops.spectral_conv_supported(x, self.weight))

    def _fast_dist_ok(self, x) -> bool:
        """Sharded grids: GEMM chain whose k loops read the peers' buffers directly (needs peer-mapped memory, i.e.
        NCCL ranks on one node, and l/m truncations common to both transforms)."""
        f, i = self.forward_transform, self.inverse_transform
        return (x.is_cuda and spectral_dist_ops.ENABLED and self.operator_type == "dhconv" and not self.separable
                and type(f) is DistributedRealSHT and type(i) is DistributedInverseRealSHT
                and f.lmax == i.lmax and f.mmax == i.mmax and comm.get_size("h") * comm.get_size("w") <= 8
                and spectral_dist_ops.dist_spectral_conv_supported(x, self.weight))

    def _dist_plans(self, device, dtype):
        f, i = self.forward_transform, self.inverse_transform
        ph, pw, rh, rw = comm.get_size("h"), comm.get_size("w"), comm.get_rank("h"), comm.get_rank("w")
        return (spectral_dist_ops.DistSHTPlan.get(f.nlat, f.nlon, f.lmax, f.mmax, f.grid, ph, pw, rh, rw, device, dtype),
                spectral_dist_ops.DistSHTPlan.get(i.nlat, i.nlon, i.lmax, i.mmax, i.grid, ph, pw, rh, rw, device, dtype))

    def _plans(self, device, dtype):
        f, i = self.forward_transform, self.inverse_transform
        return (spectral_ops.SHTPlan.get(f.nlat, f.nlon, f.lmax, f.mmax, f.grid, device, dtype),
                spectral_ops.SHTPlan.get(i.nlat, i.nlon, i.lmax, i.mmax, i.grid, device, dtype))

    def forward(self, x):
        if self._fast_ok(x):
            pin, pout = self._plans(x.device, x.dtype)
            if self.scale_residual:
                y, residual = spectral_ops.spectral_conv_dhconv(x, self.weight, pin, pout, True)
            else:
                y, residual = spectral_ops.spectral_conv_dhconv(x, self.weight, pin, pout, False), x
            if hasattr(self, "bias"):
                y = y + self.bias.to(y.dtype)
            return y, residual
        if self._fast_dist_ok(x):
            pin, pout = self._dist_plans(x.device, x.dtype)
            if self.scale_residual:
                y, residual = spectral_dist_ops.dist_spectral_conv_dhconv(x, self.weight, pin, pout, True)
            else:
                y, residual = spectral_dist_ops.dist_spectral_conv_dhconv(x, self.weight, pin, pout, False), x
            if hasattr(self, "bias"):
                y = y + self.bias.to(y.dtype)
            return y, residual

        dtype = x.dtype
        residual = x
        x = x.float()
        with torch.autocast(device_type=x.device.type, enabled=False):
            x = self.forward_transform(x).contiguous()
            if self.scale_residual:
                residual = self.inverse_transform(x).to(dtype)
        x = self._contract(x, self.weight).contiguous()
        with torch.autocast(device_type=x.device.type, enabled=False):
            x = self.inverse_transform(x)
        if hasattr(self, "bias"):
            x = x + self.bias
        return x.to(dtype), residual


class FactorizedSpectralConv(nn.Module):
    """Spectral convolution whose weight is held in a low-rank factorisation (dense/CP/Tucker/TT)."""

    def __init__(self, forward_transform, inverse_transform, in_channels, out_channels, operator_type="diagonal",
                 rank=0.2, factorization=None, separable=False, decomposition_kwargs=None, bias=False, gain=1.0):
        super().__init__()
        self.forward_transform, self.inverse_transform = forward_transform, inverse_transform
        self.in_channels, self.out_channels = in_channels, out_channels
        self.modes_lat, self.modes_lon = inverse_transform.lmax, inverse_transform.mmax
        self.scale_residual = _grids_differ(forward_transform, inverse_transform)
        self.operator_type, self.separable = operator_type, separable
        self.rank = rank
        self.modes_lat_local, self.modes_lon_local, self.nlat_local, self.nlon_local = _local_modes(inverse_transform)
        factorization = factorization or "ComplexDense"
        if not factorization.lower().startswith("complex"):
            factorization = f"Complex{factorization}"
        shape = [in_channels] + ([] if separable else [out_channels])
        if operator_type == "diagonal":
            shape += [self.modes_lat_local, self.modes_lon_local]
        elif operator_type == "dhconv":
            shape += [self.modes_lat_local]
        else:
            raise ValueError(f"Unsupported operator type {operator_type}")
        self.weight = FactorizedWeight(shape, rank=rank, factorization=factorization, init_std=math.sqrt(gain / in_channels))
        for p in self.weight.parameters():
            p.is_shared_mp = ["matmul", "w"] if operator_type == "dhconv" else ["matmul"]
        self._contract = get_contract_fun(operator_type, separable)
        if bias == "constant":
            self.bias = nn.Parameter(torch.zeros(1, out_channels, 1, 1))
        elif bias == "position":
            self.bias = nn.Parameter(torch.zeros(1, out_channels, self.nlat_local, self.nlon_local))
            self.bias.is_shared_mp = ["matmul"]
            self.bias.sharded_dims_mp = [None, None, "h", "w"]

    def forward(self, x):
        dtype = x.dtype
        residual = x
        x = x.float()
        with torch.autocast(device_type=x.device.type, enabled=False):
            x = self.forward_transform(x).contiguous()
            if self.scale_residual:
                residual = self.inverse_transform(x).to(dtype)
        x = self._contract(x, self.weight.to_tensor()).contiguous()
        with torch.autocast(device_type=x.device.type, enabled=False):
            x = self.inverse_transform(x)
        if hasattr(self, "bias"):
            x = x + self.bias
        return x.to(dtype), residual


class SpectralAttention(nn.Module):
    """Non-linear spectral filter: a complex MLP applied mode-wise in the spectral domain."""

    def __init__(self, forward_transform, inverse_transform, in_channels, out_channels, operator_type="diagonal",
                 hidden_size_factor=2, complex_activation="real", bias=False, spectral_layers=1, drop_rate=0.0, gain=1.0):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.operator_type, self.spectral_layers = operator_type, spectral_layers
        self.modes_lat, self.modes_lon = forward_transform.lmax, forward_transform.mmax
        self.forward_transform, self.inverse_transform = forward_transform, inverse_transform
        self.scale_residual = _grids_differ(forward_transform, inverse_transform)
        assert inverse_transform.lmax == self.modes_lat and inverse_transform.mmax == self.modes_lon
        hidden = int(hidden_size_factor * in_channels)
        if operator_type == "diagonal":
            self.mul_add_handle, self.mul_handle = compl_muladd2d_fwd, compl_mul2d_fwd
            lead = []
        elif operator_type == "l-dependant":
            self.mul_add_handle, self.mul_handle = compl_exp_muladd2d_fwd, compl_exp_mul2d_fwd
            lead = [self.modes_lat]
        else:
            raise ValueError("Unknown operator type")
        w = [math.sqrt(2.0 / in_channels) * torch.randn(*lead, in_channels, hidden, dtype=torch.complex64)]
        for _ in range(1, spectral_layers):
            w.append(math.sqrt(2.0 / hidden) * torch.randn(*lead, hidden, hidden, dtype=torch.complex64))
        self.w = nn.ParameterList([nn.Parameter(t) for t in w])
        scale = math.sqrt(gain / in_channels)
        self.wout = nn.Parameter(scale * torch.randn(*lead, hidden, out_channels, dtype=torch.complex64))
        if bias:
            self.b = nn.ParameterList([nn.Parameter(scale * torch.randn(hidden, 1, 1, dtype=torch.complex64))
                                       for _ in range(spectral_layers)])
        self.activations = nn.ModuleList([ComplexReLU(mode=complex_activation, bias_shape=(hidden, 1, 1), scale=scale)
                                          for _ in range(spectral_layers)])
        self.drop = nn.Dropout(drop_rate) if drop_rate > 0.0 else nn.Identity()

    def forward_mlp(self, x):
        xr = torch.view_as_real(x)
        for l in range(self.spectral_layers):
            if hasattr(self, "b"):
                xr = self.mul_add_handle(xr, self.w[l], self.b[l])
            else:
                xr = self.mul_handle(xr, self.w[l])
            xc = self.activations[l](torch.view_as_complex(xr.contiguous()))
            xr = torch.view_as_real(xc)
            xr = self.drop(xr)
        return torch.view_as_complex(self.mul_handle(xr, self.wout).contiguous())

    def forward(self, x):
        dtype = x.dtype
        residual = x
        x = x.float()
        with torch.autocast(device_type=x.device.type, enabled=False):
            x = self.forward_transform(x)
            if self.scale_residual:
                residual = self.inverse_transform(x).to(dtype)
        x = self.forward_mlp(x)
        with torch.autocast(device_type=x.device.type, enabled=False):
            x = self.inverse_transform(x)
        return x.to(dtype), residual
