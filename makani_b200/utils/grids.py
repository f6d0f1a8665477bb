"""Latitude/longitude grid helpers: quadrature weights on the sphere and equiangular -> Gauss grid conversion.

Behavioural contract: makani/utils/grids.py:22-115.  `GridQuadrature(rule, img_shape, crop_shape, crop_offset,
normalize, pole_mask)(x)` integrates the last two dimensions; rules "naive" (sin(theta) dtheta dlambda,
renormalised to 4 pi), "clenshaw-curtiss" and "legendre-gauss".  All rules are separable with a weight that
depends on latitude only; `lat_weights` exposes that vector (longitude element folded in), which is what the
fused loss/metric kernels consume.  With spatial model parallelism the weights are restricted to the local
tile (`local_shape`, `local_offset`).
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..sht.quadrature import clenshaw_curtiss_weights, legendre_gauss_weights


class GridConverter(torch.nn.Module):
    def __init__(self, src_grid, dst_grid, lat_rad, lon_rad):
        super().__init__()
        self.src, self.dst = src_grid, dst_grid
        self.src_lat, self.src_lon = lat_rad, lon_rad
        if self.src != self.dst:
            if self.dst != "legendre-gauss":
                raise NotImplementedError(f"destination grid type {self.dst} not implemented")
            cost, _ = legendre_gauss_weights(lat_rad.shape[0], -1, 1)
            tq = torch.arccos(torch.from_numpy(cost)) - math.pi / 2.0
            self.dst_lat = tq.to(lat_rad.device)
            self.dst_lon = lon_rad
            # source latitudes descend (north -> south); find for each target the enclosing source interval
            perm = torch.arange(lat_rad.shape[0] - 1, -1, -1, dtype=torch.long, device=lat_rad.device)
            jj = torch.searchsorted(lat_rad, self.dst_lat, sorter=perm) - 1
            self.indices = jj[perm]
            self.interp_weights = ((self.dst_lat - lat_rad[self.indices]) / torch.diff(lat_rad)[self.indices]).reshape(-1, 1)
        else:
            self.dst_lat, self.dst_lon = self.src_lat, self.src_lon

    def get_src_coords(self):
        return self.src_lat, self.src_lon

    def get_dst_coords(self):
        return self.dst_lat, self.dst_lon

    def forward(self, data):
        if self.src == self.dst:
            return data
        return torch.lerp(data[..., self.indices, :], data[..., self.indices + 1, :], self.interp_weights.to(dtype=data.dtype))


def latitude_weights(rule: str, nlat: int, nlon: int, normalize: bool = False, pole_mask: int = 0) -> torch.Tensor:
    """float64 [nlat]: area element per grid point (latitude weight times 2 pi / nlon)."""
    if rule == "naive":
        jac = torch.clamp(torch.sin(torch.linspace(0, math.pi, nlat, dtype=torch.float64)), min=0.0)
        q = (2 * math.pi / nlon) * (math.pi / nlat) * jac
        q = q * (4.0 * math.pi) / (q.sum() * nlon)
    elif rule == "clenshaw-curtiss":
        _, w = clenshaw_curtiss_weights(nlat, -1, 1)
        q = (2 * math.pi / nlon) * torch.from_numpy(np.flip(w).copy())
    elif rule == "legendre-gauss":
        _, w = legendre_gauss_weights(nlat, -1, 1)
        q = (2 * math.pi / nlon) * torch.from_numpy(np.flip(w).copy())
    else:
        raise ValueError(f"Unknown quadrature rule {rule}")
    if normalize:
        q = q / (4.0 * math.pi)
    if pole_mask is not None and pole_mask > 0:
        q[:pole_mask] = 0.0
        q[nlat - pole_mask:] = 0.0
    return q


class GridQuadrature(torch.nn.Module):
    def __init__(self, quadrature_rule, img_shape, crop_shape=None, crop_offset=(0, 0), normalize=False, pole_mask=None,
                 local_shape=None, local_offset=(0, 0)):
        super().__init__()
        q = latitude_weights(quadrature_rule, img_shape[0], img_shape[1], normalize, pole_mask or 0)
        width = img_shape[1]
        if crop_shape is not None:
            q = q[crop_offset[0]: crop_offset[0] + crop_shape[0]]
            width = crop_shape[1]
        if local_shape is not None:
            q = q[local_offset[0]: local_offset[0] + local_shape[0]]
            width = local_shape[1]
        self.register_buffer("lat_weights", q.float().contiguous(), persistent=False)
        self.register_buffer("quad_weight", q.float().reshape(1, 1, -1, 1).repeat(1, 1, 1, width).contiguous(), persistent=False)

    def forward(self, x):
        return torch.sum(x * self.quad_weight, dim=(-2, -1))
