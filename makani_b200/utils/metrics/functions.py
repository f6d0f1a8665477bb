"""Quadrature-weighted verification metrics on the sphere (L1, RMSE, anomaly correlation) and 1-D integration
rules for the ACC area-under-curve.  Contract: makani/utils/metrics/functions.py:20-163.

Every metric is built from area integrals, so with spatial model parallelism each rank integrates its own
tile and the per-channel partial integrals are summed over the `spatial` group (the reference gathers the full
field on every rank first, makani/utils/metric.py:145-152,189-191).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import comm
from ..grids import GridQuadrature


def _spatial_sum(t: torch.Tensor) -> torch.Tensor:
    if comm.get_size("spatial") > 1:
        t = t.contiguous()
        dist.all_reduce(t, group=comm.get_group("spatial"))
    return t


def _reduce(v, channel_reduction, batch_reduction):
    if channel_reduction == "mean":
        v = torch.mean(v, dim=1)
    elif channel_reduction == "sum":
        v = torch.sum(v, dim=1)
    if batch_reduction == "mean":
        v = torch.mean(v, dim=0)
    elif batch_reduction == "sum":
        v = torch.sum(v, dim=0)
    return v


class _GeometricBase(torch.nn.Module):
    def __init__(self, grid_type, img_shape, crop_shape=None, crop_offset=(0, 0), normalize=False, channel_reduction="mean",
                 batch_reduction="mean", local_shape=None, local_offset=(0, 0)):
        super().__init__()
        self.quadrature = GridQuadrature(grid_type, img_shape=img_shape, crop_shape=crop_shape, crop_offset=crop_offset,
                                         normalize=normalize, local_shape=local_shape, local_offset=local_offset)
        self.channel_reduction, self.batch_reduction = channel_reduction, batch_reduction


class GeometricL1(_GeometricBase):
    def forward(self, x, y):
        d = _spatial_sum(self.quadrature(torch.abs(x.float() - y.float())))
        return _reduce(d, self.channel_reduction, self.batch_reduction)


class GeometricRMSE(_GeometricBase):
    def forward(self, x, y):
        d = _spatial_sum(self.quadrature(torch.square(x.float() - y.float())))
        return torch.sqrt(_reduce(d, self.channel_reduction, self.batch_reduction))


class GeometricACC(_GeometricBase):
    def __init__(self, *args, eps=1e-8, **kwargs):
        super().__init__(*args, **kwargs)
        self.eps = eps

    def forward(self, x, y):
        x, y = x.float(), y.float()
        s = torch.stack([self.quadrature(x * y), self.quadrature(torch.square(x)), self.quadrature(torch.square(y))], dim=0)
        s = _spatial_sum(s)
        acc = s[0] / (torch.sqrt(s[1] * s[2]) + self.eps)
        return _reduce(acc, self.channel_reduction, self.batch_reduction)


class SimpsonQuadrature(torch.nn.Module):
    def __init__(self, num_intervals, interval_width, device):
        super().__init__()
        if num_intervals % 2 != 0:
            raise NotImplementedError("Simpson's rule needs an even number of intervals")
        w = [0.0] * (num_intervals + 1)
        for j in range(1, num_intervals // 2 + 1):
            w[2 * j - 2] += 1.0
            w[2 * j - 1] += 4.0
            w[2 * j] += 1.0
        self.weights = torch.tensor(w, dtype=torch.float32, device=device) * (interval_width / 3.0)

    def forward(self, x, dim=1):
        shape = [1] * x.dim()
        shape[dim] = -1
        return torch.sum(x * self.weights.reshape(shape), dim=dim)


class TrapezoidQuadrature(torch.nn.Module):
    def __init__(self, num_intervals, interval_width, device):
        super().__init__()
        w = [interval_width] * (num_intervals + 1)
        w[0] *= 0.5
        w[-1] *= 0.5
        self.weights = torch.tensor(w, dtype=torch.float32, device=device)

    def forward(self, x, dim=1):
        shape = [1] * x.dim()
        shape[dim] = -1
        return torch.sum(x * self.weights.reshape(shape), dim=dim)


class Quadrature(torch.nn.Module):
    def __init__(self, num_intervals, interval_width, device):
        super().__init__()
        cls = SimpsonQuadrature if (num_intervals % 2 == 0 and num_intervals > 0) else TrapezoidQuadrature
        self.quad = cls(num_intervals, interval_width, device)

    def forward(self, x, dim=1):
        return self.quad(x, dim)
