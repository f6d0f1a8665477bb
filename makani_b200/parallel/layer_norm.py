"""Normalisation layers for spatially sharded activations.

`DistributedInstanceNorm2d` computes per-(sample, channel) statistics over the *global* (H, W) extent of
data tiled [H_loc, W_loc] over the `spatial` group: each rank reduces (count, sum, sum of squares) of its
tile in fp32, the three numbers are summed over the group, and every rank normalises its own tile; the
backward pass needs the analogous two reductions.  The reference gathers (var, mean, count) from all ranks and
merges them serially with Welford updates (makani/mpu/layer_norm.py:53-114), which is the same statistic.
On CUDA bf16 the local passes are the fused kernels of `makani_b200.ops.norm` and the exchange is a single
all-reduce of a [B, C, 2] fp32 tensor.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _ext
from ..utils import comm


# MAKANI_B200_PEER_NORM_STATS=0: exchange the statistics with an NCCL all-reduce instead of in-kernel peer stores
PEER_STATS = os.environ.get("MAKANI_B200_PEER_NORM_STATS", "1") != "0"


def _allreduce_spatial(t: torch.Tensor) -> torch.Tensor:
    if comm.get_size("spatial") > 1:
        dist.all_reduce(t, group=comm.get_group("spatial"))
    return t


class _DistInstanceNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, count):
        B, C = x.shape[:2]
        fast = x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
        if fast:
            ext = _ext.require()
            sums = torch.empty(B * C, 2, dtype=torch.float32, device=x.device)
            ext.inorm_partial_stats(x, sums)
        else:
            xf = x.float()
            sums = torch.stack([xf.sum(dim=(-2, -1)), (xf * xf).sum(dim=(-2, -1))], dim=-1).reshape(B * C, 2)
        sums = _allreduce_spatial(sums.contiguous())
        mean = sums[:, 0] / count
        var = (sums[:, 1] / count - mean * mean).clamp_min(0.0)
        rstd = torch.rsqrt(var + eps)
        stats = torch.stack([mean, rstd], dim=-1).contiguous()
        wf = weight.detach().float().contiguous() if weight is not None else None
        bf = bias.detach().float().contiguous() if bias is not None else None
        if fast:
            y = torch.empty_like(x)
            ext.inorm_fwd(x, y, wf, bf, stats, C, float(eps), 0, 1)
        else:
            y = (x.float() - mean.view(B, C, 1, 1)) * rstd.view(B, C, 1, 1)
            if wf is not None:
                y = y * wf.view(1, C, 1, 1) + bf.view(1, C, 1, 1)
            y = y.to(x.dtype)
        ctx.save_for_backward(x, wf, bf, stats)
        ctx.count, ctx.fast, ctx.affine = count, fast, weight is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wf, bf, stats = ctx.saved_tensors
        B, C = x.shape[:2]
        dy = dy.contiguous()
        dw = db = None
        if ctx.fast:
            ext = _ext.require()
            sums = torch.empty(B * C, 2, dtype=torch.float32, device=x.device)
            if ctx.affine:
                dw = torch.zeros(C, dtype=torch.float32, device=x.device)
                db = torch.zeros(C, dtype=torch.float32, device=x.device)
            ext.inorm_bwd(x, dy, None, wf, bf, stats, dw, db, sums, C, float(ctx.count), 0, 1)
            sums = _allreduce_spatial(sums)
            dx = torch.empty_like(x)
            ext.inorm_bwd(x, dy, dx, wf, bf, stats, None, None, sums, C, float(ctx.count), 0, 2)
        else:
            mean, rstd = stats[:, 0].view(B, C, 1, 1), stats[:, 1].view(B, C, 1, 1)
            xh = (x.float() - mean) * rstd
            g = dy.float()
            s1, s2 = g.sum(dim=(-2, -1)), (g * xh).sum(dim=(-2, -1))
            if ctx.affine:
                dw, db = s2.sum(0), s1.sum(0)
            sums = _allreduce_spatial(torch.stack([s1, s2], dim=-1).contiguous())
            m1, m2 = (sums[..., 0] / ctx.count).view(B, C, 1, 1), (sums[..., 1] / ctx.count).view(B, C, 1, 1)
            w = wf.view(1, C, 1, 1) if wf is not None else 1.0
            dx = (rstd * w * (g - m1 - xh * m2)).to(x.dtype)
        return dx, dw, db, None, None


class DistributedInstanceNorm2d(nn.Module):
    def __init__(self, num_features, eps=1e-05, affine=False, device=None, dtype=None):
        super().__init__()
        self.eps, self.affine, self.num_features = eps, affine, num_features
        self._counts = {}
        if affine:
            self.weight = nn.Parameter(torch.ones(num_features, device=device, dtype=dtype))
            self.bias = nn.Parameter(torch.zeros(num_features, device=device, dtype=dtype))
            self.weight.is_shared_mp = ["spatial"]
            self.bias.is_shared_mp = ["spatial"]

    def _global_count(self, x) -> float:
        """Global number of grid points per (sample, channel); computed once per local tile shape."""
        key = (x.shape[-2], x.shape[-1])
        if key not in self._counts:
            cnt = torch.tensor([float(key[0] * key[1])], dtype=torch.float64, device=x.device)
            if comm.get_size("spatial") > 1:
                dist.all_reduce(cnt, group=comm.get_group("spatial"))
            self._counts[key] = float(cnt.item())
        return self._counts[key]

    def _slot(self, x):
        """Peer-memory exchange buffer for the statistics (NCCL ranks of one node, at most 8), else None."""
        n = comm.get_size("spatial")
        if not (PEER_STATS and x.is_cuda and 1 < n <= 8 and dist.get_backend(comm.get_group("spatial")) == "nccl"):
            return None
        from .peer import get_slot
        return get_slot("inorm", "spatial", x.shape[0] * x.shape[1] * 8, x.device)

    def forward(self, x, act: str = "none"):
        from ..ops import norm as norm_ops
        w = self.weight if self.affine else None
        b = self.bias if self.affine else None
        cnt = self._global_count(x)
        if norm_ops.cl_supported(x):
            # fused channels-last kernels; only the [B, C, 2] partial sums cross the spatial group: through peer memory
            # from inside the two kernels when the ranks can map each other's memory, else through an all-reduce
            slot = self._slot(x)
            return norm_ops.instance_norm(x, w, b, self.eps, act, count=cnt,
                                          reduce_fn=None if slot is not None else _allreduce_spatial, slot=slot)
        y = _DistInstanceNormFn.apply(x, w, b, self.eps, cnt)
        if act == "gelu":
            y = torch.nn.functional.gelu(y, approximate=_ext.gelu_approximation())
        return y


class DistributedLayerNorm(nn.Module):
    """Layer norm over the channel dimension of NCHW data (channels must not be sharded)."""

    def __init__(self, normalized_shape, eps=1e-05, elementwise_affine=True, bias=True, device=None, dtype=None):
        super().__init__()
        assert comm.get_size("matmul") == 1, "channel-sharded layer norm is not supported"
        self.norm = nn.LayerNorm(normalized_shape, eps=eps, elementwise_affine=elementwise_affine, bias=bias,
                                 device=device, dtype=dtype)
        if elementwise_affine:
            self.norm.weight.is_shared_mp = ["model"]
            if bias:
                self.norm.bias.is_shared_mp = ["model"]

    def forward(self, x):
        return torch.transpose(self.norm(torch.transpose(x, 1, 3)), 1, 3)
