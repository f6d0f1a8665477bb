"""Instance normalisation over (H, W) with optional fused GELU, fp32 statistics, bf16 data.

Replaces `nn.InstanceNorm2d(affine=True, eps=1e-6)` followed by the block activation
(makani/models/networks/sfnonet.py:246-252,379).  Forward is one kernel (statistics pass + normalise pass of
the same CTA, second pass served by L2 where the plane fits); backward is one kernel that recomputes the
normalised value (and GELU') from the saved input and (mean, rstd) instead of storing them.
"""

from __future__ import annotations

import torch

from . import _ext


class _InstanceNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, act):
        ext = _ext.require()
        B, C = x.shape[0], x.shape[1]
        y = torch.empty_like(x)
        stats = torch.empty(B * C, 2, dtype=torch.float32, device=x.device)
        wf = weight.detach().float().contiguous() if weight is not None else None
        bf = bias.detach().float().contiguous() if bias is not None else None
        ext.inorm_fwd(x, y, wf, bf, stats, C, float(eps), int(act), 0)
        ctx.save_for_backward(x, wf, bf, stats)
        ctx.act = int(act)
        ctx.C = C
        ctx.affine = weight is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.require()
        x, wf, bf, stats = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        C = ctx.C
        dw = torch.zeros(C, dtype=torch.float32, device=x.device) if ctx.affine else None
        db = torch.zeros(C, dtype=torch.float32, device=x.device) if ctx.affine else None
        hw = x.numel() // stats.shape[0]
        ext.inorm_bwd(x, dy, dx, wf, bf, stats, dw, db, None, C, float(hw), ctx.act, 0)
        return dx, dw, db, None, None


def instance_norm(x: torch.Tensor, weight, bias, eps: float = 1e-6, act: str = "none") -> torch.Tensor:
    """y = act(IN(x) * weight + bias) over the last two dims of NCHW `x`."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 4:
        return _InstanceNorm.apply(x, weight, bias, eps, 1 if act == "gelu" else 0)
    xf = x.float()
    y = torch.nn.functional.instance_norm(xf, None, None, None if weight is None else weight.float(),
                                          None if bias is None else bias.float(), True, 0.0, eps)
    if act == "gelu":
        y = torch.nn.functional.gelu(y)
    return y.to(x.dtype)


def channel_sums(x: torch.Tensor) -> torch.Tensor:
    """sum over (batch, H, W) of a NCHW tensor in fp32 (bias gradients)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
        ext = _ext.require()
        B, C = x.shape[0], x.shape[1]
        sums = torch.empty(B * C, 2, dtype=torch.float32, device=x.device)
        ext.inorm_partial_stats(x, sums)
        return sums[:, 0].view(B, C).sum(0)
    return x.float().sum(dim=(0, 2, 3))
