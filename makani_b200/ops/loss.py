"""Quadrature-weighted Lp norms on the sphere as a fused reduction kernel.

`weighted_lp_norms(pred, tgt, qlat, p)` returns, per (batch, channel), the pair
(sum_hw q_h |pred - tgt|^p, sum_hw q_h |tgt|^p) — the two integrals every variant of the reference's
`GeometricLpLoss` is built from (makani/utils/losses.py:213-257, makani/utils/grids.py:113-115).  The
square-root / ratio / channel weighting that follows is a handful of scalars per channel and stays in torch
autograd; the backward of the integrals is a second streaming kernel.
"""

from __future__ import annotations

import torch

from . import _ext

_SCRATCH = {}


def _scratch(device, nfloats: int) -> torch.Tensor:
    key = str(device)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < nfloats:
        buf = torch.zeros(nfloats, dtype=torch.float32, device=device)
        _SCRATCH[key] = buf
    return buf


class _LpNorms(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pred, tgt, qlat, p):
        ext = _ext.require()
        B, C, H, W = pred.shape
        out = torch.empty(B * C, 2, dtype=torch.float32, device=pred.device)
        scratch = _scratch(pred.device, ext.lp_scratch_floats(B * C, H * W))
        ext.lp_norms(pred, tgt, qlat, out, scratch, int(p))
        ctx.save_for_backward(pred, tgt, qlat)
        ctx.p = int(p)
        return out.view(B, C, 2)

    @staticmethod
    def backward(ctx, dout):
        ext = _ext.require()
        pred, tgt, qlat = ctx.saved_tensors
        # only the diff-norm depends on pred; the target norm is treated as a constant
        coef = dout[..., 0].contiguous().float().view(-1)
        grad = torch.empty_like(pred)
        ext.lp_norms_bwd(pred, tgt, qlat, coef, grad, ctx.p)
        return grad, None, None, None


def weighted_lp_norms(pred: torch.Tensor, tgt: torch.Tensor, qlat: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, 2] fp32: (int q |pred - tgt|^p, int q |tgt|^p) with latitude weights qlat[H] (longitude weight folded in)."""
    if _ext.native() and pred.is_cuda and pred.dtype in (torch.bfloat16, torch.float32):
        tgt = tgt.to(pred.dtype).contiguous()
        return _LpNorms.apply(pred.contiguous(), tgt, qlat.float().contiguous(), p)
    q = qlat.to(torch.float32).view(1, 1, -1, 1)
    pf, tf = pred.float(), tgt.float()
    d = (pf - tf).abs() ** p
    t = tf.abs() ** p
    return torch.stack([(d * q).sum(dim=(-2, -1)), (t * q).sum(dim=(-2, -1))], dim=-1)
