"""Mode-wise complex contractions of the "diagonal" and "separable" spectral operators as streaming CUDA kernels.

    diagonal        out[b, o, x, y] = sum_i a[b, i, x, y] w[i, o, x, y]      (makani/models/common/contractions.py:121-127)
    separable diag  out[b, i, x, y] = a[b, i, x, y] w[i, x, y]               (contractions.py:139-146)
    separable dh    out[b, i, x, y] = a[b, i, x, y] w[i, x]                  (contractions.py:148-154)

With a batch of one or two samples per GPU these are matrix-vector products per mode: there is no tile for the tensor
cores, the cost is reading the weights once.  The kernels (`csrc/spectral_modes.cu`) run their threads along the mode
index, read every weight element once per sample with streaming loads, and serve forward, input gradient (conjugated
weights) and weight gradient.  Anything that is not contiguous complex64 on CUDA goes through `torch.einsum`.
"""

from __future__ import annotations

import torch

from . import _ext


def _ok(*ts) -> bool:
    return _ext.native() and all(t.is_cuda and t.dtype == torch.complex64 for t in ts)


class _Diag(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w):
        ext = _ext.require()
        a, w = a.contiguous(), w.contiguous()
        B, I, X, Y = a.shape
        O = w.shape[1]
        out = torch.empty(B, O, X, Y, dtype=a.dtype, device=a.device)
        ext.modes_diag(a, w, out, B, I, O, X * Y, 0)
        ctx.save_for_backward(a, w)
        return out

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.require()
        a, w = ctx.saved_tensors
        dy = dy.contiguous()
        B, I, X, Y = a.shape
        O = w.shape[1]
        da = dw = None
        if ctx.needs_input_grad[0]:
            da = torch.empty_like(a)
            ext.modes_diag(dy, w, da, B, I, O, X * Y, 1)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)
            ext.modes_diag(a, dy, dw, B, I, O, X * Y, 2)
        return da, dw


class _Sep(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, wdiv):
        ext = _ext.require()
        a, w = a.contiguous(), w.contiguous()
        B, I, X, Y = a.shape
        out = torch.empty_like(a)
        ext.modes_sep(a, w, out, B, I, X * Y, wdiv, 0)
        ctx.save_for_backward(a, w)
        ctx.wdiv = wdiv
        return out

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.require()
        a, w = ctx.saved_tensors
        dy = dy.contiguous()
        B, I, X, Y = a.shape
        da = dw = None
        if ctx.needs_input_grad[0]:
            da = torch.empty_like(a)
            ext.modes_sep(dy, w, da, B, I, X * Y, ctx.wdiv, 1)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)
            ext.modes_sep(a, dy, dw, B, I, X * Y, ctx.wdiv, 2)
        return da, dw, None


def contract_diagonal(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a [B, I, X, Y], w [I, O, X, Y] -> [B, O, X, Y]."""
    if _ok(a, w) and a.dim() == 4 and w.dim() == 4:
        return _Diag.apply(a, w)
    return torch.einsum("bixy,ioxy->boxy", a, w)


def contract_sep_diagonal(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a [B, I, X, Y], w [I, X, Y] -> [B, I, X, Y]."""
    if _ok(a, w) and a.dim() == 4 and w.dim() == 3:
        return _Sep.apply(a, w, 1)
    return torch.einsum("bixy,ixy->bixy", a, w)


def contract_sep_dhconv(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a [B, I, X, Y], w [I, X] -> [B, I, X, Y]."""
    if _ok(a, w) and a.dim() == 4 and w.dim() == 2:
        return _Sep.apply(a, w, a.shape[3])
    return torch.einsum("bixy,ix->bixy", a, w)
