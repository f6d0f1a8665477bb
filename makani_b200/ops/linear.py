"""Linear layers on the last dimension ("traditional" token layout [..., C]) as tcgen05 GEMMs.

`Y[t, o] = act(sum_c X[t, c] W[o, c] + b[o])`: both operands are K-major, the bias is per output column and the
result is written row-major.  Used by the AFNO / ViT token MLPs.
"""

from __future__ import annotations

import torch

from . import _ext
from .gemm import ACT_GELU, ACT_MULAUX, ACT_NONE, BIAS_COL, Operand, Output, gemm, pad_to


def fast_path_ok(x: torch.Tensor) -> bool:
    return _ext.native() and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[-1] % 8 == 0


def _wq(w):
    return w.detach().to(torch.bfloat16).contiguous()


def _lin_fwd(x2, wq, bias, act, want_pre, deriv=False):
    T, C = x2.shape
    O = wq.shape[0]
    y = torch.empty(T, O, dtype=torch.bfloat16, device=x2.device)
    pre = torch.empty_like(y) if want_pre else None
    gemm(T, O, C, Operand(x2, ld=C), Operand(wq, ld=C), Output(y, rs_lo=O), bias=bias, bias_mode=BIAS_COL, act=act, preact=pre,
         preact_deriv=deriv)
    return y, pre


def _lin_dgrad(dy, wq, act=ACT_NONE, aux=None):
    T, O = dy.shape
    C = wq.shape[1]
    dx = torch.empty(T, C, dtype=torch.bfloat16, device=dy.device)
    # dX[t, c] = sum_o dY[t, o] W[o, c]: B operand rows c, K = o, element (c, o) at o*C + c -> row-contiguous
    gemm(T, C, O, Operand(dy, ld=O), Operand(wq, ld=C, mn_major=True), Output(dx, rs_lo=C), act=act, resid=aux)
    return dx


def _lin_wgrad(dy, x2):
    T, O = dy.shape
    C = x2.shape[1]
    dw = torch.zeros(O, C, dtype=torch.float32, device=dy.device)
    tiles = ((O + 127) // 128) * ((C + 255) // 256)
    splits = max(1, min((T + 63) // 64, (2 * _ext.sm_count() + tiles - 1) // tiles))
    # dW[o, c] = sum_t dY[t, o] X[t, c]: both operands row-contiguous in their own index, K = t
    gemm(O, C, T, Operand(dy, ld=O, mn_major=True), Operand(x2, ld=C, mn_major=True), Output(dw, rs_lo=C),
         accumulate=True, splits=splits)
    return dw


class _MLP2Last(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        w1q, w2q = _wq(w1), _wq(w2)
        b1f = b1.detach().float().contiguous() if b1 is not None else None
        b2f = b2.detach().float().contiguous() if b2 is not None else None
        h, dact = _lin_fwd(x2, w1q, b1f, ACT_GELU, True, deriv=True)     # second output: GELU'(pre-activation)
        y, _ = _lin_fwd(h, w2q, b2f, ACT_NONE, False)
        ctx.save_for_backward(x2, w1q, w2q, dact, h)
        ctx.flags = (b1 is not None, b2 is not None)
        ctx.shp = shp
        return y.reshape(*shp[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1q, w2q, dact, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dpre = _lin_dgrad(dy2, w2q, act=ACT_MULAUX, aux=dact)
        dw2 = _lin_wgrad(dy2, h)
        db2 = dy2.float().sum(0) if ctx.flags[1] else None
        dx = _lin_dgrad(dpre, w1q).reshape(ctx.shp) if ctx.needs_input_grad[0] else None
        dw1 = _lin_wgrad(dpre, x2)
        db1 = dpre.float().sum(0) if ctx.flags[0] else None
        return dx, dw1, db1, dw2, db2


class _LinearLast(torch.autograd.Function):
    """y = x W^T + b on the last dimension: one GEMM forward, data- and weight-gradient GEMMs backward."""

    @staticmethod
    def forward(ctx, x, w, b):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        wq = _wq(w)
        y, _ = _lin_fwd(x2, wq, b.detach().float().contiguous() if b is not None else None, ACT_NONE, False)
        ctx.save_for_backward(x2, wq)
        ctx.has_bias, ctx.shp = b is not None, shp
        return y.reshape(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wq = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = _lin_dgrad(dy2, wq).reshape(ctx.shp) if ctx.needs_input_grad[0] else None
        dw = _lin_wgrad(dy2, x2) if ctx.needs_input_grad[1] else None
        db = dy2.float().sum(0) if ctx.has_bias else None
        return dx, dw, db


def linear_lastdim(x, w, b=None):
    """`torch.nn.functional.linear` for bf16 CUDA tokens whose feature counts are multiples of 8; anything else falls
    back to the torch op."""
    if fast_path_ok(x) and w.shape[0] % 8 == 0:
        _ext.require()
        return _LinearLast.apply(x, w, b)
    return torch.nn.functional.linear(x, w.to(x.dtype), None if b is None else b.to(x.dtype))


def mlp2_lastdim(x, w1, b1, w2, b2):
    _ext.require()
    return _MLP2Last.apply(x, w1, b1, w2, b2)
