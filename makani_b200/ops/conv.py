"""Pointwise (1x1) convolutions on NCHW bf16 activations as tcgen05 GEMMs with fused epilogues.

`Y[b, co, hw] = act(sum_ci W[co, ci] X[b, ci, hw] + bias[co]) (+ residual)` maps to one batched GEMM with
A = W (K-major), B = X[b] (N-major view, no transpose pass) and D written in place in NCHW.  The backward
pass is two more GEMMs (data gradient with W read M-major; weight gradient as a split-k reduction with fp32
atomics) — the GELU derivative is applied in the data-gradient epilogue.

The reference runs these layers through cuDNN/cuBLAS under autocast
(makani/models/common/layers.py:86-216, makani/models/networks/sfnonet.py:167,207,463).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _ext
from .gemm import ACT_DGELU, ACT_GELU, ACT_NONE, BIAS_ROW, Operand, Output, gemm, pad_to


def fast_path_ok(x: torch.Tensor) -> bool:
    """True when the native NCHW GEMM path applies: bf16, 4-D contiguous, H*W a multiple of 8."""
    return (x.dim() == 4 and x.dtype == torch.bfloat16 and x.is_contiguous()
            and (x.shape[2] * x.shape[3]) % 8 == 0)


def prep_weight(w: torch.Tensor) -> torch.Tensor:
    """fp32 [Co, Ci(,1,1)] -> bf16 [Co, pad8(Ci)] (zero padded) as the K-major A operand."""
    w2 = w.reshape(w.shape[0], -1)
    co, ci = w2.shape
    cip = pad_to(ci, 8)
    out = torch.zeros(co, cip, dtype=torch.bfloat16, device=w.device)
    out[:, :ci] = w2.detach().to(torch.bfloat16)
    return out


def _conv_fwd(x, wq, ci, bias, act, resid, want_preact):
    B, C, H, W = x.shape
    assert C == ci
    hw = H * W
    co = wq.shape[0]
    y = torch.empty(B, co, H, W, dtype=torch.bfloat16, device=x.device)
    pre = torch.empty_like(y) if want_preact else None
    gemm(co, hw, ci,
         Operand(wq, ld=wq.shape[1]),
         Operand(x, ld=hw, mn_major=True, zs_lo=ci * hw),
         Output(y, rs_lo=hw, d_zlo=co * hw),
         zlo_n=B, bias=bias, bias_mode=BIAS_ROW, act=act, resid=resid, preact=pre)
    return y, pre


def _conv_dgrad(dy, wq, ci, act=ACT_NONE, aux=None):
    """dX[b, ci, hw] = sum_co W[co, ci] dY[b, co, hw]  (optionally times GELU'(aux))."""
    B, co, H, W = dy.shape
    hw = H * W
    dx = torch.empty(B, ci, H, W, dtype=torch.bfloat16, device=dy.device)
    gemm(ci, hw, co,
         Operand(wq, ld=wq.shape[1], mn_major=True),
         Operand(dy, ld=hw, mn_major=True, zs_lo=co * hw),
         Output(dx, rs_lo=hw, d_zlo=ci * hw),
         zlo_n=B, act=act, resid=aux)
    return dx


def _conv_wgrad(dy, x, splits: Optional[int] = None):
    """dW[co, ci] = sum_{b,hw} dY[b, co, hw] X[b, ci, hw] in fp32 (split-k, atomically accumulated)."""
    B, co, H, W = dy.shape
    ci = x.shape[1]
    hw = H * W
    dw = torch.zeros(co, ci, dtype=torch.float32, device=dy.device)
    if splits is None:
        tiles = ((co + 127) // 128) * ((ci + 255) // 256) * B
        kblocks = (hw + 63) // 64
        splits = max(1, min(kblocks, (2 * 148 + tiles - 1) // tiles))
    gemm(co, ci, hw,
         Operand(dy, ld=hw, zs_lo=co * hw),
         Operand(x, ld=hw, zs_lo=ci * hw),
         Output(dw, rs_lo=ci),
         zlo_n=B, accumulate=True, splits=splits)
    return dw


def _chan_sum(dy):
    # bias gradient: sum over batch and space (fp32), one read of dy
    from .norm import channel_sums
    return channel_sums(dy)


class _Conv1x1(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, resid, act):
        wq = prep_weight(w)
        ci = w.shape[1]
        bias_f = bias.detach().float().contiguous() if bias is not None else None
        y, pre = _conv_fwd(x, wq, ci, bias_f, act, resid, want_preact=(act == ACT_GELU))
        ctx.save_for_backward(x, wq, pre)
        ctx.ci = ci
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.has_resid = resid is not None
        ctx.wshape = w.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wq, pre = ctx.saved_tensors
        dy = dy.contiguous()
        dres = dy if ctx.has_resid else None
        if ctx.act == ACT_GELU:
            from .elementwise import dgelu_mul
            g = dgelu_mul(dy, pre)
        else:
            g = dy
        dx = _conv_dgrad(g, wq, ctx.ci) if ctx.needs_input_grad[0] else None
        dw = _conv_wgrad(g, x).reshape(ctx.wshape) if ctx.needs_input_grad[1] else None
        db = _chan_sum(g) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, dres, None


class _MLP2(torch.autograd.Function):
    """y = W2 gelu(W1 x + b1) + b2 (+ resid): two GEMMs forward, four backward, GELU' fused in the dgrad epilogue."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, resid):
        w1q, w2q = prep_weight(w1), prep_weight(w2)
        ci, ch = w1.shape[1], w1.shape[0]
        b1f = b1.detach().float().contiguous() if b1 is not None else None
        b2f = b2.detach().float().contiguous() if b2 is not None else None
        h, pre = _conv_fwd(x, w1q, ci, b1f, ACT_GELU, None, want_preact=True)
        y, _ = _conv_fwd(h, w2q, ch, b2f, ACT_NONE, resid, want_preact=False)
        ctx.save_for_backward(x, w1q, w2q, pre, h)
        ctx.dims = (ci, ch)
        ctx.flags = (b1 is not None, b2 is not None, resid is not None)
        ctx.wshapes = (w1.shape, w2.shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1q, w2q, pre, h = ctx.saved_tensors
        ci, ch = ctx.dims
        has_b1, has_b2, has_res = ctx.flags
        dy = dy.contiguous()
        dpre = _conv_dgrad(dy, w2q, ch, act=ACT_DGELU, aux=pre)
        dw2 = _conv_wgrad(dy, h).reshape(ctx.wshapes[1])
        db2 = _chan_sum(dy) if has_b2 else None
        dx = _conv_dgrad(dpre, w1q, ci) if ctx.needs_input_grad[0] else None
        dw1 = _conv_wgrad(dpre, x).reshape(ctx.wshapes[0])
        db1 = _chan_sum(dpre) if has_b1 else None
        return dx, dw1, db1, dw2, db2, (dy if has_res else None)


def conv1x1(x, w, bias=None, resid=None, act: str = "none"):
    """1x1 convolution on NCHW. CUDA bf16 -> tcgen05 GEMM; anything else -> reference torch ops."""
    if x.is_cuda and fast_path_ok(x) and (resid is None or fast_path_ok(resid)):
        _ext.require()
        return _Conv1x1.apply(x, w, bias, resid, ACT_GELU if act == "gelu" else ACT_NONE)
    w4 = w.reshape(w.shape[0], -1, 1, 1).to(x.dtype)
    y = torch.nn.functional.conv2d(x, w4, None if bias is None else bias.to(x.dtype))
    if act == "gelu":
        y = torch.nn.functional.gelu(y)
    if resid is not None:
        y = y + resid
    return y


def mlp2(x, w1, b1, w2, b2, resid=None):
    """Two-layer pointwise MLP with GELU (encoder, decoder and block MLP of the SFNO/AFNO networks)."""
    if x.is_cuda and fast_path_ok(x) and (resid is None or fast_path_ok(resid)):
        _ext.require()
        return _MLP2.apply(x, w1, b1, w2, b2, resid)
    f = torch.nn.functional
    h = f.gelu(f.conv2d(x, w1.reshape(w1.shape[0], -1, 1, 1).to(x.dtype), None if b1 is None else b1.to(x.dtype)))
    y = f.conv2d(h, w2.reshape(w2.shape[0], -1, 1, 1).to(x.dtype), None if b2 is None else b2.to(x.dtype))
    if resid is not None:
        y = y + resid
    return y
