"""Pointwise (1x1) convolutions as tcgen05 GEMMs with fused epilogues, for NCHW and channels-last activations.

`Y[b, co, hw] = act(sum_ci W[co, ci] X[b, ci, hw] + bias[co]) (+ residual)` is one batched GEMM launch; which
operand plays which role depends only on the memory layouts, no data is ever transposed:

  * channels-last activations (`torch.channels_last`, channels contiguous) are the fast internal format: a token
    tile is one contiguous slab of memory (TMA- and TLB-friendly).  Output channels-last: M = tokens, N = Cout,
    D row-major [tokens, Cout], bias per column.
  * NCHW tensors are accepted at the network boundary (input fields, predictions): as input they are read
    row-contiguous, as output the roles are swapped (M = Cout, N = tokens) so the result lands in NCHW directly.

The backward pass is two more GEMMs (data gradient; weight gradient as a split-k reduction with fp32 atomics)
and the GELU derivative is applied in the data-gradient epilogue from the saved pre-activation.
The reference runs these layers through cuDNN/cuBLAS under autocast
(makani/models/common/layers.py:86-216, makani/models/networks/sfnonet.py:167,207,463).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _ext
from .gemm import ACT_GELU, ACT_MULAUX, ACT_NONE, BIAS_COL, BIAS_ROW, Operand, Output, gemm, pad_to

NCHW, CL = "nchw", "cl"


def layout_of(x: torch.Tensor) -> Optional[str]:
    if x.dim() != 4:
        return None
    if x.is_contiguous():
        return NCHW
    if x.is_contiguous(memory_format=torch.channels_last):
        return CL
    return None


def fast_path_ok(x: torch.Tensor) -> bool:
    """True when the native GEMM path applies: CUDA/CPU-emulated bf16 4-D tensor in a supported layout with 16-byte strides."""
    if x.dim() != 4 or x.dtype != torch.bfloat16 or not _ext.native():
        return False
    lay = layout_of(x)
    if lay == NCHW:
        return (x.shape[2] * x.shape[3]) % 8 == 0
    if lay == CL:
        return x.shape[1] % 8 == 0
    return False


def empty_like_layout(B, C, H, W, layout, dtype, device):
    if layout == CL:
        return torch.empty(B, C, H, W, dtype=dtype, device=device, memory_format=torch.channels_last)
    return torch.empty(B, C, H, W, dtype=dtype, device=device)


def default_out_layout(co: int) -> str:
    return CL if co % 8 == 0 else NCHW


def prep_weight(w: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """fp32 [Co, Ci(,1,1)] -> bf16 [Co, pad8(Ci)] (zero padded), the K-major weight operand."""
    w2 = w.reshape(w.shape[0], -1)
    co, ci = w2.shape
    cip = pad_to(ci, 8)
    out = torch.zeros(co, cip, dtype=dtype, device=w.device)
    out[:, :ci] = w2.detach().to(dtype)
    return out


def _tok_rows(x, lay):
    """Operand whose rows are the tokens of one image and whose K index is the channel."""
    B, C, H, W = x.shape
    T = H * W
    if lay == CL:
        return Operand(x, ld=C, mn_major=False, zs_lo=T * C)
    return Operand(x, ld=T, mn_major=True, zs_lo=C * T)


def _chan_rows(x, lay):
    """Operand whose rows are the channels and whose K index runs over the tokens of one image."""
    B, C, H, W = x.shape
    T = H * W
    if lay == CL:
        return Operand(x, ld=C, mn_major=True, zs_lo=T * C)
    return Operand(x, ld=T, mn_major=False, zs_lo=C * T)


def _out(y, lay):
    B, C, H, W = y.shape
    T = H * W
    if lay == CL:
        return Output(y, rs_lo=C, d_zlo=T * C)      # rows = tokens
    return Output(y, rs_lo=T, d_zlo=C * T)          # rows = channels


def _conv_fwd(x, wq, ci, bias, act, resid, want_preact, out_layout=None, out=None, sync=None, dests=None, deriv=False):
    """`out` (optional) receives the result instead of a fresh tensor; `sync` / `dests` are handed to the GEMM
    (handshake descriptor and additional copies of the output buffer in peers' memory).  With `deriv` the second
    output holds GELU'(pre-activation) instead of the pre-activation."""
    B, C, H, W = x.shape
    assert C == ci
    T = H * W
    co = wq.shape[0]
    lay = layout_of(x)
    out_layout = out_layout or (layout_of(resid) if resid is not None else default_out_layout(co))
    y = out if out is not None else empty_like_layout(B, co, H, W, out_layout, x.dtype, x.device)
    pre = torch.empty_like(y) if want_preact else None
    if resid is not None:
        assert layout_of(resid) == out_layout, "residual must have the layout of the output"
    wop = Operand(wq, ld=wq.shape[1])
    if out_layout == CL:
        gemm(T, co, ci, _tok_rows(x, lay), wop, _out(y, CL), zlo_n=B, bias=bias, bias_mode=BIAS_COL, act=act,
             resid=resid, preact=pre, sync=sync, dests=dests, preact_deriv=deriv)
    else:
        gemm(co, T, ci, wop, _tok_rows(x, lay), _out(y, NCHW), zlo_n=B, bias=bias, bias_mode=BIAS_ROW, act=act,
             resid=resid, preact=pre, sync=sync, dests=dests, preact_deriv=deriv)
    return y, pre


def _conv_dgrad(dy, wq, ci, act=ACT_NONE, aux=None, x_layout=None, out=None, sync=None, dests=None):
    """dX[b, ci, hw] = sum_co W[co, ci] dY[b, co, hw]  (optionally times GELU'(aux)), produced in `x_layout`."""
    B, co, H, W = dy.shape
    T = H * W
    lay = layout_of(dy)
    x_layout = x_layout or (layout_of(aux) if aux is not None else lay)
    dx = out if out is not None else empty_like_layout(B, ci, H, W, x_layout, dy.dtype, dy.device)
    wt = Operand(wq, ld=wq.shape[1], mn_major=True)     # rows = ci, K = co
    if x_layout == CL:
        gemm(T, ci, co, _tok_rows(dy, lay), wt, _out(dx, CL), zlo_n=B, act=act, resid=aux, sync=sync, dests=dests)
    else:
        gemm(ci, T, co, wt, _tok_rows(dy, lay), _out(dx, NCHW), zlo_n=B, act=act, resid=aux, sync=sync, dests=dests)
    return dx


def _conv_wgrad(dy, x, splits: Optional[int] = None):
    """dW[co, ci] = sum_{b,hw} dY[b, co, hw] X[b, ci, hw] in fp32 (split-k, atomically accumulated)."""
    B, co, H, W = dy.shape
    ci = x.shape[1]
    T = H * W
    dw = torch.zeros(co, ci, dtype=torch.float32, device=dy.device)
    if splits is None:
        tiles = ((co + 127) // 128) * ((ci + 255) // 256) * B
        kblocks = (T + 63) // 64
        splits = max(1, min(kblocks, (2 * _ext.sm_count() + tiles - 1) // tiles))
    gemm(co, ci, T, _chan_rows(dy, layout_of(dy)), _chan_rows(x, layout_of(x)), Output(dw, rs_lo=ci), zlo_n=B,
         accumulate=True, splits=splits)
    return dw


def _chan_sum(dy):
    # bias gradient: sum over batch and space (fp32), one read of dy
    from .norm import channel_sums
    return channel_sums(dy)


def _canon(t):
    """Gradients arrive in whatever layout autograd produced; bring them to a supported dense layout."""
    if layout_of(t) is None:
        t = t.contiguous()
    return t


class _Conv1x1(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, resid, act, out_layout):
        wq = prep_weight(w)
        ci = w.shape[1]
        bias_f = bias.detach().float().contiguous() if bias is not None else None
        y, pre = _conv_fwd(x, wq, ci, bias_f, act, resid, want_preact=(act == ACT_GELU), out_layout=out_layout)
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
        dy = _canon(dy)
        dres = dy if ctx.has_resid else None
        if ctx.act == ACT_GELU:
            from .elementwise import dgelu_mul
            g = dgelu_mul(dy, pre)
        else:
            g = dy
        dx = _conv_dgrad(g, wq, ctx.ci, x_layout=layout_of(x)) if ctx.needs_input_grad[0] else None
        dw = _conv_wgrad(g, x).reshape(ctx.wshape) if ctx.needs_input_grad[1] else None
        db = _chan_sum(g) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, dres, None, None


class _MLP2(torch.autograd.Function):
    """y = W2 gelu(W1 x + b1) + b2 (+ resid): two GEMMs forward, four backward, GELU' fused in the dgrad epilogue.
    The hidden activation is always channels-last."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, resid, out_layout):
        w1q, w2q = prep_weight(w1), prep_weight(w2)
        ci, ch = w1.shape[1], w1.shape[0]
        b1f = b1.detach().float().contiguous() if b1 is not None else None
        b2f = b2.detach().float().contiguous() if b2 is not None else None
        hid_layout = CL if ch % 8 == 0 else NCHW
        # the first GEMM's second output is GELU'(pre-activation): the backward epilogue then only multiplies
        h, dact = _conv_fwd(x, w1q, ci, b1f, ACT_GELU, None, want_preact=True, out_layout=hid_layout, deriv=True)
        y, _ = _conv_fwd(h, w2q, ch, b2f, ACT_NONE, resid, want_preact=False, out_layout=out_layout)
        ctx.save_for_backward(x, w1q, w2q, dact, h)
        ctx.dims = (ci, ch)
        ctx.flags = (b1 is not None, b2 is not None, resid is not None)
        ctx.wshapes = (w1.shape, w2.shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1q, w2q, dact, h = ctx.saved_tensors
        ci, ch = ctx.dims
        has_b1, has_b2, has_res = ctx.flags
        dy = _canon(dy)
        dpre = _conv_dgrad(dy, w2q, ch, act=ACT_MULAUX, aux=dact, x_layout=layout_of(dact))
        dw2 = _conv_wgrad(dy, h).reshape(ctx.wshapes[1])
        db2 = _chan_sum(dy) if has_b2 else None
        dx = _conv_dgrad(dpre, w1q, ci, x_layout=layout_of(x)) if ctx.needs_input_grad[0] else None
        dw1 = _conv_wgrad(dpre, x).reshape(ctx.wshapes[0])
        db1 = _chan_sum(dpre) if has_b1 else None
        return dx, dw1, db1, dw2, db2, (dy if has_res else None), None


def _native(x, resid):
    return x.is_cuda and fast_path_ok(x) and (resid is None or fast_path_ok(resid))


def conv1x1(x, w, bias=None, resid=None, act: str = "none", out_layout: Optional[str] = None):
    """1x1 convolution on a 4-D activation. CUDA bf16 -> tcgen05 GEMM; anything else -> reference torch ops."""
    if _native(x, resid):
        _ext.require()
        return _Conv1x1.apply(x, w, bias, resid, ACT_GELU if act == "gelu" else ACT_NONE, out_layout)
    w4 = w.reshape(w.shape[0], -1, 1, 1).to(x.dtype)
    y = torch.nn.functional.conv2d(x, w4, None if bias is None else bias.to(x.dtype))
    if act == "gelu":
        y = torch.nn.functional.gelu(y, approximate=_ext.gelu_approximation())
    if resid is not None:
        y = y + resid
    return y


def mlp2(x, w1, b1, w2, b2, resid=None, out_layout: Optional[str] = None):
    """Two-layer pointwise MLP with GELU (encoder, decoder and block MLP of the SFNO/AFNO networks)."""
    if _native(x, resid):
        _ext.require()
        return _MLP2.apply(x, w1, b1, w2, b2, resid, out_layout)
    f = torch.nn.functional
    h = f.gelu(f.conv2d(x, w1.reshape(w1.shape[0], -1, 1, 1).to(x.dtype), None if b1 is None else b1.to(x.dtype)),
               approximate=_ext.gelu_approximation())
    y = f.conv2d(h, w2.reshape(w2.shape[0], -1, 1, 1).to(x.dtype), None if b2 is None else b2.to(x.dtype))
    if resid is not None:
        y = y + resid
    return y
