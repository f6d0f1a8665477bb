"""Instance normalisation over (H, W) with optional fused GELU, fp32 statistics, bf16 data.

Replaces `nn.InstanceNorm2d(affine=True, eps=1e-6)` followed by the block activation
(makani/models/networks/sfnonet.py:246-252,379).  Two layouts are served:

  * channels-last (the internal fast format): a statistics kernel (per-channel sums accumulated in registers,
    merged with atomics) and an apply kernel whose threads keep their channels' scale/shift in registers;
  * NCHW: one kernel per (sample, channel) plane doing both passes.

The backward pass recomputes the normalised value (and GELU') from the saved input and (mean, rstd) instead of
storing them.
"""

from __future__ import annotations

import torch

from . import _ext


def _is_cl(x):
    return x.dim() == 4 and (not x.is_contiguous()) and x.is_contiguous(memory_format=torch.channels_last)


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


class _InstanceNormCL(torch.autograd.Function):
    """Channels-last variant.  For a spatially distributed instance norm `count` is the global number of grid points
    and the [B, C, 2] partial sums are merged across the ranks either by `reduce_fn` (any collective) or, when `slot`
    (a `makani_b200.parallel.peer.PeerSlot`) is given, inside the two kernels themselves: the last CTA of the
    reduction stores this rank's sums into every peer's buffer and the normalising kernel adds the segments up."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, act, count, reduce_fn, slot=None):
        ext = _ext.require()
        B, C, H, W = x.shape
        y = torch.empty_like(x)     # preserves channels_last
        sums = torch.zeros(B, C, 2, dtype=torch.float32, device=x.device)
        stats = torch.empty(B, C, 2, dtype=torch.float32, device=x.device)
        wf = weight.detach().float().contiguous() if weight is not None else None
        bf = bias.detach().float().contiguous() if bias is not None else None
        cnt = float(count if count else H * W)
        if slot is not None:
            from ..parallel.peer import sync_descriptor
            slot.set_layout(B * C * 8)
            ext.inorm_cl_sums(x, None, None, None, None, sums, None, None, B, C, 0, 0,
                              sync_descriptor(produce=slot), slot.dests(include_self=True))
            ext.inorm_cl_apply(x, None, y, wf, bf, sums, stats, B, C, cnt, float(eps), int(act), 0,
                               sync_descriptor(consume=slot), slot.sources())
        else:
            # statistics local to this device are accumulated around the first token (mode bit 1): no cancellation in
            # E[x^2] - E[x]^2 for fields with |mean| >> std; sums merged across ranks stay unshifted
            m0 = 2 if reduce_fn is None else 0
            ext.inorm_cl_sums(x, None, None, None, None, sums, None, None, B, C, 0, m0)
            if reduce_fn is not None:
                sums = reduce_fn(sums)
            ext.inorm_cl_apply(x, None, y, wf, bf, sums, stats, B, C, cnt, float(eps), int(act), m0)
        ctx.save_for_backward(x, wf, bf, stats)
        ctx.act, ctx.cnt, ctx.reduce_fn, ctx.affine, ctx.slot = int(act), cnt, reduce_fn, weight is not None, slot
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.require()
        x, wf, bf, stats = ctx.saved_tensors
        B, C, H, W = x.shape
        if not _is_cl(dy):
            dy = dy.contiguous(memory_format=torch.channels_last)
        sums = torch.zeros(B, C, 2, dtype=torch.float32, device=x.device)
        dw = torch.zeros(C, dtype=torch.float32, device=x.device) if ctx.affine else None
        db = torch.zeros(C, dtype=torch.float32, device=x.device) if ctx.affine else None
        dx = torch.empty_like(x)
        slot = ctx.slot
        if slot is not None:
            from ..parallel.peer import sync_descriptor
            slot.set_layout(B * C * 8)
            ext.inorm_cl_sums(x, dy, wf, bf, stats, sums, dw, db, B, C, ctx.act, 1,
                              sync_descriptor(produce=slot), slot.dests(include_self=True))
            ext.inorm_cl_apply(x, dy, dx, wf, bf, sums, stats, B, C, ctx.cnt, 0.0, ctx.act, 1,
                               sync_descriptor(consume=slot), slot.sources())
        else:
            ext.inorm_cl_sums(x, dy, wf, bf, stats, sums, dw, db, B, C, ctx.act, 1)
            if ctx.reduce_fn is not None:
                sums = ctx.reduce_fn(sums)
            ext.inorm_cl_apply(x, dy, dx, wf, bf, sums, stats, B, C, ctx.cnt, 0.0, ctx.act, 1)
        return dx, dw, db, None, None, None, None, None


def cl_supported(x) -> bool:
    return (_ext.native() and x.is_cuda and x.dtype == torch.bfloat16 and _is_cl(x) and x.shape[1] % 8 == 0
            and x.shape[1] <= 1024)


def instance_norm(x: torch.Tensor, weight, bias, eps: float = 1e-6, act: str = "none", count=None, reduce_fn=None,
                  slot=None) -> torch.Tensor:
    """y = act(IN(x) * weight + bias) over the last two dims of a 4-D activation `x`."""
    a = 1 if act == "gelu" else 0
    if cl_supported(x):
        return _InstanceNormCL.apply(x, weight, bias, eps, a, count, reduce_fn, slot)
    if _ext.native() and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and count is None and reduce_fn is None:
        return _InstanceNorm.apply(x.contiguous(), weight, bias, eps, a)
    assert count is None and reduce_fn is None, "distributed statistics need the channels-last CUDA path"
    xf = x.float()
    y = torch.nn.functional.instance_norm(xf, None, None, None if weight is None else weight.float(),
                                          None if bias is None else bias.float(), True, 0.0, eps)
    if act == "gelu":
        y = torch.nn.functional.gelu(y, approximate=_ext.gelu_approximation())
    return y.to(x.dtype)


def channel_sums(x: torch.Tensor) -> torch.Tensor:
    """sum over (batch, H, W) of a 4-D activation in fp32 (bias gradients)."""
    if cl_supported(x):
        ext = _ext.require()
        B, C = x.shape[0], x.shape[1]
        sums = torch.zeros(B, C, 2, dtype=torch.float32, device=x.device)
        ext.inorm_cl_sums(x, None, None, None, None, sums, None, None, B, C, 0, 0)
        return sums[..., 0].sum(0)
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
        ext = _ext.require()
        B, C = x.shape[0], x.shape[1]
        sums = torch.empty(B * C, 2, dtype=torch.float32, device=x.device)
        ext.inorm_partial_stats(x, sums)
        return sums[:, 0].view(B, C).sum(0)
    return x.float().sum(dim=(0, 2, 3))
