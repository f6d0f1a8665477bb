"""Channel-parallel pointwise linear map with the reduction fused into the GEMMs (peer memory, one NVSwitch node).

The reference's `DistributedMatmul` (makani/mpu/layers.py:221-270) computes a local GEMM on weights sharded
`[out / fout, in / fin]` and then all-reduces the partial products over the input-feature group with NCCL (forward) and
the input gradients over the output-feature group (backward).  Here the GEMM's epilogue stores each finished tile of the
partial product into the segment it owns in every group member's buffer (stores over NVLink while the next tile is
being computed) and a second kernel adds the segments up (plus bias) locally: an all-gather of partial products
executed by the producer, which moves the same bytes as a reduce-scatter + all-gather at group size 2 (the recipe
sizes, fin = fout = 2) and needs no NCCL call.  The backward input gradient uses the same pair of kernels over the
other group; the weight gradient is local.  Activations are bf16 channels-last.
"""

from __future__ import annotations

import torch

from ..parallel import peer
from ..utils import comm
from . import _ext
from .conv import CL, _canon, _chan_sum, _conv_dgrad, _conv_fwd, _conv_wgrad, layout_of, prep_weight
from .gemm import ACT_NONE


def supported(x: torch.Tensor, w: torch.Tensor, inp_group: str, out_group: str) -> bool:
    """CUDA bf16 channels-last input, 8-aligned local channel counts, groups that can map each other's memory."""
    if not (_ext.native() and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and layout_of(x) == CL):
        return False
    if w.shape[0] % 8 or w.shape[1] % 8:
        return False
    import torch.distributed as dist
    for g in (inp_group, out_group):
        n = comm.get_size(g)
        if n > 8 or (n > 1 and dist.get_backend(comm.get_group(g)) != "nccl"):
            return False
    return comm.get_size(inp_group) > 1 or comm.get_size(out_group) > 1


def _start_reduced_conv(name, group, run, B, C, H, W, dtype, device):
    """Launches `run(out, sync, dests)` (a GEMM that writes a [B, C, H, W] channels-last partial result, delivering its
    tiles to every member of `group`) and returns a handle for `_finish_reduced_conv`."""
    n = comm.get_size(group)
    if n == 1:
        y = torch.empty(B, C, H, W, dtype=dtype, device=device, memory_format=torch.channels_last)
        run(y, None, None)
        return None, y
    slot = peer.get_slot(name, group, B * C * H * W * torch.empty((), dtype=dtype).element_size(), device)
    part = slot.tensor(dtype, (B, H, W, C)).permute(0, 3, 1, 2)          # channels-last view of this rank's segment
    run(part, peer.sync_descriptor(produce=slot), slot.dests())
    return slot, (B, C, H, W, dtype, device)


def _finish_reduced_conv(handle, bias=None):
    """Sum of the partial results over the group (+ bias).  Work launched between start and finish overlaps the
    arrival of the peers' tiles."""
    slot, rest = handle
    if slot is None:
        y = rest
        if bias is not None:
            y = y + bias.to(y.dtype).view(1, -1, 1, 1)
        return y
    B, C, H, W, dtype, device = rest
    y = torch.empty(B, C, H, W, dtype=dtype, device=device, memory_format=torch.channels_last)
    slot.reduce_into(y, bias, C)
    return y


def _reduced_conv(name, group, run, B, C, H, W, dtype, device, bias=None):
    return _finish_reduced_conv(_start_reduced_conv(name, group, run, B, C, H, W, dtype, device), bias)


class _FusedDistMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, inp_group, out_group):
        wq = prep_weight(w, x.dtype)
        ci, co = w.shape[1], w.shape[0]
        B, _, H, W = x.shape
        bias_f = bias.detach().float().reshape(-1).contiguous() if bias is not None else None

        def run(out, sync, dests):
            _conv_fwd(x, wq, ci, None, ACT_NONE, None, False, out_layout=CL, out=out, sync=sync, dests=dests)

        y = _reduced_conv("mm_fwd", inp_group, run, B, co, H, W, x.dtype, x.device, bias_f)
        ctx.save_for_backward(x, wq)
        ctx.meta = (ci, co, w.shape, inp_group, out_group, bias is not None, None if bias is None else bias.shape)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wq = ctx.saved_tensors
        ci, co, wshape, inp_group, out_group, has_bias, bshape = ctx.meta
        dy = _canon(dy)
        if layout_of(dy) != CL:
            dy = dy.contiguous(memory_format=torch.channels_last)
        B, _, H, W = dy.shape
        handle = None
        if ctx.needs_input_grad[0]:
            def run(out, sync, dests):
                _conv_dgrad(dy, wq, ci, x_layout=CL, out=out, sync=sync, dests=dests)

            handle = _start_reduced_conv("mm_bwd", out_group, run, B, ci, H, W, dy.dtype, dy.device)
        # the weight and bias gradients are local: they run while the peers' input-gradient tiles are still arriving
        # (what the reference's overlapped variant does with an asynchronous all-reduce, makani/mpu/layers.py:171-218)
        dw = _conv_wgrad(dy, x).reshape(wshape) if ctx.needs_input_grad[1] else None
        db = _chan_sum(dy).reshape(bshape) if has_bias and ctx.needs_input_grad[2] else None
        dx = _finish_reduced_conv(handle) if handle is not None else None
        return dx, dw, db, None, None


def fused_dist_matmul(x, w, bias, inp_group: str, out_group: str):
    """y = sum over `inp_group` of (x_local @ w_local^T) + bias;  dx = sum over `out_group` of (dy @ w_local)."""
    return _FusedDistMatmul.apply(x, w, bias, inp_group, out_group)
