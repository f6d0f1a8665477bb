"""AFNO spectral filter as a chain of tensor-core GEMMs: 2-D real FFT, block-diagonal complex two-layer MLP with ReLU,
soft shrinkage and inverse FFT of NHWC tokens, without cuFFT, einsum or a zero-filled spectrum buffer.

What it computes (makani/models/networks/afnonet.py:63-112 and afnonet_v2.py:77-112):

    X = rfft2(x, norm="ortho")                       x: [B, H, W, C] real
    X = X[kept rows kx, first `ncols` columns ky]    (mode window; everything outside counts as zero afterwards)
    O1 = relu_c(X W1 + b1),  O2 = softshrink_c(O1 W2 + b2)      per channel block; relu / shrink act on re and im separately
    y = irfft2(O2 placed back in the window, s=(H, W), norm="ortho") (+ skip)

How: each DFT is a real GEMM against a small constant cos / sin matrix (complex values travel as a (re, im) index
next to the channel index), restricted to the kept modes, so the window costs nothing and no full spectrum is ever
materialised; the block MLP is a batched GEMM over the blocks on 2x2 real block matrices with bias + ReLU and bias +
soft shrinkage in the epilogues; the inverse transforms are two more GEMMs and the skip is added in the last epilogue.
Six launches forward; the backward pass is the same four transform stages run with the transposed matrices (the DFT
matrices are orthogonal up to the Hermitian weights), two data-gradient GEMMs whose epilogues apply the ReLU / shrinkage
masks from the saved outputs, and two weight-gradient GEMMs.  The intermediate layouts are chosen such that every
operand of every GEMM has one uniform stride along its contraction index:

    T1 [B, ky, h, ri, C]   Y [B*ky*kx, blk, ri, bs]   O1 [B*ky*kx, blk, 2*hid]   O2 [B*ky, blk, kx, ri, bs]   T4 [h, B*ky, ri, C]

On CPU tensors the same calls run through the GEMM emulator, which is how the layout choreography is tested
without a GPU.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

from . import _ext
from .gemm import (ACT_DRELU, ACT_DSHRINK, ACT_NONE, ACT_RELU, ACT_SHRINK, BIAS_COL, Operand, Output, gemm, pad_to)

_PLANS = {}


class AFNOPlan:
    """Constant DFT matrices for one (H, W, kept rows, kept columns) geometry on one device / dtype."""

    def __init__(self, H: int, W: int, kx: Sequence[int], ncols: int, device, dtype):
        self.H, self.W, self.kx, self.ncols = H, W, tuple(int(k) for k in kx), int(ncols)
        self.nkx = len(self.kx)
        f64 = torch.float64
        w = torch.arange(W, dtype=f64)
        ky = torch.arange(ncols, dtype=f64)
        th = 2.0 * math.pi * ky[:, None] * w[None, :] / W                      # [ncols, W]
        sw = 1.0 / math.sqrt(W)
        fw = torch.stack([torch.cos(th) * sw, -torch.sin(th) * sw], dim=1).reshape(2 * ncols, W)
        # inverse along W (complex -> real, Hermitian weights: 1 for ky = 0 and the Nyquist column, else 2)
        cw = torch.full((ncols,), 2.0, dtype=f64)
        cw[0] = 1.0
        if W % 2 == 0 and ncols > W // 2:
            cw[W // 2] = 1.0
        gw = torch.stack([torch.cos(th) * (cw[:, None] * sw), -torch.sin(th) * (cw[:, None] * sw)], dim=1).reshape(2 * ncols, W).t()
        h = torch.arange(H, dtype=f64)
        kxv = torch.tensor(self.kx, dtype=f64)
        ph = 2.0 * math.pi * kxv[:, None] * h[None, :] / H                      # [nkx, H]
        sh = 1.0 / math.sqrt(H)
        c, s = torch.cos(ph) * sh, torch.sin(ph) * sh
        # rows (kx, ri'), columns (h, ri):  Y = sum_h T[h] exp(-i ph)
        fh = torch.stack([torch.stack([c, s], dim=-1), torch.stack([-s, c], dim=-1)], dim=1).reshape(2 * self.nkx, 2 * H)

        def prep(m):
            rows, cols = m.shape
            out = torch.zeros(rows, pad_to(cols, 8), dtype=dtype, device=device)
            out[:, :cols] = m.to(dtype)
            return out

        self.fw, self.fw_t = prep(fw), prep(fw.t())           # [2 ncols, W],  [W, 2 ncols]
        self.gw, self.gw_t = prep(gw), prep(gw.t())           # [W, 2 ncols],  [2 ncols, W]
        self.fh, self.gh = prep(fh), prep(fh.t())             # [2 nkx, 2 H],  [2 H, 2 nkx]  (inverse = transpose)

    @staticmethod
    def get(H, W, kx, ncols, device, dtype) -> "AFNOPlan":
        key = (H, W, tuple(kx), ncols, str(device), dtype)
        plan = _PLANS.get(key)
        if plan is None:
            plan = _PLANS[key] = AFNOPlan(H, W, kx, ncols, device, dtype)
        return plan


def mode_window_v1(H: int, W: int, fraction: float) -> Tuple[Tuple[int, ...], int]:
    """Rows [total - kept, total + kept) (clipped to the grid) and the first `kept` columns, total = H // 2 + 1
    (makani/models/networks/afnonet.py:78-81)."""
    total = H // 2 + 1
    kept = int(total * fraction)
    return tuple(range(max(total - kept, 0), min(total + kept, H))), min(kept, W // 2 + 1)


def mode_window_v2(H: int, W: int, fraction: float) -> Tuple[Tuple[int, ...], int]:
    """The `kept` lowest and `kept` highest rows (all rows at fraction 1) and the first int((W // 2 + 1) * fraction)
    columns (makani/models/networks/afnonet_v2.py:83-103)."""
    th, tw = H // 2 + 1, W // 2 + 1
    kh, kw = int(th * fraction), int(tw * fraction)
    if kh == th:
        return tuple(range(H)), kw
    return tuple(list(range(kh)) + list(range(H - kh, H))), kw


# ---------------------------------------------------------------------------------------------- the four transform stages

def _stage_w_analysis(x, mat, plan: AFNOPlan):
    """x [B, H, W, C] -> [B, ncols, H, 2, C]: `mat` [2 ncols, W] applied along W, per (b, h) row."""
    B, H, W, C = x.shape
    nc = plan.ncols
    out = torch.empty(B, nc, H, 2, C, dtype=x.dtype, device=x.device)
    gemm(2 * nc, C, W, Operand(mat, ld=mat.shape[1]), Operand(x, ld=C, mn_major=True, zs_lo=W * C, zs_hi=H * W * C),
         Output(out, rs_lo=C, rdiv=2, rs_hi=H * 2 * C, d_zlo=2 * C, d_zhi=nc * H * 2 * C), zlo_n=H, zhi_n=B)
    return out


def _stage_h_blocks(src, mat, plan: AFNOPlan, B, C, nb):
    """src [B*ncols, nb, nkx, 2, bs] -> [H, B*ncols, 2, C]: `mat` [2 H, 2 nkx] applied along kx, per (b, ky, block)."""
    H, nc, nkx = plan.H, plan.ncols, plan.nkx
    bs = C // nb
    out = torch.empty(H, B * nc, 2, C, dtype=src.dtype, device=src.device)
    gemm(2 * H, bs, 2 * nkx, Operand(mat, ld=mat.shape[1]),
         Operand(src, ld=bs, mn_major=True, zs_lo=nkx * 2 * bs, zs_hi=nb * nkx * 2 * bs),
         Output(out, rs_lo=C, rdiv=2, rs_hi=B * nc * 2 * C, d_zlo=bs, d_zhi=2 * C), zlo_n=nb, zhi_n=B * nc)
    return out


def _stage_w_synthesis(src, mat, plan: AFNOPlan, B, C, resid):
    """src [H, B*ncols, 2, C] -> [B, H, W, C]: `mat` [W, 2 ncols] applied along (ky, ri), per (b, h); + resid."""
    H, W, nc = plan.H, plan.W, plan.ncols
    out = torch.empty(B, H, W, C, dtype=src.dtype, device=src.device)
    gemm(W, C, 2 * nc, Operand(mat, ld=mat.shape[1]),
         Operand(src, ld=C, mn_major=True, zs_lo=B * nc * 2 * C, zs_hi=nc * 2 * C),
         Output(out, rs_lo=C, d_zlo=W * C, d_zhi=H * W * C), zlo_n=H, zhi_n=B, resid=resid)
    return out


def _stage_h_tokens(t1, plan: AFNOPlan, B, C, nb):
    """t1 [B, ncols, H, 2, C] -> token-major spectrum Y [B*ncols*nkx, nb, 2, bs] (forward DFT along H)."""
    H, nc, nkx = plan.H, plan.ncols, plan.nkx
    bs = C // nb
    y = torch.empty(B * nc * nkx, nb, 2, bs, dtype=t1.dtype, device=t1.device)
    gemm(2 * nkx, C, 2 * H, Operand(plan.fh, ld=plan.fh.shape[1]),
         Operand(t1, ld=C, mn_major=True, zs_lo=H * 2 * C, zs_hi=nc * H * 2 * C),
         Output(y, rs_lo=bs, rdiv=2, rs_hi=2 * C, ndiv=bs, ns_hi=2 * bs, d_zlo=nkx * 2 * C, d_zhi=nc * nkx * 2 * C),
         zlo_n=nc, zhi_n=B)
    return y


class _AFNOFilter(torch.autograd.Function):
    """y = irfft2(softshrink(relu(rfft2(x) W1 + b1) W2 + b2)) (+ skip) on the kept modes.

    w1x [nb, 2 hid, 2 bs] and w2x [nb, 2 bs, 2 hid] are the real 2x2-block forms of the complex block weights (rows: output
    (ri, o), columns: input (ri, i)); b1x [nb, 2 hid] / b2x [nb, 2 bs] the stacked (re, im) biases or None."""

    @staticmethod
    def forward(ctx, x, w1x, b1x, w2x, b2x, skip, plan, lam):
        B, H, W, C = x.shape
        nb = w1x.shape[0]
        bs, hid = C // nb, w1x.shape[1] // 2
        nc, nkx = plan.ncols, plan.nkx
        T = B * nc * nkx
        dt = x.dtype
        w1q, w2q = w1x.detach().to(dt).contiguous(), w2x.detach().to(dt).contiguous()
        b1f = b1x.detach().float().contiguous() if b1x is not None else None
        b2f = b2x.detach().float().contiguous() if b2x is not None else None
        t1 = _stage_w_analysis(x, plan.fw, plan)
        y = _stage_h_tokens(t1, plan, B, C, nb)
        o1 = torch.empty(T, nb, 2 * hid, dtype=dt, device=x.device)
        gemm(T, 2 * hid, 2 * bs, Operand(y, ld=2 * C, zs_lo=2 * bs), Operand(w1q, ld=2 * bs, zs_lo=2 * hid * 2 * bs),
             Output(o1, rs_lo=nb * 2 * hid, d_zlo=2 * hid), zlo_n=nb, bias=b1f, bias_mode=BIAS_COL, bias_zs=2 * hid, act=ACT_RELU)
        o2 = torch.empty(B * nc, nb, nkx, 2, bs, dtype=dt, device=x.device)
        gemm(T, 2 * bs, 2 * hid, Operand(o1, ld=nb * 2 * hid, zs_lo=2 * hid), Operand(w2q, ld=2 * hid, zs_lo=2 * bs * 2 * hid),
             Output(o2, rs_lo=2 * bs, rdiv=nkx, rs_hi=nb * nkx * 2 * bs, d_zlo=nkx * 2 * bs), zlo_n=nb, bias=b2f,
             bias_mode=BIAS_COL, bias_zs=2 * bs, act=ACT_SHRINK, act_param=float(lam))
        t4 = _stage_h_blocks(o2, plan.gh, plan, B, C, nb)
        out = _stage_w_synthesis(t4, plan.gw, plan, B, C, skip)
        ctx.save_for_backward(y, o1, o2, w1q, w2q)
        ctx.plan, ctx.dims = plan, (B, C, nb, bs, hid)
        # skip_is_x: the skip is the input itself (the usual residual form); its gradient then rides in the epilogue of
        # the last backward GEMM instead of a separate elementwise add
        ctx.flags = (b1x is not None, b2x is not None, skip is not None, skip is x)
        return out

    @staticmethod
    def backward(ctx, dy):
        y, o1, o2, w1q, w2q = ctx.saved_tensors
        plan = ctx.plan
        B, C, nb, bs, hid = ctx.dims
        has_b1, has_b2, has_skip, skip_is_x = ctx.flags
        H, nc, nkx = plan.H, plan.ncols, plan.nkx
        T = B * nc * nkx
        dy = dy.contiguous()
        dt = dy.dtype
        dev = dy.device
        # adjoint of the synthesis along W, then along H with the shrinkage mask (saved output != 0) in the epilogue
        dt4 = _stage_w_analysis(dy, plan.gw_t, plan)                                   # [B, ncols, H, 2, C]
        do2 = torch.empty_like(o2)
        gemm(2 * nkx, bs, 2 * H, Operand(plan.fh, ld=plan.fh.shape[1]),
             Operand(dt4, ld=C, mn_major=True, zs_lo=bs, zs_hi=H * 2 * C),
             Output(do2, rs_lo=bs, d_zlo=nkx * 2 * bs, d_zhi=nb * nkx * 2 * bs), zlo_n=nb, zhi_n=B * nc,
             act=ACT_DSHRINK, resid=o2)
        # second layer: data gradient with the ReLU mask (saved output > 0), weight gradient summed over the (b, ky) batches
        do1 = torch.empty_like(o1)
        gemm(nkx, 2 * hid, 2 * bs, Operand(do2, ld=2 * bs, zs_lo=nkx * 2 * bs, zs_hi=nb * nkx * 2 * bs),
             Operand(w2q, ld=2 * hid, mn_major=True, zs_lo=2 * bs * 2 * hid),
             Output(do1, rs_lo=nb * 2 * hid, d_zlo=2 * hid, d_zhi=nkx * nb * 2 * hid), zlo_n=nb, zhi_n=B * nc,
             act=ACT_DRELU, resid=o1)
        dw2 = torch.zeros(nb, 2 * bs, 2 * hid, dtype=torch.float32, device=dev)
        gemm(2 * bs, 2 * hid, nkx, Operand(do2, ld=2 * bs, mn_major=True, zs_lo=nkx * 2 * bs, zs_hi=nb * nkx * 2 * bs),
             Operand(o1, ld=nb * 2 * hid, mn_major=True, zs_lo=2 * hid, zs_hi=nkx * nb * 2 * hid),
             Output(dw2, rs_lo=2 * hid, d_zlo=2 * bs * 2 * hid), zlo_n=nb, zhi_n=B * nc, accumulate=True)
        db2 = do2.reshape(B * nc, nb, nkx, 2 * bs).float().sum(dim=(0, 2)) if has_b2 else None
        # first layer
        dyt = torch.empty(B * nc, nb, nkx, 2, bs, dtype=dt, device=dev)
        gemm(T, 2 * bs, 2 * hid, Operand(do1, ld=nb * 2 * hid, zs_lo=2 * hid),
             Operand(w1q, ld=2 * bs, mn_major=True, zs_lo=2 * hid * 2 * bs),
             Output(dyt, rs_lo=2 * bs, rdiv=nkx, rs_hi=nb * nkx * 2 * bs, d_zlo=nkx * 2 * bs), zlo_n=nb)
        dw1 = torch.zeros(nb, 2 * hid, 2 * bs, dtype=torch.float32, device=dev)
        tiles = nb * ((2 * hid + 127) // 128)
        splits = max(1, min((T + 63) // 64, (2 * _ext.sm_count() + tiles - 1) // tiles))
        gemm(2 * hid, 2 * bs, T, Operand(do1, ld=nb * 2 * hid, mn_major=True, zs_lo=2 * hid),
             Operand(y, ld=2 * C, mn_major=True, zs_lo=2 * bs),
             Output(dw1, rs_lo=2 * bs, d_zlo=2 * hid * 2 * bs), zlo_n=nb, accumulate=True, splits=splits)
        db1 = do1.float().sum(dim=0) if has_b1 else None
        # adjoint of the analysis along H and along W; the skip's gradient joins in the last epilogue
        dt1 = _stage_h_blocks(dyt, plan.gh, plan, B, C, nb)                            # [H, B*ncols, 2, C]
        dx = _stage_w_synthesis(dt1, plan.fw_t, plan, B, C, dy if skip_is_x else None)
        return dx, dw1, db1, dw2, db2, (dy if (has_skip and not skip_is_x) else None), None, None


def expand_complex_weight(wr: torch.Tensor, wi: torch.Tensor) -> torch.Tensor:
    """Complex block weights [nb, in, out] (real and imaginary parts) -> real block form [nb, 2 out, 2 in] with rows
    (ri', o), columns (ri, i): [[wr^T, -wi^T], [wi^T, wr^T]].  Plain torch, so autograd carries the gradient back."""
    wrt, wit = wr.transpose(1, 2), wi.transpose(1, 2)
    return torch.cat([torch.cat([wrt, -wit], dim=2), torch.cat([wit, wrt], dim=2)], dim=1)


def fast_path_ok(x: torch.Tensor, nb: int, hid: int) -> bool:
    if not _ext.native() or x.dim() != 4 or not x.is_contiguous():
        return False
    C = x.shape[-1]
    if C % nb or (C // nb) % 8 or hid % 8:
        return False
    if x.is_cuda:
        return x.dtype == torch.bfloat16
    return x.dtype in (torch.float32, torch.float64)


def afno_filter(x, w1r, w1i, b1r, b1i, w2r, w2i, b2r, b2i, kx: Sequence[int], ncols: int, lam: float,
                skip: Optional[torch.Tensor] = None) -> torch.Tensor:
    """NHWC tokens x [B, H, W, C]; block weights w1 [nb, bs, hid], w2 [nb, hid, bs] and biases b1 [nb, hid], b2 [nb, bs]
    given as real / imaginary parts (biases may be None); `kx` the kept rows and `ncols` the kept columns of the
    half-spectrum; `skip` (same shape as x) is added to the result."""
    B, H, W, C = x.shape
    plan = AFNOPlan.get(H, W, tuple(kx), int(ncols), x.device, x.dtype)
    w1x, w2x = expand_complex_weight(w1r, w1i), expand_complex_weight(w2r, w2i)
    b1x = torch.cat([b1r, b1i], dim=1) if b1r is not None else None
    b2x = torch.cat([b2r, b2i], dim=1) if b2r is not None else None
    return _AFNOFilter.apply(x, w1x, b1x, w2x, b2x, skip, plan, float(lam))


_ROW_INDEX = {}


def _row_index(kx, device):
    """Kept-row indices as a device tensor, created once per (rows, device) so that no host-to-device copy happens inside
    a CUDA-graph capture."""
    key = (kx, str(device))
    if key not in _ROW_INDEX:
        _ROW_INDEX[key] = torch.as_tensor(list(kx), device=device)
    return _ROW_INDEX[key]


def afno_filter_reference(x, w1r, w1i, b1r, b1i, w2r, w2i, b2r, b2i, kx, ncols, lam, skip=None):
    """The same operator with torch.fft and einsum in fp32 (fallback for layouts the GEMM chain does not take, and the
    oracle of the tests)."""
    B, H, W, C = x.shape
    nb = w1r.shape[0]
    bs = C // nb
    xf = torch.fft.rfft2(x.float(), dim=(1, 2), norm="ortho").reshape(B, H, W // 2 + 1, nb, bs)
    idx = _row_index(tuple(kx), x.device)
    xs = xf[:, idx][:, :, :ncols]
    mul = lambda a, w: torch.einsum("...bi,bio->...bo", a, w.float())
    zero = 0.0
    o1r = torch.relu(mul(xs.real, w1r) - mul(xs.imag, w1i) + (b1r.float() if b1r is not None else zero))
    o1i = torch.relu(mul(xs.imag, w1r) + mul(xs.real, w1i) + (b1i.float() if b1i is not None else zero))
    o2r = mul(o1r, w2r) - mul(o1i, w2i) + (b2r.float() if b2r is not None else zero)
    o2i = mul(o1i, w2r) + mul(o1r, w2i) + (b2i.float() if b2i is not None else zero)
    o2 = torch.nn.functional.softshrink(torch.stack([o2r, o2i], dim=-1), lambd=lam)
    out = torch.zeros(B, H, W // 2 + 1, nb, bs, 2, dtype=torch.float32, device=x.device)
    win = torch.zeros(B, len(kx), W // 2 + 1, nb, bs, 2, dtype=torch.float32, device=x.device)
    win[:, :, :ncols] = o2
    out = out.index_copy(1, idx, win)
    y = torch.fft.irfft2(torch.view_as_complex(out).reshape(B, H, W // 2 + 1, C), s=(H, W), dim=(1, 2), norm="ortho").to(x.dtype)
    return y + skip if skip is not None else y
