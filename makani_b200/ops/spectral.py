"""Spherical-harmonic spectral convolution as a chain of tensor-core GEMMs.

The reference computes `x -> SHT -> per-degree complex contraction -> inverse SHT` with cuFFT plus cuBLAS
einsums in fp32 (makani/models/common/spectral_convolution.py:124-148, contractions.py:130-136, and the
torch-harmonics RealSHT/InverseRealSHT it imports).  Here every stage is one launch of the batched GEMM
engine, and each stage writes its result directly in the layout the next one reads, so no transpose or
truncation pass ever touches HBM:

    x  [B, H, W, C]                  real grid data, channels-last (bf16)
    S1 longitude DFT      -> T1 [B, H, (m,ri), C]       A = DFT matrix [(m,ri), W], batched over latitude rows
    S2 Legendre analysis  -> T2 [B, l, m, (ri, C)]      A = P_l^m(theta_k) w_k, batched over m, rows l < m skipped
    S3 complex contraction-> T3 [B, m, l, (ri, Co)]     B = W_l as a real 2x2-block matrix, batched over l, rows m > l skipped
    S4 Legendre synthesis -> T4 [B, H', (m,ri), Co]     k-loop restricted to l >= m
    S5 inverse DFT        -> y  [B, H', W', Co]

(ri = real/imaginary part; the Legendre tables are padded along latitude to 16-byte TMA strides.)
The adjoints used by the backward pass are the same five launches with the constant operands read in the
other major (no transposed copies of the tables are stored).
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..sht.legendre import legendre_table
from ..sht.quadrature import precompute_latitudes
from . import _ext
from .gemm import Operand, Output, Tri, gemm, pad_to


class SHTPlan:
    """Constant operands (DFT matrices, Legendre tables) for one (nlat, nlon, lmax, mmax, grid) transform pair."""

    _cache: Dict[Tuple, "SHTPlan"] = {}

    def __init__(self, nlat: int, nlon: int, lmax: int, mmax: int, grid: str, device, dtype=torch.bfloat16):
        self.nlat, self.nlon, self.lmax, self.mmax, self.grid = nlat, nlon, lmax, mmax, grid
        self.device, self.dtype = torch.device(device), dtype
        self.hp = pad_to(nlat, 8)          # padded latitude extent of T1/T4 rows and of the tables
        self.k2 = 2 * mmax                 # DFT K extent (m, ri)
        self.k2p = pad_to(self.k2, 8)
        theta, wq = precompute_latitudes(nlat, grid)
        self.theta, self.wq = theta, wq
        p = legendre_table(mmax, lmax, theta)                     # [m, l, k] float64
        pw = p * wq[None, None, :]
        tab = np.zeros((2, mmax, lmax, self.hp), dtype=np.float32)
        tab[0, :, :, :nlat] = pw
        tab[1, :, :, :nlat] = p
        self.pw = torch.from_numpy(tab[0]).to(self.device, dtype).contiguous()   # analysis table (weighted)
        self.p = torch.from_numpy(tab[1]).to(self.device, dtype).contiguous()    # synthesis table
        # forward DFT rows (m, ri) ordered as ri-major: row = ri*mmax... no: row index j = 2*m + ri
        phi = 2.0 * np.pi * np.arange(nlon) / nlon
        m = np.arange(mmax)[:, None]
        ang = m * phi[None, :]
        f = np.zeros((self.k2, nlon), dtype=np.float64)
        f[0::2] = np.cos(ang) * (2.0 * np.pi / nlon)
        f[1::2] = -np.sin(ang) * (2.0 * np.pi / nlon)
        self.f = torch.from_numpy(f.astype(np.float32)).to(self.device, dtype).contiguous()      # [(m,ri), W]
        # inverse DFT: x_i = sum_m c_m (Xr cos - Xi sin); c_0 = 1, c_m = 2, Nyquist (if kept) = 1
        cm = np.full((mmax, 1), 2.0)
        cm[0] = 1.0
        if nlon % 2 == 0 and mmax > nlon // 2:
            cm[nlon // 2] = 1.0
        g = np.zeros((nlon, self.k2p), dtype=np.float64)
        g[:, 0:self.k2:2] = (cm * np.cos(ang)).T
        g[:, 1:self.k2:2] = (-cm * np.sin(ang)).T
        self.gt = torch.from_numpy(g.astype(np.float32)).to(self.device, dtype).contiguous()     # [W, (m,ri) padded]

    @classmethod
    def get(cls, nlat, nlon, lmax, mmax, grid, device, dtype=torch.bfloat16) -> "SHTPlan":
        key = (nlat, nlon, lmax, mmax, grid, str(torch.device(device)), dtype)
        plan = cls._cache.get(key)
        if plan is None:
            plan = cls(nlat, nlon, lmax, mmax, grid, device, dtype)
            cls._cache[key] = plan
        return plan


# ------------------------------------------------------------------------------------------------ stages
# Activations are channels-last: x is logically [B, C, H, W] and physically [B][k][i][c] (k latitude, i longitude).
# Row index of the DFT side is j = 2*m + ri.  T1 / T4 are [B, H, 2*mmax, C]; T2 is [B, l, m, (ri, C)];
# T3 is [B, m, l, (ri, Co)].


def _to_cl(x: torch.Tensor) -> torch.Tensor:
    if x.is_contiguous(memory_format=torch.channels_last) and not (x.is_contiguous() and x.shape[1] != 1):
        return x
    return x.contiguous(memory_format=torch.channels_last)


def dft_analysis(x: torch.Tensor, mat: torch.Tensor, mat_mn: bool, mat_ld: int, k2: int) -> torch.Tensor:
    """T1[b, k, j, c] = sum_i M[j, i] x[b, c, k, i];  M given K-major ([j, i]) or MN-major ([i, j])."""
    B, C, H, W = x.shape
    t1 = torch.empty(B, H, k2, C, dtype=x.dtype, device=x.device)
    gemm(k2, C, W,
         Operand(mat, ld=mat_ld, mn_major=mat_mn),
         Operand(x, ld=C, mn_major=True, zs_lo=W * C, zs_hi=H * W * C),
         Output(t1, rs_lo=C, d_zlo=k2 * C, d_zhi=H * k2 * C),
         zlo_n=H, zhi_n=B, bn=128 if C <= 128 or C % 256 != 0 else 256)
    return t1


def dft_synthesis(t4: torch.Tensor, mat: torch.Tensor, mat_mn: bool, mat_ld: int, W: int) -> torch.Tensor:
    """y[b, c, k, i] = sum_j T4[b, k, j, c] M[i, j];  M given K-major ([i, j]) or MN-major ([j, i]).  y is channels-last."""
    B, H, k2, C = t4.shape
    y = torch.empty(B, C, H, W, dtype=t4.dtype, device=t4.device, memory_format=torch.channels_last)
    gemm(W, C, k2,
         Operand(mat, ld=mat_ld, mn_major=mat_mn),
         Operand(t4, ld=C, mn_major=True, zs_lo=k2 * C, zs_hi=H * k2 * C),
         Output(y, rs_lo=C, d_zlo=W * C, d_zhi=H * W * C),
         zlo_n=H, zhi_n=B, bn=128 if C <= 128 or C % 256 != 0 else 256)
    return y


def legendre_analysis(t1: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """T2[b, l, m, n] = sum_k table[m, l, k] T1[b, k, m, n], n = (ri, c);  zero for l < m."""
    B, H, k2, C = t1.shape
    mmax, lmax, hpt = table.shape
    n2 = 2 * C
    t2 = torch.empty(B, lmax, mmax, n2, dtype=t1.dtype, device=t1.device)
    gemm(lmax, n2, H,
         Operand(table, ld=hpt, zs_hi=lmax * hpt),
         Operand(t1, ld=k2 * C, mn_major=True, zs_hi=n2, zs_lo=H * k2 * C),
         Output(t2, rs_lo=mmax * n2, d_zhi=n2, d_zlo=lmax * mmax * n2),
         zhi_n=mmax, zlo_n=B, tri=Tri(rmin_a=1))
    return t2


def legendre_synthesis(t: torch.Tensor, lm_order: bool, table: torch.Tensor, H: int) -> torch.Tensor:
    """T4[b, k, m, n] = sum_l table[m, l, k] T[b, ., ., n]  with T given as [b, m, l, n] (lm_order False)
    or [b, l, m, n] (lm_order True); only l >= m contributes."""
    if lm_order:
        B, lmax, mmax, n2 = t.shape
        ld, zs_m = mmax * n2, n2
    else:
        B, mmax, lmax, n2 = t.shape
        ld, zs_m = n2, lmax * n2
    hpt = table.shape[2]
    t4 = torch.empty(B, H, 2 * mmax, n2 // 2, dtype=t.dtype, device=t.device)
    gemm(H, n2, lmax,
         Operand(table, ld=hpt, mn_major=True, zs_hi=lmax * hpt),
         Operand(t, ld=ld, mn_major=True, zs_hi=zs_m, zs_lo=lmax * mmax * n2),
         Output(t4, rs_lo=mmax * n2, d_zhi=n2, d_zlo=H * mmax * n2),
         zhi_n=mmax, zlo_n=B, tri=Tri(kmin_a=1))
    return t4


def contract(t2: torch.Tensor, wx: torch.Tensor, transpose_w: bool) -> torch.Tensor:
    """T3[b, m, l, q] = sum_p T2[b, l, m, p] Wx[l, q, p]   (transpose_w False; Wx [l, 2Co, 2Ci])
       T3[b, m, l, p] = sum_q T2[b, l, m, q] Wx[l, q, p]   (transpose_w True: adjoint w.r.t. the input)."""
    B, lmax, mmax, kin = t2.shape
    nq, npp = wx.shape[1], wx.shape[2]
    nout = npp if transpose_w else nq
    t3 = torch.empty(B, mmax, lmax, nout, dtype=t2.dtype, device=t2.device)
    gemm(mmax, nout, kin,
         Operand(t2, ld=kin, zs_hi=mmax * kin, zs_lo=lmax * mmax * kin),
         Operand(wx, ld=npp, mn_major=transpose_w, zs_hi=nq * npp),
         Output(t3, rs_lo=lmax * nout, d_zhi=nout, d_zlo=mmax * lmax * nout),
         zhi_n=lmax, zlo_n=B, tri=Tri(rmax_a=1, rmax_b=1))
    return t3


def contract_wgrad2(dt: torch.Tensor, t2: torch.Tensor, l0: int = 0, m0: int = 0) -> torch.Tensor:
    """(dWr, dWi)[l, o, c] as fp32 [2, L, Co, Ci] without forming the full real 2x2-block gradient:

        dWr[l, o, c] = sum_{b, m <= l} dTr T2r + dTi T2i        dWi[l, o, c] = sum_{b, m <= l} dTi T2r - dTr T2i

    Both are GEMMs over k = (m, ri) (the two parts sit side by side in memory); the second one reads a copy of dT
    with its parts swapped and one sign flipped.  `l0`, `m0`: global offsets of the local (l, m) block."""
    B, L, M, nq = dt.shape
    co, ci = nq // 2, t2.shape[3] // 2
    if dt.is_cuda and dt.dtype == torch.bfloat16 and co % 8 == 0 and dt.is_contiguous() and _ext.native():
        dts = torch.empty_like(dt)
        _ext.require().swap_ri(dt, dts, co)
    else:
        d5 = dt.view(B, L, M, 2, co)
        dts = torch.cat([d5[..., 1:2, :], -d5[..., 0:1, :]], dim=-2).contiguous()
    out = (torch.empty if B == 1 else torch.zeros)(2, L, co, ci, dtype=torch.float32, device=dt.device)
    tri = Tri(kmax_a=2, kmax_b=2 * (1 + l0 - m0))
    for part, a in enumerate((dt, dts)):
        gemm(co, ci, 2 * M,
             Operand(a, ld=co, mn_major=True, zs_hi=M * nq, zs_lo=L * M * nq),
             Operand(t2, ld=ci, mn_major=True, zs_hi=M * 2 * ci, zs_lo=L * M * 2 * ci),
             Output(out, rs_lo=ci, offset=part * L * co * ci, d_zhi=co * ci),
             zhi_n=L, zlo_n=B, accumulate=(B > 1), tri=tri)
    return out


def fold_weight_grad2(dw2: torch.Tensor) -> torch.Tensor:
    """fp32 [2, L, Co, Ci] = (dWr, dWi) -> complex64 [Ci, Co, L]."""
    _, L, co, ci = dw2.shape
    if dw2.is_cuda and _ext.native():
        dw = torch.empty(ci, co, L, dtype=torch.complex64, device=dw2.device)
        _ext.require().spectral_fold(dw2, dw, True, True)
        return dw
    return torch.complex(dw2[0], dw2[1]).permute(2, 1, 0).contiguous()


# ------------------------------------------------------------------------------------------------ weights


# Inference re-uses the expanded weights: they are cached per parameter while gradients are disabled and dropped when
# the parameter is modified in place (`_version`) or by the fused optimiser, which writes through raw pointers and
# announces every update through `note_weights_changed`.
_WEIGHT_EPOCH = 0
_EXPANDED = {}


def note_weights_changed() -> None:
    global _WEIGHT_EPOCH
    _WEIGHT_EPOCH += 1
    _EXPANDED.clear()


def expand_weight(w: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """complex [Ci, Co, L] -> real [L, 2Co, 2Ci] with rows (ri', o), columns (ri, c):  [[Wr, -Wi], [Wi, Wr]]."""
    if not torch.is_grad_enabled() and w.is_cuda:
        key = (w.data_ptr(), tuple(w.shape), dtype)
        hit = _EXPANDED.get(key)
        if hit is not None and hit[0] == (w._version, _WEIGHT_EPOCH):
            return hit[1]
        wx = _expand_weight(w, dtype)
        _EXPANDED[key] = ((w._version, _WEIGHT_EPOCH), wx)
        return wx
    return _expand_weight(w, dtype)


def _expand_weight(w: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    ci, co, L = w.shape
    if w.is_cuda and dtype == torch.bfloat16:
        wx = torch.empty(L, 2 * co, 2 * ci, dtype=dtype, device=w.device)
        _ext.require().spectral_expand(w.detach().contiguous(), wx)
        return wx
    wr = w.real.permute(2, 1, 0)
    wi = w.imag.permute(2, 1, 0)
    top = torch.cat([wr, -wi], dim=2)
    bot = torch.cat([wi, wr], dim=2)
    return torch.cat([top, bot], dim=1).to(dtype).contiguous()


def fold_weight_grad(dwx: torch.Tensor) -> torch.Tensor:
    """fp32 [L, 2Co, 2Ci] -> complex64 [Ci, Co, L] gradient (dWr = d00 + d11, dWi = d10 - d01)."""
    L, co2, ci2 = dwx.shape
    co, ci = co2 // 2, ci2 // 2
    if dwx.is_cuda:
        dw = torch.zeros(ci, co, L, dtype=torch.complex64, device=dwx.device)
        _ext.require().spectral_fold(dwx.contiguous(), dw)
        return dw
    d00, d01 = dwx[:, :co, :ci], dwx[:, :co, ci:]
    d10, d11 = dwx[:, co:, :ci], dwx[:, co:, ci:]
    return torch.complex(d00 + d11, d10 - d01).permute(2, 1, 0).contiguous()


# ------------------------------------------------------------------------------------------------ autograd


class _SpectralConv(torch.autograd.Function):
    """y = iSHT_out(W . SHT_in(x)) and, when `want_resid`, r = iSHT_out(SHT_in(x)) (regridded residual).
    Input and outputs are channels-last."""

    @staticmethod
    def forward(ctx, x, w, plan_in: SHTPlan, plan_out: SHTPlan, want_resid: bool):
        x = _to_cl(x)
        wx = expand_weight(w, x.dtype)
        t1 = dft_analysis(x, plan_in.f, False, plan_in.nlon, plan_in.k2)
        t2 = legendre_analysis(t1, plan_in.pw)
        del t1
        t3 = contract(t2, wx, False)
        t4 = legendre_synthesis(t3, False, plan_out.p, plan_out.nlat)
        del t3
        y = dft_synthesis(t4, plan_out.gt, False, plan_out.k2p, plan_out.nlon)
        del t4
        r = None
        if want_resid:
            t4r = legendre_synthesis(t2, True, plan_out.p, plan_out.nlat)
            r = dft_synthesis(t4r, plan_out.gt, False, plan_out.k2p, plan_out.nlon)
        ctx.save_for_backward(t2, wx)
        ctx.plans = (plan_in, plan_out)
        ctx.want_resid = want_resid
        ctx.wshape = w.shape
        if want_resid:
            return y, r
        return y

    @staticmethod
    def backward(ctx, dy, dr=None):
        t2, wx = ctx.saved_tensors
        plan_in, plan_out = ctx.plans
        dy = _to_cl(dy)
        # adjoint of the inverse DFT / synthesis on the output grid
        dt4 = dft_analysis(dy, plan_out.gt, True, plan_out.k2p, plan_out.k2)
        dt3 = legendre_analysis(dt4, plan_out.p)                       # [B, l, m, (ri, o)]
        del dt4
        dw = None
        if ctx.needs_input_grad[1]:
            dw = fold_weight_grad2(contract_wgrad2(dt3, t2)).reshape(ctx.wshape)
        dx = None
        if ctx.needs_input_grad[0]:
            dt2 = contract(dt3, wx, True)                              # [B, m, l, (ri, c)]
            if ctx.want_resid and dr is not None:
                dr = _to_cl(dr)
                dr4 = dft_analysis(dr, plan_out.gt, True, plan_out.k2p, plan_out.k2)
                dr2 = legendre_analysis(dr4, plan_out.p)               # [B, l, m, n]
                dt2 = dt2 + dr2.transpose(1, 2)
                del dr4, dr2
            dt1 = legendre_synthesis(dt2.contiguous(), False, plan_in.pw, plan_in.nlat)
            dx = dft_synthesis(dt1, plan_in.f, True, plan_in.nlon, plan_in.nlon)
        return dx, dw, None, None, None


def spectral_conv_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (_ext.native() and x.dim() == 4 and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.dim() == 3 and w.shape[1] % 8 == 0
            and x.shape[3] % 8 == 0)


def spectral_conv_dhconv(x, w, plan_in: SHTPlan, plan_out: SHTPlan, want_resid: bool):
    """Fused spherical convolution with per-degree ("dhconv") complex weights on the GEMM engine."""
    return _SpectralConv.apply(x, w, plan_in, plan_out, want_resid)
