"""Spatially distributed spherical-harmonic convolution with the communication fused into the GEMMs.

The reference distributes the transforms with four all-to-all transposes per direction around local FFT /
Legendre kernels (torch-harmonics DistributedRealSHT / DistributedInverseRealSHT, imported at
makani/models/networks/sfnonet.py:30-36; the same choreography for the FFT case is spelled out in
makani/mpu/layers.py:66-101), i.e. eight NCCL all-to-alls plus eight transposing copies per spectral layer and
direction.  Here no transpose exists.  Grid data is sharded (latitude over group "h", longitude over group
"w"), coefficients are sharded (l over "h", m over "w"), and every transform stage is one launch of the batched
tcgen05 GEMM whose k loop walks over the peers of one group:

    S1  T1[b, k_loc, (m_loc, ri), c] = sum_{w-peers q} sum_{i in lon(q)} F[(m, ri), i] x_q[b, k_loc, i, c]
    S2  T2[b, l_loc, m_loc, (ri, c)] = sum_{h-peers q} sum_{k in lat(q)} Pw[m, l, k] T1_q[b, k, m, (ri, c)]
    S3  T3[b, m_loc, l_loc, (ri, o)] = per-degree complex contraction (local; weights are sharded in l)
    S4  T4[b, k_loc, (m_loc, ri), o] = sum_{h-peers q} sum_{l in l(q)} P[m, l, k] T3_q[b, m, l, (ri, o)]
    S5  y[b, k_loc, i_loc, o]        = sum_{w-peers q} sum_{m in m(q)} G[i, (m, ri)] T4_q[b, k_loc, (m, ri), o]

The stage that produces a buffer which peers need (x, T1, T3, T4) stores every finished tile from its epilogue
into its segment of every peer's copy of that buffer (plain stores / TMA stores over NVLink, no multicast), so
the all-gather happens tile by tile while the tensor cores work on the next tiles and each byte crosses NVLink
once per destination.  The consuming stage then walks its k loop over the segments of its own local copy
(re-reads hit local HBM / L2) and only computes the output slice it owns.  Producer/consumer ordering between
ranks uses the monotonic device counters of `makani_b200.parallel.peer` and is part of the same kernels.  On CPU
(gloo) the same code runs with an all-gather standing in for the peer stores, which is how the layout algebra is
tested without GPUs.
"""

from __future__ import annotations

import os
from typing import Dict, List, Tuple

import numpy as np
import torch

from ..parallel import peer
from ..parallel.helpers import compute_split_shapes
from ..sht.legendre import legendre_table
from ..sht.quadrature import precompute_latitudes
from . import _ext
from .gemm import Operand, Output, Segment, Tri, gemm, pad_to
from .spectral import _to_cl, contract_wgrad2, expand_weight, fold_weight_grad2

SEG_ALIGN = 64   # elements: one 128-byte k-slab of bf16
# MAKANI_B200_FUSED_DIST_SHT=0 falls back to the all-to-all formulation (for A/B timing of the two designs)
ENABLED = os.environ.get("MAKANI_B200_FUSED_DIST_SHT", "1") != "0"


def _seg_layout(shapes: List[int]) -> Tuple[List[int], int]:
    pos, total = [], 0
    for n in shapes:
        pos.append(total)
        total += pad_to(max(n, 1), SEG_ALIGN)
    return pos, total


def _scatter_k(mat: np.ndarray, shapes: List[int]) -> np.ndarray:
    """[..., K] -> [..., Kp] with the k axis cut into `shapes` and every piece placed at a 64-aligned position."""
    pos, total = _seg_layout(shapes)
    out = np.zeros(mat.shape[:-1] + (total,), dtype=mat.dtype)
    start = 0
    for n, p in zip(shapes, pos):
        out[..., p:p + n] = mat[..., start:start + n]
        start += n
    return out


class DistSHTPlan:
    """Constant operands of one rank for a transform pair on a (ph x pw) process grid."""

    _cache: Dict[Tuple, "DistSHTPlan"] = {}

    def __init__(self, nlat, nlon, lmax, mmax, grid, ph, pw, rh, rw, device, dtype=torch.bfloat16):
        self.nlat, self.nlon, self.lmax, self.mmax, self.grid = nlat, nlon, lmax, mmax, grid
        self.ph, self.pw, self.rh, self.rw = ph, pw, rh, rw
        self.device, self.dtype = torch.device(device), dtype
        self.lat_shapes = compute_split_shapes(nlat, ph)
        self.lon_shapes = compute_split_shapes(nlon, pw)
        self.l_shapes = compute_split_shapes(lmax, ph)
        self.m_shapes = compute_split_shapes(mmax, pw)
        off = lambda shapes, r: int(sum(shapes[:r]))
        self.lat0, self.lon0, self.l0, self.m0 = off(self.lat_shapes, rh), off(self.lon_shapes, rw), off(self.l_shapes, rh), off(self.m_shapes, rw)
        self.hl, self.wl, self.ll, self.ml = self.lat_shapes[rh], self.lon_shapes[rw], self.l_shapes[rh], self.m_shapes[rw]
        self.hmax, self.wmax, self.llmax, self.mlmax = max(self.lat_shapes), max(self.lon_shapes), max(self.l_shapes), max(self.m_shapes)
        self.hlp = pad_to(self.hl, 8)
        self.lat_pos, self.kh = _seg_layout(self.lat_shapes)
        self.lon_pos, self.kw = _seg_layout(self.lon_shapes)
        self.l_pos, self.kl = _seg_layout(self.l_shapes)
        self.j_shapes = [2 * m for m in self.m_shapes]
        self.j_pos, self.kj = _seg_layout(self.j_shapes)

        theta, wq = precompute_latitudes(nlat, grid)
        msl = slice(self.m0, self.m0 + self.ml)
        lsl = slice(self.l0, self.l0 + self.ll)
        ksl = slice(self.lat0, self.lat0 + self.hl)
        p = legendre_table(mmax, lmax, theta)[msl]                # [m_loc, l, k] float64
        pw_ = p * wq[None, None, :]
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.device, dtype).contiguous()
        # analysis form: rows l_loc, k = latitude of all ranks in padded segments
        self.pw_an = to(_scatter_k(pw_[:, lsl, :], self.lat_shapes))
        self.p_an = to(_scatter_k(p[:, lsl, :], self.lat_shapes))
        # synthesis form: rows (contiguous) = local latitudes, k = l of all ranks in padded segments
        def syn(tab):
            t = _scatter_k(np.swapaxes(tab[:, :, ksl], 1, 2), self.l_shapes)      # [m_loc, hl, Kl]
            out = np.zeros((self.ml, self.kl, self.hlp), dtype=np.float64)
            out[:, :, : self.hl] = np.swapaxes(t, 1, 2)
            return to(out)
        self.p_syn = syn(p)
        self.pw_syn = syn(pw_)

        phi = 2.0 * np.pi * np.arange(nlon) / nlon
        m = np.arange(mmax)[:, None]
        ang = m * phi[None, :]
        k2 = 2 * mmax
        f = np.zeros((k2, nlon))
        f[0::2] = np.cos(ang) * (2.0 * np.pi / nlon)
        f[1::2] = -np.sin(ang) * (2.0 * np.pi / nlon)
        cm = np.full((mmax, 1), 2.0)
        cm[0] = 1.0
        if nlon % 2 == 0 and mmax > nlon // 2:
            cm[nlon // 2] = 1.0
        g = np.zeros((nlon, k2))
        g[:, 0::2] = (cm * np.cos(ang)).T
        g[:, 1::2] = (-cm * np.sin(ang)).T
        jsl = slice(2 * self.m0, 2 * (self.m0 + self.ml))
        isl = slice(self.lon0, self.lon0 + self.wl)
        self.f_an = to(_scatter_k(f[jsl, :], self.lon_shapes))          # [(m_loc, ri), Kw]
        self.gt_an = to(_scatter_k(g.T[jsl, :], self.lon_shapes))       # adjoint of the inverse DFT
        self.g_syn = to(_scatter_k(g[isl, :], self.j_shapes))           # [i_loc, Kj]
        self.ft_syn = to(_scatter_k(f.T[isl, :], self.j_shapes))        # adjoint of the forward DFT

    @classmethod
    def get(cls, nlat, nlon, lmax, mmax, grid, ph, pw, rh, rw, device, dtype=torch.bfloat16) -> "DistSHTPlan":
        key = (nlat, nlon, lmax, mmax, grid, ph, pw, rh, rw, str(torch.device(device)), dtype)
        plan = cls._cache.get(key)
        if plan is None:
            plan = cls(nlat, nlon, lmax, mmax, grid, ph, pw, rh, rw, device, dtype)
            cls._cache[key] = plan
        return plan


# ------------------------------------------------------------------------------------------------ helpers


def _slot(name, group, nbytes, device, size):
    return peer.get_slot(name, group, nbytes, device) if size > 1 else None


def _dests(slot):
    return slot.dests() if slot is not None else None


def _segments(slot, shapes, pos, starts):
    return [Segment(src, n, p, g) for src, n, p, g in zip(slot.sources(), shapes, pos, starts)]


def _starts(shapes):
    out, s = [], 0
    for n in shapes:
        out.append(s)
        s += n
    return out


def _bn(C):
    return 128 if C <= 128 or C % 256 != 0 else 256


def _esz(dtype):
    return torch.empty((), dtype=dtype).element_size()


# ------------------------------------------------------------------------------------------------ stages
# Buffers read by peers use the group-wide maximum extents so that every rank's copy has the same strides:
#   XW [B, hl, wmax, C]   T1 [B, hmax, 2 ml, C]   T3 [B, ml, llmax, n2]   T2S [B, llmax, ml, n2]   T4 [B, hl, 2 mlmax, C]


def stage_grid_to_slot(x: torch.Tensor, plan: DistSHTPlan):
    """Places this rank's channels-last grid block where the longitude peers can read it."""
    B, C, hl, wl = x.shape
    if plan.pw == 1:
        return None, x
    slot = peer.get_slot("xw", "w", B * plan.hmax * plan.wmax * C * _esz(x.dtype), x.device)
    view = slot.tensor(x.dtype, (B, hl, plan.wmax, C))
    slot.publish(x, B * hl, wl * C, wl * C, plan.wmax * C)
    return slot, view


def stage_dft_analysis(xslot, xv, table, plan: DistSHTPlan, B, C):
    """S1 (or the adjoint of S5 with `table = gt_an`): longitude DFT onto this rank's orders."""
    hl, ml = plan.hl, plan.ml
    dev, dt = xv.device, xv.dtype
    k2 = 2 * ml
    t1slot = _slot("t1", "h", B * plan.hmax * 2 * plan.mlmax * C * _esz(dt), dev, plan.ph)
    if t1slot is None:
        t1 = torch.empty(B, hl, k2, C, dtype=dt, device=dev)
        hstride = hl
    else:
        t1 = t1slot.tensor(dt, (B, plan.hmax, k2, C))
        hstride = plan.hmax
    out = Output(t1, rs_lo=C, d_zlo=k2 * C, d_zhi=hstride * k2 * C)
    sync = peer.sync_descriptor(consume=xslot, produce=t1slot)
    if xslot is None:
        W = plan.nlon
        gemm(k2, C, W, Operand(table, ld=plan.kw), Operand(xv, ld=C, mn_major=True, zs_lo=W * C, zs_hi=hl * W * C),
             out, zlo_n=hl, zhi_n=B, bn=_bn(C), sync=sync, dests=_dests(t1slot))
    else:
        segs = _segments(xslot, plan.lon_shapes, plan.lon_pos, _starts(plan.lon_shapes))
        gemm(k2, C, plan.kw, Operand(table, ld=plan.kw),
             Operand(xv, ld=C, mn_major=True, zs_lo=plan.wmax * C, zs_hi=hl * plan.wmax * C),
             out, zlo_n=hl, zhi_n=B, bn=_bn(C), segments=segs, sync=sync, dests=_dests(t1slot))
    return t1slot, t1, hstride


def stage_legendre_analysis(t1slot, t1, hstride, table, plan: DistSHTPlan, B, C):
    """S2 (or the adjoint of S4 with `table = p_an`): T2[b, l_loc, m_loc, (ri, c)], zero where l < m."""
    ml, ll = plan.ml, plan.ll
    n2, k2 = 2 * C, 2 * ml
    t2 = torch.empty(B, ll, ml, n2, dtype=t1.dtype, device=t1.device)
    out = Output(t2, rs_lo=ml * n2, d_zhi=n2, d_zlo=ll * ml * n2)
    tri = Tri(rmin_a=1, rmin_b=plan.m0 - plan.l0)
    bop = Operand(t1, ld=k2 * C, mn_major=True, zs_hi=n2, zs_lo=hstride * k2 * C)
    aop = Operand(table, ld=plan.kh, zs_hi=ll * plan.kh)
    sync = peer.sync_descriptor(consume=t1slot)
    if t1slot is None:
        gemm(ll, n2, plan.nlat, aop, bop, out, zhi_n=ml, zlo_n=B, tri=tri)
    else:
        segs = _segments(t1slot, plan.lat_shapes, plan.lat_pos, _starts(plan.lat_shapes))
        gemm(ll, n2, plan.kh, aop, bop, out, zhi_n=ml, zlo_n=B, tri=tri, segments=segs, sync=sync)
    return t2


def t3_buffer(plan: DistSHTPlan, B, n2, dtype, device):
    slot = _slot("t3", "h", B * plan.mlmax * plan.llmax * n2 * _esz(dtype), device, plan.ph)
    if slot is None:
        return None, torch.empty(B, plan.ml, plan.ll, n2, dtype=dtype, device=device), plan.ll
    return slot, slot.tensor(dtype, (B, plan.ml, plan.llmax, n2)), plan.llmax


def stage_contract(t2, wx, transpose_w, plan: DistSHTPlan, private: bool = False):
    """S3: per-degree complex contraction of this rank's (l, m) block, written where the latitude peers read it
    (or into an ordinary tensor when `private`)."""
    B, ll, ml, kin = t2.shape
    nq, npp = wx.shape[1], wx.shape[2]
    nout = npp if transpose_w else nq
    if private:
        slot, t3, lstride = None, torch.empty(B, ml, ll, nout, dtype=t2.dtype, device=t2.device), ll
    else:
        slot, t3, lstride = t3_buffer(plan, B, nout, t2.dtype, t2.device)
    gemm(ml, nout, kin,
         Operand(t2, ld=kin, zs_hi=ml * kin, zs_lo=ll * ml * kin),
         Operand(wx, ld=npp, mn_major=transpose_w, zs_hi=nq * npp),
         Output(t3, rs_lo=lstride * nout, d_zhi=nout, d_zlo=ml * lstride * nout),
         zhi_n=ll, zlo_n=B, tri=Tri(rmax_a=1, rmax_b=1 + plan.l0 - plan.m0), sync=peer.sync_descriptor(produce=slot),
         dests=_dests(slot))
    return slot, t3, lstride


def stage_lm_to_slot(t2: torch.Tensor, plan: DistSHTPlan):
    """Makes a [B, l_loc, m_loc, n] coefficient block readable by the latitude peers (regridded-residual path)."""
    B, ll, ml, n2 = t2.shape
    slot = _slot("t2s", "h", B * plan.llmax * plan.mlmax * n2 * _esz(t2.dtype), t2.device, plan.ph)
    if slot is None:
        return None, t2, ll
    view = slot.tensor(t2.dtype, (B, plan.llmax, ml, n2))
    slot.publish(t2, B, ll * ml * n2, ll * ml * n2, plan.llmax * ml * n2)
    return slot, view, plan.llmax


def stage_legendre_synthesis(tslot, t, lstride, lm_order, table, plan: DistSHTPlan, B, C):
    """S4 (or the adjoint of S2 with `table = pw_syn`): T4[b, k_loc, (m_loc, ri), c] from coefficients given as
    [b, m, l, n] (`lm_order` False) or [b, l, m, n] (True)."""
    ml, hl = plan.ml, plan.hl
    n2 = 2 * C
    dev, dt = t.device, t.dtype
    if lm_order:
        bop = Operand(t, ld=ml * n2, mn_major=True, zs_hi=n2, zs_lo=lstride * ml * n2)
    else:
        bop = Operand(t, ld=n2, mn_major=True, zs_hi=lstride * n2, zs_lo=ml * lstride * n2)
    t4slot = _slot("t4", "w", B * plan.hmax * 2 * plan.mlmax * C * _esz(dt), dev, plan.pw)
    if t4slot is None:
        t4 = torch.empty(B, hl, 2 * ml, C, dtype=dt, device=dev)
        jstride = 2 * ml
    else:
        t4 = t4slot.tensor(dt, (B, hl, 2 * plan.mlmax, C))
        jstride = 2 * plan.mlmax
    out = Output(t4, rs_lo=jstride * C, d_zhi=n2, d_zlo=hl * jstride * C)
    aop = Operand(table, ld=plan.hlp, mn_major=True, zs_hi=plan.kl * plan.hlp)
    tri = Tri(kmin_a=1, kmin_b=plan.m0)
    sync = peer.sync_descriptor(consume=tslot, produce=t4slot)
    if tslot is None:
        gemm(hl, n2, plan.lmax, aop, bop, out, zhi_n=ml, zlo_n=B, tri=tri, sync=sync, dests=_dests(t4slot))
    else:
        segs = _segments(tslot, plan.l_shapes, plan.l_pos, _starts(plan.l_shapes))
        gemm(hl, n2, plan.kl, aop, bop, out, zhi_n=ml, zlo_n=B, tri=tri, segments=segs, sync=sync, dests=_dests(t4slot))
    return t4slot, t4, jstride


def stage_dft_synthesis(t4slot, t4, jstride, table, plan: DistSHTPlan, B, C):
    """S5 (or the adjoint of S1 with `table = ft_syn`): y[b, c, k_loc, i_loc] (channels-last)."""
    hl, wl = plan.hl, plan.wl
    y = torch.empty(B, C, hl, wl, dtype=t4.dtype, device=t4.device, memory_format=torch.channels_last)
    out = Output(y, rs_lo=C, d_zlo=wl * C, d_zhi=hl * wl * C)
    bop = Operand(t4, ld=C, mn_major=True, zs_lo=jstride * C, zs_hi=hl * jstride * C)
    aop = Operand(table, ld=plan.kj)
    sync = peer.sync_descriptor(consume=t4slot)
    if t4slot is None:
        gemm(wl, C, 2 * plan.mmax, aop, bop, out, zlo_n=hl, zhi_n=B, bn=_bn(C))
    else:
        segs = _segments(t4slot, plan.j_shapes, plan.j_pos, _starts(plan.j_shapes))
        gemm(wl, C, plan.kj, aop, bop, out, zlo_n=hl, zhi_n=B, bn=_bn(C), segments=segs, sync=sync)
    return y


def dist_sht_analysis(x, plan: DistSHTPlan, table_f=None, table_p=None):
    """[B, C, h_loc, w_loc] grid block -> T2 [B, l_loc, m_loc, (ri, C)]."""
    B, C = x.shape[0], x.shape[1]
    xslot, xv = stage_grid_to_slot(x, plan)
    t1slot, t1, hs = stage_dft_analysis(xslot, xv, plan.f_an if table_f is None else table_f, plan, B, C)
    return stage_legendre_analysis(t1slot, t1, hs, plan.pw_an if table_p is None else table_p, plan, B, C)


def dist_sht_synthesis(tslot, t, lstride, lm_order, plan: DistSHTPlan, B, C, table_p=None, table_g=None):
    t4slot, t4, js = stage_legendre_synthesis(tslot, t, lstride, lm_order, plan.p_syn if table_p is None else table_p, plan, B, C)
    return stage_dft_synthesis(t4slot, t4, js, plan.g_syn if table_g is None else table_g, plan, B, C)


# ------------------------------------------------------------------------------------------------ autograd


class _DistSpectralConv(torch.autograd.Function):
    """y = iSHT_out(W . SHT_in(x)) on sharded grids, and the regridded residual when asked for."""

    @staticmethod
    def forward(ctx, x, w, plan_in: DistSHTPlan, plan_out: DistSHTPlan, want_resid: bool):
        x = _to_cl(x)
        B, C = x.shape[0], x.shape[1]
        wx = expand_weight(w, x.dtype)
        Co = wx.shape[1] // 2
        t2 = dist_sht_analysis(x, plan_in)
        s3, t3, ls = stage_contract(t2, wx, False, plan_in)
        y = dist_sht_synthesis(s3, t3, ls, False, plan_out, B, Co)
        r = None
        if want_resid:
            s2, t2v, ls2 = stage_lm_to_slot(t2, plan_in)
            r = dist_sht_synthesis(s2, t2v, ls2, True, plan_out, B, C)
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
        B, Co = dy.shape[0], dy.shape[1]
        C = t2.shape[3] // 2
        dt3 = dist_sht_analysis(dy, plan_out, plan_out.gt_an, plan_out.p_an)        # [B, l, m, (ri, o)]
        dw = None
        if ctx.needs_input_grad[1]:
            dw = fold_weight_grad2(contract_wgrad2(dt3, t2, plan_in.l0, plan_in.m0)).reshape(ctx.wshape)
        dx = None
        if ctx.needs_input_grad[0]:
            if ctx.want_resid and dr is not None:
                dr2 = dist_sht_analysis(_to_cl(dr), plan_out, plan_out.gt_an, plan_out.p_an)   # [B, l, m, (ri, c)]
                # contraction into a private buffer, then the sum goes where the latitude peers read it
                _, priv, _ = stage_contract(dt3, wx, True, plan_in, private=True)
                nout = wx.shape[2]
                slot, t3v, ls = t3_buffer(plan_in, B, nout, dt3.dtype, dt3.device)
                if slot is None:
                    torch.add(priv, dr2.transpose(1, 2), out=t3v)
                else:
                    total = priv + dr2.transpose(1, 2)
                    slot.publish(total, B * plan_in.ml, plan_in.ll * nout, plan_in.ll * nout, ls * nout)
            else:
                slot, t3v, ls = stage_contract(dt3, wx, True, plan_in)
            dx = dist_sht_synthesis(slot, t3v, ls, False, plan_in, B, C, plan_in.pw_syn, plan_in.ft_syn)
        return dx, dw, None, None, None


def dist_spectral_conv_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return _ext.native() and x.dim() == 4 and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.dim() == 3 and w.shape[1] % 8 == 0


def dist_spectral_conv_dhconv(x, w, plan_in: DistSHTPlan, plan_out: DistSHTPlan, want_resid: bool):
    return _DistSpectralConv.apply(x, w, plan_in, plan_out, want_resid)
