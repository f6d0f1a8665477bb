"""CPU checks of the op layer: the GEMM addressing emulation that stands in for the tcgen05 kernel, the layout logic
of the pointwise convolutions (NCHW / channels-last in every combination), fused AdamW reference path, losses."""

import math

import numpy as np
import pytest
import torch

from makani_b200.ops import conv as C
from makani_b200.ops.gemm import ACT_DGELU, ACT_GELU, ACT_MULAUX, ACT_NONE, BIAS_ROW, Operand, Output, Tri, gemm
from makani_b200.ops.optim import FusedAdamW
from makani_b200.ops.spectral import expand_weight, fold_weight_grad


def test_emulated_gemm_majors_batches_and_scatter():
    torch.manual_seed(0)
    M, N, K, Z = 5, 7, 6, 3
    a = torch.randn(Z, K, M)          # MN-major A
    b = torch.randn(Z, N, K)          # K-major B
    d = torch.zeros(Z, M, N)
    gemm(M, N, K, Operand(a, ld=M, mn_major=True, zs_lo=K * M), Operand(b, ld=K, zs_lo=N * K), Output(d, rs_lo=N, d_zlo=M * N), zlo_n=Z)
    assert torch.allclose(d, torch.einsum("zkm,znk->zmn", a, b), atol=1e-5)
    # split row / column addressing and accumulate
    d2 = torch.zeros(2, M, 4, N // 1)
    a2 = torch.randn(M * 2, K)
    b2 = torch.randn(N, K)
    out = torch.zeros(M, 2, N)
    gemm(2 * M, N, K, Operand(a2, ld=K), Operand(b2, ld=K), Output(out, rdiv=2, rs_hi=2 * N, rs_lo=N), alpha=2.0)
    assert torch.allclose(out.reshape(2 * M, N), 2.0 * a2 @ b2.t(), atol=1e-5)
    acc = torch.ones(2 * M, N)
    gemm(2 * M, N, K, Operand(a2, ld=K), Operand(b2, ld=K), Output(acc, rs_lo=N), accumulate=True)
    assert torch.allclose(acc, 1.0 + a2 @ b2.t(), atol=1e-5)


def test_emulated_gemm_saved_gelu_derivative_matches_autograd():
    """`preact_deriv` stores d gelu / d pre in the second output; multiplying an upstream gradient by it (ACT_MULAUX)
    gives what autograd gives through gelu, and what ACT_DGELU gives from a saved pre-activation."""
    torch.manual_seed(3)
    M, N, K = 6, 9, 5
    a, b, bias = torch.randn(M, K), torch.randn(N, K), torch.randn(M)
    y, dact, pre = torch.zeros(M, N), torch.zeros(M, N), torch.zeros(M, N)
    gemm(M, N, K, Operand(a, ld=K), Operand(b, ld=K), Output(y, rs_lo=N), bias=bias, bias_mode=BIAS_ROW, act=ACT_GELU,
         preact=dact, preact_deriv=True)
    gemm(M, N, K, Operand(a, ld=K), Operand(b, ld=K), Output(torch.zeros(M, N), rs_lo=N), bias=bias, bias_mode=BIAS_ROW,
         act=ACT_GELU, preact=pre)
    z = (a @ b.t() + bias[:, None]).requires_grad_()
    yr = torch.nn.functional.gelu(z)
    assert torch.allclose(y, yr.detach(), atol=1e-5) and torch.allclose(pre, z.detach(), atol=1e-5)
    # upstream gradient g = u v^T through both backward flavours
    u, v = torch.randn(M, 1), torch.randn(N, 1)
    g = u @ v.t()
    (dz,) = torch.autograd.grad(yr, z, g)
    out1, out2 = torch.zeros(M, N), torch.zeros(M, N)
    gemm(M, N, 1, Operand(u, ld=1), Operand(v, ld=1), Output(out1, rs_lo=N), act=ACT_MULAUX, resid=dact)
    gemm(M, N, 1, Operand(u, ld=1), Operand(v, ld=1), Output(out2, rs_lo=N), act=ACT_DGELU, resid=pre)
    assert torch.allclose(out1, dz, atol=1e-5) and torch.allclose(out2, dz, atol=1e-5)


@pytest.mark.parametrize("x_cl", [False, True])
@pytest.mark.parametrize("out_layout", [C.NCHW, C.CL])
def test_conv_layout_combinations_match_torch(x_cl, out_layout):
    torch.manual_seed(1)
    B, Ci, Co, H, W = 2, 8, 16, 4, 8
    x = torch.randn(B, Ci, H, W)
    if x_cl:
        x = x.contiguous(memory_format=torch.channels_last)
    w = torch.randn(Co, Ci)
    bias = torch.randn(Co)
    res = torch.randn(B, Co, H, W)
    if out_layout == C.CL:
        res = res.contiguous(memory_format=torch.channels_last)
    wq = C.prep_weight(w, torch.float32)
    y, pre = C._conv_fwd(x, wq, Ci, bias, ACT_GELU, res, True, out_layout)
    ref_pre = torch.nn.functional.conv2d(x, w.view(Co, Ci, 1, 1), bias)
    assert C.layout_of(y) == out_layout
    assert torch.allclose(pre, ref_pre, atol=1e-5)
    assert torch.allclose(y, torch.nn.functional.gelu(ref_pre) + res, atol=1e-5)
    # data gradient (with GELU') and weight gradient
    dy = torch.randn(B, Co, H, W)
    if out_layout == C.CL:
        dy = dy.contiguous(memory_format=torch.channels_last)
    aux = torch.randn(B, Ci, H, W)
    if x_cl:
        aux = aux.contiguous(memory_format=torch.channels_last)
    dx = C._conv_dgrad(dy, wq, Ci, act=ACT_DGELU, aux=aux, x_layout=C.layout_of(x))
    xa = aux.clone().requires_grad_()
    torch.nn.functional.gelu(xa).backward(torch.einsum("bohw,oi->bihw", dy, w))
    assert torch.allclose(dx, xa.grad, atol=1e-4)
    dw = C._conv_wgrad(dy, x, splits=3)
    assert torch.allclose(dw, torch.einsum("bohw,bihw->oi", dy, x), atol=1e-4)


def test_spectral_weight_expand_and_fold_are_adjoint():
    torch.manual_seed(2)
    w = torch.randn(3, 5, 4, dtype=torch.complex64)
    wx = expand_weight(w, torch.float32)
    x = torch.randn(6, dtype=torch.complex64)
    l = 2
    xr = torch.cat([x[:3].real, x[:3].imag])
    out = wx[l] @ xr
    ref = torch.einsum("i,io->o", x[:3], w[:, :, l])
    assert torch.allclose(out[:5], ref.real, atol=1e-5) and torch.allclose(out[5:], ref.imag, atol=1e-5)
    g = torch.randn(4, 10, 6)
    dw = fold_weight_grad(g)
    # <expand(w), g> == Re<w, fold(g)> summed over real and imaginary parts
    lhs = (wx * g).sum()
    rhs = (w.real * dw.real + w.imag * dw.imag).sum()
    assert abs(lhs.item() - rhs.item()) < 1e-3


@pytest.mark.parametrize("adamw", [True, False])
def test_fused_adamw_cpu_path_matches_torch(adamw):
    torch.manual_seed(3)
    p1, p2 = torch.randn(7, 3, requires_grad=True), torch.randn(5, requires_grad=True)
    r1, r2 = p1.detach().clone().requires_grad_(), p2.detach().clone().requires_grad_()
    opt = FusedAdamW([p1, p2], lr=1e-2, weight_decay=0.1, adamw=adamw)
    ref = (torch.optim.AdamW if adamw else torch.optim.Adam)([r1, r2], lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        for p, r in ((p1, r1), (p2, r2)):
            g = torch.randn_like(p)
            p.grad, r.grad = g.clone(), g.clone()
        opt.step(); ref.step()
    assert torch.allclose(p1, r1, atol=1e-6) and torch.allclose(p2, r2, atol=1e-6)


def test_complex_modulus_second_moment():
    torch.manual_seed(4)
    p = torch.randn(4, dtype=torch.complex64, requires_grad=True)
    opt = FusedAdamW([p], lr=1e-2, weight_decay=0.0, complex_mode="modulus")
    p.grad = torch.randn(4, dtype=torch.complex64)
    g = p.grad.clone()
    p0 = p.detach().clone()
    opt.step()
    # first step of Adam: update = lr * g / (|g| + eps)
    expect = p0 - 1e-2 * g / (g.abs() + 1e-8)
    assert torch.allclose(p.detach(), expect, atol=1e-5)


def test_lamb_matches_a_direct_restatement():
    import math
    from makani_b200.ops.optim import LAMB
    torch.manual_seed(0)
    ps = [torch.randn(5, 3, requires_grad=True), torch.randn(4, dtype=torch.complex64, requires_grad=True), torch.zeros(3, requires_grad=True)]
    ref = [p.detach().clone() for p in ps]
    opt = LAMB(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.1, max_grad_norm=0.5)
    m = [torch.zeros_like(torch.view_as_real(r) if r.is_complex() else r) for r in ref]
    v = [torch.zeros_like(x) for x in m]
    for step in range(1, 4):
        gs = [torch.randn_like(p) for p in ps]
        for p, g in zip(ps, gs):
            p.grad = g.clone()
        opt.step()
        gr = [torch.view_as_real(g) if g.is_complex() else g for g in gs]
        gnorm = math.sqrt(sum(float(g.square().sum()) for g in gr))
        clip = max(1.0, gnorm / 0.5)
        for i, r in enumerate(ref):
            rr = torch.view_as_real(r) if r.is_complex() else r
            g = gr[i] / clip
            m[i] = 0.9 * m[i] + 0.1 * g
            v[i] = 0.95 * v[i] + 0.05 * g * g
            u = (m[i] / (1 - 0.9 ** step)) / ((v[i] / (1 - 0.95 ** step)).sqrt() + 1e-6) + 0.1 * rr
            pn, un = float(rr.norm()), float(u.norm())
            ratio = pn / un if pn > 0 and un > 0 else 1.0
            rr.sub_(1e-2 * ratio * u)
        for p, r in zip(ps, ref):
            a = torch.view_as_real(p.detach()) if p.is_complex() else p.detach()
            b = torch.view_as_real(r) if r.is_complex() else r
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
