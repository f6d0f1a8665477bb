"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op (run with -m gpu)."""

import math

import pytest
import torch

from makani_b200.ops import _ext
from makani_b200.ops.gemm import (ACT_DGELU, ACT_GELU, ACT_MULAUX, ACT_NONE, BIAS_COL, BIAS_ROW, Operand, Output, Tri, _emulate,
                                  gemm)

pytestmark = pytest.mark.gpu


def _dev():
    assert torch.cuda.is_available(), "GPU tests need CUDA"
    _ext.require()
    return torch.device("cuda", 0)


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def _run_both(M, N, K, A, B, D, **kw):
    """Run the kernel on CUDA copies and the emulation on fp32 CPU copies of the same storages; return both D."""
    dev = _dev()
    cpu_kw = dict(kw)
    for name in ("bias", "resid", "preact"):
        if kw.get(name) is not None:
            cpu_kw[name] = kw[name].detach().cpu().float().clone()
    A_c = Operand(A.tensor.cpu().float().clone(), A.ld, A.mn_major, A.offset, A.zs_lo, A.zs_hi)
    B_c = Operand(B.tensor.cpu().float().clone(), B.ld, B.mn_major, B.offset, B.zs_lo, B.zs_hi)
    D_c = Output(D.tensor.cpu().float().clone(), D.rs_lo, D.offset, D.rdiv, D.rs_hi, D.ndiv, D.ns_hi, D.d_zlo, D.d_zhi)
    gemm(M, N, K, A_c, B_c, D_c, **{k: v for k, v in cpu_kw.items() if k not in ("splits", "bn")})
    gemm(M, N, K, A, B, D, **kw)
    torch.cuda.synchronize()
    _ext.check_device_errors(dev)
    outs = [(D.tensor, D_c.tensor)]
    if kw.get("preact") is not None:
        outs.append((kw["preact"], cpu_kw["preact"]))
    return outs


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 300, 136), (384, 1000, 384), (77, 72, 1000)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_majors_bf16(a_mn, b_mn, shape, bn):
    dev = _dev()
    M, N, K = shape
    torch.manual_seed(M + N + K)
    pad = lambda n: (n + 7) // 8 * 8
    a = torch.randn(pad(K), pad(M), device=dev).to(torch.bfloat16) if a_mn else torch.randn(pad(M), pad(K), device=dev).to(torch.bfloat16)
    b = torch.randn(pad(K), pad(N), device=dev).to(torch.bfloat16) if b_mn else torch.randn(pad(N), pad(K), device=dev).to(torch.bfloat16)
    d = torch.zeros(M, pad(N), device=dev, dtype=torch.bfloat16)
    outs = _run_both(M, N, K, Operand(a, ld=a.shape[1], mn_major=a_mn), Operand(b, ld=b.shape[1], mn_major=b_mn),
                     Output(d, rs_lo=pad(N)), bn=bn)
    for got, ref in outs:
        assert _rel(got, ref) < 1e-2


def test_gemm_rejects_addressing_outside_the_storage():
    """The host checks the corner elements of A, B and the output before anything is launched."""
    from makani_b200.ops.gemm import gemm
    dev = _dev()
    M, N, K = 256, 128, 64
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    small = torch.zeros(M - 1, N, device=dev, dtype=torch.bfloat16)      # one output row short
    with pytest.raises(RuntimeError, match="leaves the tensor's storage"):
        gemm(M, N, K, Operand(a, ld=K), Operand(b, ld=K), Output(small, rs_lo=N))
    with pytest.raises(RuntimeError, match="leaves the tensor's storage"):
        gemm(M, N, K, Operand(a, ld=K + 8), Operand(b, ld=K), Output(torch.zeros(M, N, device=dev, dtype=torch.bfloat16), rs_lo=N))
    _ext.check_device_errors(dev)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False)])
def test_gemm_tf32(a_mn, b_mn):
    dev = _dev()
    M, N, K = 150, 270, 200
    torch.manual_seed(0)
    a = torch.randn(K, 152, device=dev) if a_mn else torch.randn(152, K, device=dev)
    b = torch.randn(K, 272, device=dev) if b_mn else torch.randn(272, K, device=dev)
    d = torch.zeros(M, 272, device=dev)
    outs = _run_both(M, N, K, Operand(a, ld=a.shape[1], mn_major=a_mn), Operand(b, ld=b.shape[1], mn_major=b_mn),
                     Output(d, rs_lo=272))
    for got, ref in outs:
        assert _rel(got, ref) < 2e-3


def test_gemm_epilogue_bias_gelu_resid_preact():
    dev = _dev()
    M, N, K, Z = 96, 520, 80, 3
    torch.manual_seed(1)
    w = torch.randn(M, K, device=dev).to(torch.bfloat16)
    x = torch.randn(Z, K, N, device=dev).to(torch.bfloat16)
    bias = torch.randn(M, device=dev)
    res = torch.randn(Z, M, N, device=dev).to(torch.bfloat16)
    for act, use_res in [(ACT_NONE, False), (ACT_GELU, True), (ACT_DGELU, True)]:
        d = torch.zeros(Z, M, N, device=dev, dtype=torch.bfloat16)
        pre = torch.zeros_like(d) if act == ACT_GELU else None
        outs = _run_both(M, N, K, Operand(w, ld=K), Operand(x, ld=N, mn_major=True, zs_lo=K * N),
                         Output(d, rs_lo=N, d_zlo=M * N), zlo_n=Z, bias=bias, bias_mode=BIAS_ROW, act=act,
                         resid=res if use_res else None, preact=pre)
        for got, ref in outs:
            assert _rel(got, ref) < 1e-2


def test_gemm_bias_col_f32_out():
    dev = _dev()
    M, N, K = 130, 100, 72
    torch.manual_seed(2)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    bias = torch.randn(N, device=dev)
    d = torch.zeros(M, N, device=dev)
    outs = _run_both(M, N, K, Operand(a, ld=K), Operand(b, ld=K), Output(d, rs_lo=N), bias=bias, bias_mode=BIAS_COL, alpha=0.5)
    assert _rel(*outs[0]) < 5e-3


def test_gemm_splitk_accumulate_and_batch_reduce():
    dev = _dev()
    M, N, K, Z = 200, 74, 5000, 2
    torch.manual_seed(3)
    a = torch.randn(Z, M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(Z, N, K, device=dev).to(torch.bfloat16)
    d = torch.zeros(M, N, device=dev)
    outs = _run_both(M, N, K, Operand(a, ld=K, zs_lo=M * K), Operand(b, ld=K, zs_lo=N * K), Output(d, rs_lo=N),
                     zlo_n=Z, accumulate=True, splits=7)
    assert _rel(*outs[0]) < 5e-3


def test_gemm_scatter_and_triangular():
    dev = _dev()
    # batched over z_hi with rows below z_hi known zero, split row/column scatter into a padded buffer
    Zh, Zl, M, N, K = 5, 2, 140, 48, 100
    torch.manual_seed(4)
    a = torch.randn(Zh, M, 104, device=dev)
    r = torch.arange(M, device=dev).view(1, -1, 1)
    z = torch.arange(Zh, device=dev).view(-1, 1, 1) * 30
    a = (a * (r >= z)).to(torch.bfloat16)
    b = torch.randn(Zl, Zh, N, 104, device=dev).to(torch.bfloat16)
    # D[zl][r//2][zh][n//8][r%2][n%8]
    d = torch.full((Zl, M // 2, Zh, N // 8, 2, 8), 7.0, device=dev, dtype=torch.bfloat16)
    s = d.stride()
    outs = _run_both(M, N, K, Operand(a, ld=104, zs_hi=M * 104), Operand(b, ld=104, zs_lo=Zh * N * 104, zs_hi=N * 104),
                     Output(d, rdiv=2, rs_hi=s[1], rs_lo=s[4], ndiv=8, ns_hi=s[3], d_zlo=s[0], d_zhi=s[2]),
                     zlo_n=Zl, zhi_n=Zh, tri=Tri(rmin_a=30))
    assert _rel(*outs[0]) < 1e-2
    # k-range restriction: contributions only from k >= 16*z_hi
    a2 = torch.randn(Zh, M, 104, device=dev).to(torch.bfloat16)
    k = torch.arange(104, device=dev).view(1, 1, -1)
    b2 = (torch.randn(Zh, N, 104, device=dev) * (k >= torch.arange(Zh, device=dev).view(-1, 1, 1) * 16)).to(torch.bfloat16)
    d2 = torch.zeros(Zh, M, N, device=dev, dtype=torch.bfloat16)
    outs = _run_both(M, N, K, Operand(a2, ld=104, zs_hi=M * 104), Operand(b2, ld=104, zs_hi=N * 104),
                     Output(d2, rs_lo=N, d_zhi=M * N), zhi_n=Zh, tri=Tri(kmin_a=16, kmax_a=0, kmax_b=90))
    # the emulation masks k >= 90 exactly; the kernel may include the rest of the last 64-wide slab, so compare on a
    # version of the inputs that is zero beyond 90
    assert _rel(outs[0][0][:, :, :], outs[0][1]) < 0.5  # loose: structure only
    a3 = a2.clone(); a3[..., 90:] = 0
    d3 = torch.zeros_like(d2)
    outs = _run_both(M, N, K, Operand(a3, ld=104, zs_hi=M * 104), Operand(b2, ld=104, zs_hi=N * 104),
                     Output(d3, rs_lo=N, d_zhi=M * N), zhi_n=Zh, tri=Tri(kmin_a=16, kmax_a=0, kmax_b=90))
    assert _rel(*outs[0]) < 1e-2


def test_gemm_many_tiles_persistent():
    """More tiles than SMs and a long k loop: exercises stage/accumulator phase tracking."""
    dev = _dev()
    M, N, K = 128 * 9, 256 * 40, 64 * 23
    torch.manual_seed(5)
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    d = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    gemm(M, N, K, Operand(a, ld=K), Operand(b, ld=K), Output(d, rs_lo=N))
    ref = a.float() @ b.float().t()
    torch.cuda.synchronize()
    _ext.check_device_errors(dev)
    assert _rel(d, ref) < 1e-2


def test_gemm_cta_pairs_epilogues_ragged():
    """Token-major shapes that run on CTA pairs (256-row tiles, M > 128): ragged M and N, both tile widths, every
    TMA-store epilogue (plain, bias+GELU+saved pre-activation, +residual, *GELU'), batch of two, MN-major weight."""
    dev = _dev()
    torch.manual_seed(21)
    Z, M, K = 2, 1000, 520       # K >= 512: the launcher's default puts these shapes on CTA pairs
    for N in (384, 200):
        x = torch.randn(Z, M, K, device=dev).to(torch.bfloat16)
        w = torch.randn(N, K, device=dev).to(torch.bfloat16)
        wt = w.t().contiguous()                                   # [K, N]: the same weight read row-contiguous
        bias = torch.randn(N, device=dev)
        res = torch.randn(Z, M, N, device=dev).to(torch.bfloat16)
        for bn in (128, 256):
            for act, use_res, use_pre, wmn in [(ACT_NONE, False, False, False), (ACT_GELU, False, True, False),
                                               (ACT_NONE, True, False, True), (ACT_DGELU, True, False, True)]:
                d = torch.zeros(Z, M, N, device=dev, dtype=torch.bfloat16)
                pre = torch.zeros_like(d) if use_pre else None
                B = Operand(wt, ld=N, mn_major=True) if wmn else Operand(w, ld=K)
                outs = _run_both(M, N, K, Operand(x, ld=K, zs_lo=M * K), B, Output(d, rs_lo=N, d_zlo=M * N), zlo_n=Z,
                                 bias=bias if act != ACT_DGELU else None, bias_mode=BIAS_COL, act=act,
                                 resid=res if use_res else None, preact=pre, bn=bn)
                for got, ref in outs:
                    assert _rel(got, ref) < 1e-2, (N, bn, act, use_res)


def test_gemm_saved_gelu_derivative_and_multiply():
    """The forward epilogue that saves GELU'(pre-activation) in its second output, and the backward epilogue that only
    multiplies by it: token-major shapes (TMA-store epilogues, single CTAs and pairs, ragged edges) and a strided
    channel-major layout (generic epilogue), each against the fp32 emulation."""
    dev = _dev()
    torch.manual_seed(23)
    Z, M = 2, 1000
    for K, N in ((384, 200), (520, 384)):
        x = torch.randn(Z, M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        bias = torch.randn(N, device=dev)
        d = torch.zeros(Z, M, N, device=dev, dtype=torch.bfloat16)
        sec = torch.zeros_like(d)
        outs = _run_both(M, N, K, Operand(x, ld=K, zs_lo=M * K), Operand(w, ld=K), Output(d, rs_lo=N, d_zlo=M * N), zlo_n=Z,
                         bias=bias, bias_mode=BIAS_COL, act=ACT_GELU, preact=sec, preact_deriv=True)
        for got, ref in outs:
            assert _rel(got, ref) < 1e-2, (K, N)
        # backward flavour: (dy W) * saved derivative
        dy = torch.randn(Z, M, K, device=dev).to(torch.bfloat16)
        dd = torch.zeros(Z, M, N, device=dev, dtype=torch.bfloat16)
        outs = _run_both(M, N, K, Operand(dy, ld=K, zs_lo=M * K), Operand(w, ld=K), Output(dd, rs_lo=N, d_zlo=M * N), zlo_n=Z,
                         act=ACT_MULAUX, resid=sec)
        for got, ref in outs:
            assert _rel(got, ref) < 1e-2, (K, N)
    # channel-major output with a row bias: the generic epilogue
    Mc, Nc, Kc = 96, 520, 80
    wc = torch.randn(Mc, Kc, device=dev).to(torch.bfloat16)
    xc = torch.randn(Z, Kc, Nc, device=dev).to(torch.bfloat16)
    bc = torch.randn(Mc, device=dev)
    dc = torch.zeros(Z, Mc, Nc, device=dev, dtype=torch.bfloat16)
    sc = torch.zeros_like(dc)
    outs = _run_both(Mc, Nc, Kc, Operand(wc, ld=Kc), Operand(xc, ld=Nc, mn_major=True, zs_lo=Kc * Nc),
                     Output(dc, rs_lo=Nc, d_zlo=Mc * Nc), zlo_n=Z, bias=bc, bias_mode=BIAS_ROW, act=ACT_GELU, preact=sc,
                     preact_deriv=True)
    for got, ref in outs:
        assert _rel(got, ref) < 1e-2
    _ext.check_device_errors(dev)


def test_gemm_headline_token_count():
    """One 1x1-convolution GEMM at the flagship resolution (M = 721 * 1440 tokens, 384 -> 384 channels) against
    torch.matmul on a sample of row blocks, first, middle and last rows included."""
    dev = _dev()
    torch.manual_seed(22)
    M, N, K = 721 * 1440, 384, 768     # the block MLP's second layer: runs on CTA pairs
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) / math.sqrt(K)).to(torch.bfloat16)
    d = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    gemm(M, N, K, Operand(x, ld=K), Operand(w, ld=K), Output(d, rs_lo=N))
    torch.cuda.synchronize()
    _ext.check_device_errors(dev)
    for r0 in (0, 127, 128 * 4055, 256 * 2027 + 3, M - 300):
        ref = x[r0: r0 + 300].float() @ w.float().t()
        assert _rel(d[r0: r0 + 300], ref) < 1e-2, r0


def test_conv1x1_and_mlp2_fwd_bwd():
    from makani_b200.ops.conv import conv1x1, mlp2
    dev = _dev()
    torch.manual_seed(6)
    B, Ci, Ch, Co, H, W = 2, 20, 48, 12, 24, 40
    x = torch.randn(B, Ci, H, W, device=dev)
    w1 = (torch.randn(Ch, Ci, 1, 1, device=dev) * 0.3).requires_grad_()
    b1 = (torch.randn(Ch, device=dev) * 0.1).requires_grad_()
    w2 = (torch.randn(Co, Ch, 1, 1, device=dev) * 0.3).requires_grad_()
    b2 = (torch.randn(Co, device=dev) * 0.1).requires_grad_()
    res = torch.randn(B, Co, H, W, device=dev)
    gy = torch.randn(B, Co, H, W, device=dev)

    def ref():
        xr = x.clone().requires_grad_()
        rr = res.clone().requires_grad_()
        f = torch.nn.functional
        y = f.conv2d(f.gelu(f.conv2d(xr, w1, b1)), w2, b2) + rr
        g = torch.autograd.grad(y, [xr, w1, b1, w2, b2, rr], gy)
        return [y] + list(g)

    def fast():
        xr = x.to(torch.bfloat16).requires_grad_()
        rr = res.to(torch.bfloat16).requires_grad_()
        y = mlp2(xr, w1, b1, w2, b2, rr)
        g = torch.autograd.grad(y, [xr, w1, b1, w2, b2, rr], gy.to(torch.bfloat16))
        return [y] + list(g)

    for name, a, b in zip(["y", "dx", "dw1", "db1", "dw2", "db2", "dres"], fast(), ref()):
        assert _rel(a.float(), b) < 3e-2, name

    # single conv with GELU and residual
    xr = x.to(torch.bfloat16).requires_grad_()
    y = conv1x1(xr, w1, b1, act="gelu")
    g = torch.autograd.grad(y, [xr, w1, b1], torch.ones_like(y))
    xf = x.clone().requires_grad_()
    yr = torch.nn.functional.gelu(torch.nn.functional.conv2d(xf, w1, b1))
    gr = torch.autograd.grad(yr, [xf, w1, b1], torch.ones_like(yr))
    assert _rel(y.float(), yr) < 2e-2
    for a, b in zip(g, gr):
        assert _rel(a.float(), b) < 3e-2
    _ext.check_device_errors(dev)


def test_instance_norm_fwd_bwd():
    from makani_b200.ops.norm import instance_norm
    dev = _dev()
    torch.manual_seed(7)
    for (B, C, H, W) in [(2, 6, 24, 40), (1, 3, 9, 7)]:
        for act in ["none", "gelu"]:
            x = (torch.randn(B, C, H, W, device=dev) * 2 + 0.5)
            w = (torch.rand(C, device=dev) + 0.5).requires_grad_()
            b = (torch.randn(C, device=dev) * 0.2).requires_grad_()
            gy = torch.randn(B, C, H, W, device=dev)
            xb = x.to(torch.bfloat16).requires_grad_()
            y = instance_norm(xb, w, b, 1e-6, act)
            g = torch.autograd.grad(y, [xb, w, b], gy.to(torch.bfloat16))
            xf = x.to(torch.bfloat16).float().requires_grad_()
            yr = torch.nn.functional.instance_norm(xf, None, None, w, b, True, 0.0, 1e-6)
            if act == "gelu":
                yr = torch.nn.functional.gelu(yr)
            gr = torch.autograd.grad(yr, [xf, w, b], gy.to(torch.bfloat16).float())
            assert _rel(y.float(), yr) < 1e-2
            for a, r_ in zip(g, gr):
                assert _rel(a.float(), r_) < 2e-2


def test_instance_norm_large_mean_small_spread():
    """Channels-last instance norm of a field whose mean is 300 times its spread (one-pass variance must not cancel):
    a 361x720 grid, statistics against torch in fp64 on the same bf16 data."""
    from makani_b200.ops.norm import instance_norm
    dev = _dev()
    torch.manual_seed(31)
    B, C, H, W = 1, 64, 361, 720
    x = (300.0 + torch.randn(B, C, H, W, device=dev)).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = torch.rand(C, device=dev) + 0.5
    b = torch.randn(C, device=dev) * 0.1
    y = instance_norm(x, w, b, 1e-6, "none")
    xd = x.double()
    mean = xd.mean(dim=(2, 3), keepdim=True)
    var = xd.var(dim=(2, 3), unbiased=False, keepdim=True)
    ref = (xd - mean) / torch.sqrt(var + 1e-6) * w.double().view(1, -1, 1, 1) + b.double().view(1, -1, 1, 1)
    torch.cuda.synchronize()
    assert _rel(y.float(), ref) < 1e-2, _rel(y.float(), ref)


def test_instance_norm_channels_last_fwd_bwd():
    from makani_b200.ops.norm import instance_norm
    dev = _dev()
    torch.manual_seed(17)
    for (B, C, H, W) in [(2, 16, 24, 40), (1, 384, 33, 64), (3, 8, 9, 7)]:
        for act in ["none", "gelu"]:
            x = (torch.randn(B, C, H, W, device=dev) * 2 + 0.5)
            w = (torch.rand(C, device=dev) + 0.5).requires_grad_()
            b = (torch.randn(C, device=dev) * 0.2).requires_grad_()
            gy = torch.randn(B, C, H, W, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            xb = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last).requires_grad_()
            y = instance_norm(xb, w, b, 1e-6, act)
            assert y.is_contiguous(memory_format=torch.channels_last)
            g = torch.autograd.grad(y, [xb, w, b], gy)
            xf = x.to(torch.bfloat16).float().requires_grad_()
            yr = torch.nn.functional.instance_norm(xf, None, None, w, b, True, 0.0, 1e-6)
            if act == "gelu":
                yr = torch.nn.functional.gelu(yr)
            gr = torch.autograd.grad(yr, [xf, w, b], gy.float())
            assert _rel(y.float(), yr) < 1e-2
            for a, r_ in zip(g, gr):
                assert _rel(a.float(), r_) < 2e-2
    _ext.check_device_errors(dev)


def test_conv_channels_last_chain():
    """NCHW in -> channels-last hidden -> NCHW out, the layout path the SFNO encoder/decoder take."""
    from makani_b200.ops.conv import CL, NCHW, layout_of, mlp2
    dev = _dev()
    torch.manual_seed(16)
    B, Ci, Ch, Co, H, W = 2, 10, 64, 64, 24, 40
    x = torch.randn(B, Ci, H, W, device=dev)
    w1 = (torch.randn(Ch, Ci, 1, 1, device=dev) * 0.3).requires_grad_()
    b1 = (torch.randn(Ch, device=dev) * 0.1).requires_grad_()
    w2 = (torch.randn(Co, Ch, 1, 1, device=dev) * 0.2).requires_grad_()
    w3 = (torch.randn(7, Co, 1, 1, device=dev) * 0.2).requires_grad_()
    b3 = (torch.randn(Co, device=dev) * 0.1).requires_grad_()
    xb = x.to(torch.bfloat16).requires_grad_()
    h = mlp2(xb, w1, b1, w2, None)                      # NCHW -> CL
    assert layout_of(h) == CL
    y = mlp2(h, w2.detach().transpose(0, 1).contiguous().requires_grad_(), b3, w3, None)   # CL -> NCHW (7 channels)
    assert layout_of(y) == NCHW and y.shape == (B, 7, H, W)
    f = torch.nn.functional
    xf = x.to(torch.bfloat16).float().requires_grad_()
    hr = f.conv2d(f.gelu(f.conv2d(xf, w1, b1)), w2)
    assert _rel(h.float(), hr) < 2e-2
    gy = torch.randn_like(hr)
    g = torch.autograd.grad(h, [xb, w1, b1, w2], gy.to(torch.bfloat16).contiguous(memory_format=torch.channels_last))
    gr = torch.autograd.grad(hr, [xf, w1, b1, w2], gy)
    for a, r_ in zip(g, gr):
        assert _rel(a.float(), r_) < 3e-2
    _ext.check_device_errors(dev)


def test_lp_norms_fwd_bwd():
    from makani_b200.ops.loss import weighted_lp_norms
    dev = _dev()
    torch.manual_seed(8)
    # W = 64 takes the 16-byte loads, W = 50 the scalar path; 1100 x 64 spans two chunks of a plane
    for (B, C, H, W), dtype, p in [(s_, d_, p_) for s_ in [(2, 5, 33, 64), (2, 5, 33, 50), (1, 3, 1100, 64)]
                                   for d_ in [torch.float32, torch.bfloat16] for p_ in [1, 2]]:
        q = torch.rand(H, device=dev) / (H * W)
        if True:
            pr = torch.randn(B, C, H, W, device=dev).to(dtype).requires_grad_()
            tg = torch.randn(B, C, H, W, device=dev).to(dtype)
            out = weighted_lp_norms(pr, tg, q, p)
            coef = torch.rand(B, C, device=dev)
            (g,) = torch.autograd.grad((out[..., 0] * coef).sum(), pr)
            prf = pr.detach().float().requires_grad_()
            d = ((prf - tg.float()).abs() ** p * q.view(1, 1, -1, 1)).sum(dim=(-2, -1))
            t = (tg.float().abs() ** p * q.view(1, 1, -1, 1)).sum(dim=(-2, -1))
            (gr,) = torch.autograd.grad((d * coef).sum(), prf)
            assert _rel(out[..., 0], d) < 1e-4 and _rel(out[..., 1], t) < 1e-4
            assert _rel(g.float(), gr) < (1e-2 if dtype == torch.bfloat16 else 1e-5)
            # two calls in a row give the same answer (scratch counters are left at zero)
            out2 = weighted_lp_norms(pr, tg, q, p)
            assert torch.equal(out, out2)


def test_lp_norms_scratch_reuse_across_shapes():
    """The cached scratch buffer serves calls of different (planes, chunks): large, small, larger again, each checked."""
    from makani_b200.ops.loss import weighted_lp_norms
    dev = _dev()
    torch.manual_seed(18)
    for (B, C, H, W) in [(2, 6, 130, 1024), (1, 3, 33, 64), (3, 6, 130, 1024), (1, 7, 70, 1000), (2, 6, 130, 1024)]:
        q = torch.rand(H, device=dev) / (H * W)
        pr = (torch.randn(B, C, H, W, device=dev) + 3.0).to(torch.bfloat16)
        tg = torch.randn(B, C, H, W, device=dev).to(torch.bfloat16)
        out = weighted_lp_norms(pr, tg, q, 2)
        d = ((pr.float() - tg.float()) ** 2 * q.view(1, 1, -1, 1)).sum(dim=(-2, -1))
        t = (tg.float() ** 2 * q.view(1, 1, -1, 1)).sum(dim=(-2, -1))
        assert _rel(out[..., 0], d) < 1e-4 and _rel(out[..., 1], t) < 1e-4, (B, C, H, W)


def test_fused_adamw_matches_torch():
    from makani_b200.ops.optim import FusedAdamW
    dev = _dev()
    torch.manual_seed(9)
    shapes = [(37,), (64, 33), (5, 7, 3), (100000,)]
    ps = [torch.randn(s, device=dev).requires_grad_() for s in shapes]
    pc = torch.randn(11, 6, dtype=torch.complex64, device=dev).requires_grad_()
    ref = [p.detach().clone().requires_grad_() for p in ps]
    refc = torch.view_as_real(pc.detach().clone()).clone().requires_grad_()
    opt = FusedAdamW(ps + [pc], lr=1e-2, weight_decay=0.1, complex_mode="split")
    opt_ref = torch.optim.AdamW(ref + [refc], lr=1e-2, weight_decay=0.1)
    for it in range(3):
        for p, r in zip(ps, ref):
            g = torch.randn_like(p)
            p.grad = g.clone(); r.grad = g.clone()
        gc = torch.randn_like(pc)
        pc.grad = gc.clone(); refc.grad = torch.view_as_real(gc).clone()
        opt.step(); opt_ref.step()
    for p, r in zip(ps, ref):
        assert _rel(p, r) < 1e-5
    assert _rel(torch.view_as_real(pc), refc) < 1e-5


def test_spectral_expand_fold():
    from makani_b200.ops.spectral import expand_weight, fold_weight_grad
    dev = _dev()
    torch.manual_seed(10)
    w = torch.randn(12, 20, 37, dtype=torch.complex64, device=dev)
    wx = expand_weight(w)
    ref = expand_weight(w.cpu())
    assert _rel(wx.float(), ref.float()) < 1e-6
    dwx = torch.randn(37, 40, 24, device=dev)
    assert _rel(torch.view_as_real(fold_weight_grad(dwx)), torch.view_as_real(fold_weight_grad(dwx.cpu()))) < 1e-6


def test_spectral_conv_fwd_bwd():
    from makani_b200.ops.spectral import SHTPlan, spectral_conv_dhconv
    from makani_b200.sht import InverseRealSHT, RealSHT
    dev = _dev()
    torch.manual_seed(11)
    B, C, Co = 2, 8, 16
    nlat, nlon, L, M = 33, 64, 16, 17
    nlat2, nlon2 = 16, 32
    pin = SHTPlan.get(nlat, nlon, L, M, "equiangular", dev)
    pout = SHTPlan.get(nlat2, nlon2, L, M, "legendre-gauss", dev)
    sht = RealSHT(nlat, nlon, L, M, "equiangular").to(dev)
    isht = InverseRealSHT(nlat2, nlon2, L, M, "legendre-gauss").to(dev)
    x = torch.randn(B, C, nlat, nlon, device=dev)
    w = (torch.randn(C, Co, L, dtype=torch.complex64, device=dev) / math.sqrt(C)).requires_grad_()
    xb = x.to(torch.bfloat16).requires_grad_()
    y, r = spectral_conv_dhconv(xb, w, pin, pout, True)
    gy, gr = torch.randn_like(y), torch.randn_like(r)
    gx, gw = torch.autograd.grad([y, r], [xb, w], [gy, gr])
    xf = x.to(torch.bfloat16).float().requires_grad_()
    c = sht(xf)
    yr = isht(torch.einsum("bixy,iox->boxy", c, w))
    rr = isht(c)
    gxr, gwr = torch.autograd.grad([yr, rr], [xf, w], [gy.float(), gr.float()])
    assert _rel(y.float(), yr) < 3e-2
    assert _rel(r.float(), rr) < 3e-2
    assert _rel(gx.float(), gxr) < 3e-2
    assert _rel(torch.view_as_real(gw), torch.view_as_real(gwr)) < 3e-2
    _ext.check_device_errors(dev)


def test_spectral_conv_production_size():
    """The tensor-core SHT chain at the flagship resolution: 721 x 1440 equiangular -> (lmax 240, mmax 241) -> 240 x 480
    Gauss grid, 8 channels, bf16 tables and intermediates, against the exact transform evaluated in fp64."""
    from makani_b200.ops.spectral import SHTPlan, spectral_conv_dhconv
    from makani_b200.sht import InverseRealSHT, RealSHT
    dev = _dev()
    torch.manual_seed(13)
    B, C = 1, 8
    nlat, nlon, L, M = 721, 1440, 240, 241
    nlat2, nlon2 = 240, 480
    pin = SHTPlan.get(nlat, nlon, L, M, "equiangular", dev)
    pout = SHTPlan.get(nlat2, nlon2, L, M, "legendre-gauss", dev)
    sht = RealSHT(nlat, nlon, L, M, "equiangular").to(dev).double()
    isht = InverseRealSHT(nlat2, nlon2, L, M, "legendre-gauss").to(dev).double()
    x = torch.randn(B, C, nlat, nlon, device=dev)
    w = (torch.randn(C, C, L, dtype=torch.complex64, device=dev) / math.sqrt(C)).requires_grad_()
    xb = x.to(torch.bfloat16).requires_grad_()
    y, r = spectral_conv_dhconv(xb, w, pin, pout, True)
    gy, gr = torch.randn_like(y), torch.randn_like(r)
    gx, gw = torch.autograd.grad([y, r], [xb, w], [gy, gr])
    xf = x.to(torch.bfloat16).double().requires_grad_()
    wd = w.detach().to(torch.complex128).requires_grad_()
    c = sht(xf)
    yr = isht(torch.einsum("bixy,iox->boxy", c, wd))
    rr = isht(c)
    gxr, gwr = torch.autograd.grad([yr, rr], [xf, wd], [gy.double(), gr.double()])
    errs = dict(y=_rel(y, yr), r=_rel(r, rr), gx=_rel(gx, gxr), gw=_rel(torch.view_as_real(gw), torch.view_as_real(gwr)))
    print("spectral conv 721x1440 errors", {k: round(v, 4) for k, v in errs.items()})
    assert max(errs.values()) < 2e-2, errs
    _ext.check_device_errors(dev)


def test_sfno_bf16_vs_fp32_reference():
    from makani_b200.models.networks.sfnonet import SphericalFourierNeuralOperatorNet as SFNO
    dev = _dev()
    torch.manual_seed(12)
    m = SFNO(inp_shape=(33, 64), out_shape=(33, 64), scale_factor=2, inp_chans=8, out_chans=4, embed_dim=16, num_layers=3).to(dev)
    x = torch.randn(2, 8, 33, 64, device=dev)
    yr = m(x)
    yr.square().mean().backward()
    gref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    m.set_compute_dtype(torch.bfloat16)
    y = m(x)
    assert y.dtype == torch.bfloat16
    y.float().square().mean().backward()
    assert _rel(y.float(), yr) < 5e-2
    worst = 0.0
    for n, p in m.named_parameters():
        g, r = p.grad, gref[n]
        if g.is_complex():
            g, r = torch.view_as_real(g), torch.view_as_real(r)
        if r.norm().item() < 1e-5:      # e.g. a bias in front of an instance norm: its exact gradient is zero
            assert g.norm().item() < 1e-2, n
            continue
        worst = max(worst, _rel(g, r))
        assert _rel(g, r) < 0.05, n
    print("sfno bf16 vs fp32: output", round(_rel(y.float(), yr), 4), "worst parameter gradient", round(worst, 4))
    _ext.check_device_errors(dev)


def test_mode_wise_contractions():
    """Diagonal and separable complex contractions (streaming kernels) against torch.einsum: forward and both gradients."""
    from makani_b200.ops import spectral_modes as sm
    dev = _dev()
    torch.manual_seed(41)
    B, I, O, X, Y = 2, 12, 10, 37, 38
    a = torch.randn(B, I, X, Y, dtype=torch.complex64, device=dev)
    cases = [(sm.contract_diagonal, "bixy,ioxy->boxy", (I, O, X, Y)), (sm.contract_sep_diagonal, "bixy,ixy->bixy", (I, X, Y)),
             (sm.contract_sep_dhconv, "bixy,ix->bixy", (I, X))]
    for fn, eq, wshape in cases:
        w = torch.randn(*wshape, dtype=torch.complex64, device=dev)
        a1, w1 = a.clone().requires_grad_(), w.clone().requires_grad_()
        a2, w2 = a.clone().requires_grad_(), w.clone().requires_grad_()
        y1, y2 = fn(a1, w1), torch.einsum(eq, a2, w2)
        g = torch.randn_like(y2)
        y1.backward(g)
        y2.backward(g)
        for got, ref in ((y1, y2), (a1.grad, a2.grad), (w1.grad, w2.grad)):
            assert _rel(torch.view_as_real(got.detach()), torch.view_as_real(ref.detach())) < 1e-5, eq
    _ext.check_device_errors(dev)


def test_loss_curve_native_bf16_tracks_fp32_formulation():
    """Fifty optimisation steps of a small SFNO: the native bf16 kernels (fused AdamW included) against the plain torch
    fp32 formulation of the same model from the same initial weights and data; the two loss curves stay together."""
    from makani_b200.models.networks.sfnonet import SphericalFourierNeuralOperatorNet as SFNO
    from makani_b200.ops.optim import FusedAdamW
    dev = _dev()

    def run(native):
        torch.manual_seed(77)
        m = SFNO(inp_shape=(64, 128), out_shape=(64, 128), scale_factor=2, inp_chans=8, out_chans=8, embed_dim=32, num_layers=2).to(dev)
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        xs = [torch.randn(2, 8, 64, 128, device=dev, generator=g) for _ in range(4)]
        ts = [0.5 * x.roll(3, dims=-1) + 0.1 * x ** 2 for x in xs]      # a learnable map
        losses = []
        if native:
            m.set_compute_dtype(torch.bfloat16)
            opt = FusedAdamW(m.parameters(), lr=2e-3, weight_decay=0.0)
        else:
            opt = torch.optim.AdamW(m.parameters(), lr=2e-3, weight_decay=0.0)
        _ext.set_native(native)
        try:
            for it in range(50):
                opt.zero_grad()
                y = m(xs[it % 4])
                loss = (y.float() - ts[it % 4]).square().mean()
                loss.backward()
                opt.step()
                losses.append(float(loss))
        finally:
            _ext.set_native(True)
        return torch.tensor(losses)

    ref, nat = run(False), run(True)
    _ext.check_device_errors(dev)
    assert nat[-1] < 0.8 * nat[0], "the native run does not learn"
    rel = ((nat - ref).abs() / ref).max().item()
    print("loss curve: first", float(ref[0]), float(nat[0]), "last", float(ref[-1]), float(nat[-1]), "max rel diff", round(rel, 4))
    assert rel < 5e-2, rel


def test_swap_ri_and_two_block_weight_gradient():
    """(re, im) -> (im, -re) re-layout and the (dWr, dWi) GEMM pair against the complex einsum they implement."""
    from makani_b200.ops.spectral import contract_wgrad2, fold_weight_grad2
    dev = _dev()
    torch.manual_seed(21)
    B, L, M, Co, Ci = 2, 12, 12, 16, 24
    dt = torch.randn(B, L, M, 2 * Co, device=dev).to(torch.bfloat16)
    t2 = torch.randn(B, L, M, 2 * Ci, device=dev).to(torch.bfloat16)
    out = torch.empty_like(dt)
    _ext.require().swap_ri(dt, out, Co)
    d5 = dt.view(B, L, M, 2, Co)
    want = torch.cat([d5[..., 1:2, :], -d5[..., 0:1, :]], dim=-2).reshape(dt.shape)
    assert torch.equal(out, want)
    # zero the (l, m) pairs with m > l, as the Legendre stages do
    mask = (torch.arange(M, device=dev)[None, :] <= torch.arange(L, device=dev)[:, None]).view(1, L, M, 1)
    dtm, t2m = dt * mask, t2 * mask
    dw = fold_weight_grad2(contract_wgrad2(dtm.contiguous(), t2m.contiguous()))            # complex [Ci, Co, L]
    dtc = torch.complex(dtm[..., :Co].float(), dtm[..., Co:].float())                     # [B, L, M, Co]
    t2c = torch.complex(t2m[..., :Ci].float(), t2m[..., Ci:].float())
    # y = W x  =>  dL/dW = sum conj(x) dy in torch's convention for complex parameters
    ref = torch.einsum("blmo,blmc->col", dtc, t2c.conj())
    assert _rel(torch.view_as_real(dw), torch.view_as_real(ref)) < 2e-2
    _ext.check_device_errors(dev)


def test_graphed_train_step_matches_eager_steps():
    """Forward + backward + fused AdamW replayed from one CUDA graph follow the same trajectory as eager launches
    (changing learning rate included: hyper-parameters are uploaded outside the graph)."""
    from makani_b200.models.networks.sfnonet import SphericalFourierNeuralOperatorNet as SFNO
    from makani_b200.ops.optim import FusedAdamW
    from makani_b200.parallel.grad_reduce import GradReducer
    from makani_b200.utils.train_step import GraphedTrainStep, TrainStep
    dev = _dev()

    def run(cls):
        torch.manual_seed(5)
        m = SFNO(inp_shape=(33, 64), out_shape=(33, 64), scale_factor=2, inp_chans=8, out_chans=8, embed_dim=16, num_layers=2).to(dev)
        m.set_compute_dtype(torch.bfloat16)
        red = GradReducer(m)
        opt = FusedAdamW(m.parameters(), lr=1e-3)
        step = cls(m, lambda p, t, i: (p.float() - t.float()).square().mean(), opt, red)
        g = torch.Generator(device=dev).manual_seed(9)
        losses = []
        for it in range(7):
            x = torch.randn(2, 8, 33, 64, device=dev, generator=g).to(torch.bfloat16)
            t = torch.randn(2, 8, 33, 64, device=dev, generator=g).to(torch.bfloat16)
            for grp in opt.param_groups:
                grp["lr"] = 1e-3 * (0.5 if it >= 5 else 1.0)
            losses.append(float(step(x, t)))
        torch.cuda.synchronize()
        return losses, [p.detach().clone() for p in m.parameters()], step

    le, pe, _ = run(TrainStep)
    lg, pg, gs = run(GraphedTrainStep)
    assert gs.graph is not None, "the step was not captured"
    for a, b in zip(le, lg):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (le, lg)
    num = sum(float((torch.view_as_real(a) if a.is_complex() else a).sub(torch.view_as_real(b) if b.is_complex() else b).square().sum())
              for a, b in zip(pe, pg))
    den = sum(float((torch.view_as_real(a) if a.is_complex() else a).square().sum()) for a in pe)
    assert (num / den) ** 0.5 < 2e-2
    _ext.check_device_errors(dev)


def test_bounded_wait_reports_instead_of_hanging():
    """A consumer whose peer never signals gives up after its 2 s limit, sets the device error word and returns; the
    host sees the code and the context stays usable.  (The "peer" is a flag in local memory that nothing sets.)"""
    import time
    dev = _dev()
    ext = _ext.require()
    _ext.check_device_errors(dev)
    ctrl = torch.zeros(64, dtype=torch.int32, device=dev)            # ready[8] | free[8] | n_prod, n_read, done
    base = ctrl.data_ptr()
    ready, free_, n_read, done = base, base + 32, base + 68, base + 72
    # [nwait, nsig, done_ctr, {wait, expected, offset, bump, peers} x 2, {peers, signal[8]} x 2]
    sync = [1, 1, done, ready, n_read, 1, n_read, 1, 0, 0, 0, 0, 0, 1, free_] + [0] * 7 + [0] * 9
    assert len(sync) == 31
    src = torch.ones(4096, dtype=torch.bfloat16, device=dev)
    out = torch.zeros_like(src)
    t0 = time.time()
    ext.peer_sum(out, [src.data_ptr()], None, 0, sync)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.5 < waited < 10.0, waited
    with pytest.raises(RuntimeError, match="code 44"):
        _ext.check_device_errors(dev)
    assert float(out.float().abs().sum()) == 0.0                     # nothing was consumed
    _ext.check_device_errors(dev)                                    # the error word is cleared by the report
    # the same kernel proceeds as soon as the flag is there, and ordinary work still runs
    ctrl[0] = 1
    ext.peer_sum(out, [src.data_ptr()], None, 0, sync)
    torch.cuda.synchronize()
    _ext.check_device_errors(dev)
    assert torch.equal(out, src)
    assert int(ctrl[17]) == 1 and int(ctrl[8]) == 1                  # n_read bumped, "free" signalled
