"""AFNO spectral filter as a GEMM chain (`makani_b200/ops/afno.py`): the emulated chain (CPU) against the torch.fft
formulation, forward and every gradient; AFNO v2 network against the published op sequence written out directly."""

import pytest
import torch
import torch.nn.functional as F

from makani_b200.ops import afno


def _rel(a, b):
    return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()


def _params(nb, bs, hid, dt, dev="cpu"):
    ps = [0.3 * torch.randn(nb, bs, hid, dtype=dt, device=dev), 0.3 * torch.randn(nb, bs, hid, dtype=dt, device=dev),
          0.1 * torch.randn(nb, hid, dtype=dt, device=dev), 0.1 * torch.randn(nb, hid, dtype=dt, device=dev),
          0.3 * torch.randn(nb, hid, bs, dtype=dt, device=dev), 0.3 * torch.randn(nb, hid, bs, dtype=dt, device=dev),
          0.1 * torch.randn(nb, bs, dtype=dt, device=dev), 0.1 * torch.randn(nb, bs, dtype=dt, device=dev)]
    for p in ps:
        p.requires_grad_()
    return ps


@pytest.mark.parametrize("cfg", [(2, 12, 20, 32, 2, 1, 1.0, 1), (1, 10, 16, 48, 3, 2, 0.6, 2), (2, 9, 14, 16, 2, 1, 0.5, 1),
                                 (1, 8, 12, 16, 1, 1, 1.0, 2)])
def test_afno_chain_matches_fft_formulation(cfg):
    B, H, W, C, nb, f, frac, ver = cfg
    torch.manual_seed(0)
    dt = torch.float64
    bs, hid = C // nb, C // nb * f
    kx, ncols = (afno.mode_window_v1 if ver == 1 else afno.mode_window_v2)(H, W, frac)
    x = torch.randn(B, H, W, C, dtype=dt, requires_grad=True)
    ps = _params(nb, bs, hid, dt)
    assert afno.fast_path_ok(x, nb, hid)
    g = torch.randn(B, H, W, C, dtype=dt)
    res = []
    for fn in (afno.afno_filter, afno.afno_filter_reference):
        for t in [x] + ps:
            t.grad = None
        y = fn(x, *ps, kx, ncols, 0.05, skip=x)
        y.backward(g)
        res.append([y.detach()] + [t.grad.clone() for t in [x] + ps])
    for a, b in zip(*res):
        assert _rel(a, b) < 1e-5


def test_afno_windows():
    assert afno.mode_window_v1(90, 180, 1.0) == (tuple(range(90)), 46)
    rows, cols = afno.mode_window_v1(90, 180, 0.5)
    assert rows == tuple(range(23, 69)) and cols == 23
    assert afno.mode_window_v2(90, 180, 1.0) == (tuple(range(90)), 91)
    rows, cols = afno.mode_window_v2(90, 180, 0.5)
    assert rows == tuple(list(range(23)) + list(range(67, 90))) and cols == 45


@pytest.mark.parametrize("frac,norm,skip", [(1.0, "instance_norm", "linear"), (0.5, "layer_norm", "identity"), (0.7, "instance_norm", None)])
def test_afno_v2_network_matches_direct_formulation(frac, norm, skip):
    from makani_b200.models.networks.afnonet_v2 import AdaptiveFourierNeuralOperatorNet as Net
    torch.manual_seed(0)
    net = Net(inp_shape=(32, 48), patch_size=(4, 4), inp_chans=3, out_chans=2, embed_dim=32, num_layers=2, num_blocks=4,
              hard_thresholding_fraction=frac, normalization_layer=norm, skip_fno=skip, sparsity_threshold=0.01)
    for b in net.blocks:
        torch.nn.init.normal_(b.filter.w1, std=0.3)
        torch.nn.init.normal_(b.filter.w2, std=0.3)
        torch.nn.init.normal_(b.filter.b1, std=0.1)
    x = torch.randn(2, 3, 32, 48)
    y = net(x)

    def filt(f, t):
        B, C, H, W = t.shape
        th, tw = H // 2 + 1, W // 2 + 1
        kh, kw = int(th * frac), int(tw * frac)
        X = torch.fft.rfft2(t.float(), dim=(-2, -1), norm="ortho").view(B, f.num_blocks, f.block_size, H, tw)
        w1, w2 = torch.view_as_complex(f.w1.contiguous()), torch.view_as_complex(f.w2.contiguous())
        out = torch.zeros_like(X)

        def mlp(z):
            o = torch.einsum("bkixy,kio->bkoxy", z, w1)
            o = torch.complex(F.relu(o.real), F.relu(o.imag))
            return torch.einsum("bkixy,kio->bkoxy", o, w2)

        if kh == th:
            out[..., :kw] = mlp(X[..., :kw])
        else:
            out[:, :, :, :kh, :kw] = mlp(X[:, :, :, :kh, :kw])
            out[:, :, :, -kh:, :kw] = mlp(X[:, :, :, -kh:, :kw])
        out = torch.view_as_complex(F.softshrink(torch.view_as_real(out), f.sparsity_threshold)).reshape(B, C, H, tw)
        return torch.fft.irfft2(out, s=(H, W), dim=(-2, -1), norm="ortho") + f.b1 + t

    t = (net.patch_embed(x) + net.pos_embed).reshape(2, 32, net.h, net.w)
    for b in net.blocks:
        res = t
        u = filt(b.filter, b.norm1(t))
        if skip == "linear":
            u = u + b.skip_layer(res)
        elif skip == "identity":
            u = u + res
        t = b.mlp(b.norm2(u)) + res
    h = net.head(t)
    ref = h.view(2, 4, 4, -1, net.h, net.w).permute(0, 3, 4, 1, 5, 2).contiguous().view(2, -1, 32, 48)
    assert _rel(y, ref) < 1e-5
    y.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())
    sd = net.state_dict()
    for k in ("blocks.0.filter.w1", "blocks.0.filter.b1", "blocks.0.norm1.weight", "blocks.1.mlp.fwd.0.weight", "head.weight", "pos_embed"):
        assert k in sd or k.startswith("blocks.1.mlp"), k


def _gpu_case(ver, regime):
    from makani_b200.ops import _ext
    _ext.require()
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    B, H, W, C, nb = 1, 90, 180, 768, 8
    bs = hid = C // nb
    kx, ncols = (afno.mode_window_v1 if ver == 1 else afno.mode_window_v2)(H, W, 1.0)
    x32 = torch.randn(B, H, W, C, device=dev)
    ps32 = _params(nb, bs, hid, torch.float32, dev)
    lam = 0.01
    with torch.no_grad():
        for p in ps32:
            p.mul_(0.3)
        if regime == "linear":
            # every ReLU input far above zero and no shrinkage: the operator is affine, its gradient has no masks
            ps32[2].fill_(40.0)
            ps32[3].fill_(40.0)
            lam = 0.0
    g = torch.randn(B, H, W, C, device=dev)
    xb = x32.to(torch.bfloat16).requires_grad_()
    assert afno.fast_path_ok(xb, nb, hid)
    y = afno.afno_filter(xb, *ps32, kx, ncols, lam, skip=xb)
    y.backward(g.to(torch.bfloat16))
    got = [y.detach().float(), xb.grad.float()] + [p.grad.clone() for p in ps32]
    for p in ps32:
        p.grad = None
    xr = x32.to(torch.bfloat16).float().requires_grad_()
    yr = afno.afno_filter_reference(xr, *ps32, kx, ncols, lam, skip=xr)
    yr.backward(g.to(torch.bfloat16).float())
    ref = [yr.detach(), xr.grad] + [p.grad for p in ps32]
    torch.cuda.synchronize()
    _ext.check_device_errors(dev)
    names = ["y", "dx", "dw1r", "dw1i", "db1r", "db1i", "dw2r", "dw2i", "db2r", "db2i"]
    errs = {n: round(_rel(a, b), 4) for n, a, b in zip(names, got, ref)}
    print(f"afno chain bf16 errors ({regime}, window v{ver})", errs)
    return errs


@pytest.mark.gpu
@pytest.mark.parametrize("ver", [1, 2])
def test_afno_chain_gpu_bf16_affine_regime(ver):
    """The tensor-core chain at the FourCastNet token grid (90 x 180 tokens, 768 channels, 8 blocks) against the fp32
    torch.fft formulation, with biases that keep every ReLU open and no shrinkage: output and all gradients of the
    (then affine) operator agree to bf16 accuracy."""
    errs = _gpu_case(ver, "linear")
    assert max(errs.values()) < 2e-2, errs


@pytest.mark.gpu
@pytest.mark.parametrize("ver", [1, 2])
def test_afno_chain_gpu_bf16(ver):
    """Same, in the generic regime.  The output agrees to bf16 accuracy; the gradients are compared with a wider margin
    because they are discontinuous in the ReLU / shrinkage masks: a 0.3 % perturbation of the pre-activations (bf16
    DFT matrices and intermediates) flips about 0.25 % of the mask entries, and every flipped entry changes the
    gradient by its full size, i.e. by sqrt(0.0025) = 5 % in the L2 norm (the CPU emulation of the chain shows the
    same figure)."""
    errs = _gpu_case(ver, "generic")
    assert errs["y"] < 2e-2 and max(errs.values()) < 0.1, errs


def test_distributed_afno2d_v2_single_rank_matches_filter():
    """`DistributedAFNO2Dv2` on one rank (group size 1) is the plain filter on all blocks; gradients flow to every parameter."""
    from makani_b200.parallel.layers import DistributedAFNO2Dv2
    torch.manual_seed(0)
    m = DistributedAFNO2Dv2(32, num_blocks=4, hard_thresholding_fraction=0.6)
    x = torch.randn(2, 32, 10, 12, requires_grad=True)
    y = m(x)
    y.sum().backward()
    tok = x.detach().permute(0, 2, 3, 1).contiguous()
    kx, nc = afno.mode_window_v2(10, 12, 0.6)
    b1, b2 = m.b1[:, :, 0, 0], m.b2[:, :, 0, 0]
    ref = afno.afno_filter_reference(tok, m.w1[..., 0], m.w1[..., 1], b1[..., 0], b1[..., 1], m.w2[..., 0], m.w2[..., 1],
                                     b2[..., 0], b2[..., 1], kx, nc, 0.01, skip=tok).permute(0, 3, 1, 2)
    assert _rel(y, ref) < 1e-5
    assert all(p.grad is not None for p in m.parameters()) and x.grad is not None
