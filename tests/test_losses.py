"""Loss grammar against direct numpy restatements (quadrature-weighted Lp norms, channel weights, multistep weights,
temp-std re-weighting, spherical H1 norm from SHT coefficients)."""

import numpy as np
import pytest
import torch

from makani_b200.sht import RealSHT
from makani_b200.utils.grids import GridQuadrature
from makani_b200.utils.losses import LossHandler, _auto_channel_weights
from testutils import get_default_parameters

H, W, C, B = 19, 36, 4, 3


def _params(**over):
    p = get_default_parameters(img_shape_x=H, img_shape_y=W, img_crop_shape_x=H, img_crop_shape_y=W, img_crop_offset_x=0,
                               img_crop_offset_y=0, N_out_channels=C, n_future=0)
    p.update_params(over)
    return p


def _q():
    return GridQuadrature("naive", (H, W), normalize=True).quad_weight.reshape(H, W).double().numpy()


@pytest.fixture()
def fields():
    torch.manual_seed(2)
    return torch.randn(B, C, H, W), torch.randn(B, C, H, W)


@pytest.mark.parametrize("loss,p_,absolute,squared", [
    ("absolute squared geometric l2", 2, True, True), ("absolute geometric l2", 2, True, False),
    ("geometric l2", 2, False, False), ("squared geometric l2", 2, False, True),
    ("absolute geometric l1", 1, True, False), ("geometric l1", 1, False, False)])
def test_lp_variants(fields, loss, p_, absolute, squared):
    prd, tar = fields
    handler = LossHandler(_params(loss=loss)).eval()
    got = float(handler(prd, tar))
    q = _q()
    d = (np.abs((prd - tar).double().numpy()) ** p_ * q).sum(axis=(-2, -1))
    t = (np.abs(tar.double().numpy()) ** p_ * q).sum(axis=(-2, -1))
    v = d if absolute else d / t
    if not (squared and p_ == 2):
        v = v ** (1.0 / p_)
    want = (v / C).sum()                  # uniform channel weights normalised to one, summed over batch and channels
    assert abs(got - want) < 1e-4 * max(1.0, abs(want))


def test_auto_channel_weights_and_weighted_loss(fields):
    prd, tar = fields
    names = ["u10m", "t2m", "u500", "z500"]
    w = _auto_channel_weights(names).numpy()
    np.testing.assert_allclose(w, [0.1, 1.0, 0.5, 0.5], rtol=1e-6)
    handler = LossHandler(_params(loss="weighted absolute squared geometric l2", channel_names=names, channel_weights="auto")).eval()
    q = _q()
    d = (((prd - tar).double().numpy()) ** 2 * q).sum(axis=(-2, -1))
    want = (d * (w / w.sum())[None, :]).sum()
    assert abs(float(handler(prd, tar)) - want) < 1e-4 * abs(want)
    explicit = LossHandler(_params(loss="weighted absolute squared geometric l2", channel_weights=[1.0, 0.0, 0.0, 1.0])).eval()
    want2 = (d[:, [0, 3]] * 0.5).sum()
    assert abs(float(explicit(prd, tar)) - want2) < 1e-4 * abs(want2)


def test_multistep_weights_in_training_mode():
    torch.manual_seed(3)
    nf = 2
    prd, tar = torch.randn(B, C * (nf + 1), H, W), torch.randn(B, C * (nf + 1), H, W)
    handler = LossHandler(_params(loss="absolute squared geometric l2", n_future=nf)).train()
    q = _q()
    d = (((prd - tar).double().numpy()) ** 2 * q).sum(axis=(-2, -1))
    want = d.sum() / C / (nf + 1)
    assert abs(float(handler(prd, tar)) - want) < 1e-4 * abs(want)


def test_temp_std_reweighting(tmp_path, fields):
    prd, tar = fields
    gs, ts = np.array([1.0, 2.0, 3.0, 4.0], np.float32), np.array([0.5, 0.5, 1.0, 2.0], np.float32)
    np.save(tmp_path / "gs.npy", gs.reshape(1, C, 1, 1))
    np.save(tmp_path / "ts.npy", ts.reshape(1, C, 1, 1))
    p = _params(loss="absolute squared temp-std geometric l2", global_stds_path=str(tmp_path / "gs.npy"),
                time_diff_stds_path=str(tmp_path / "ts.npy"), dt=4, out_channels=[0, 1, 2, 3])
    handler = LossHandler(p).eval()
    q = _q()
    d = (((prd - tar).double().numpy()) ** 2 * q).sum(axis=(-2, -1))
    cw = (gs / (np.sqrt(4.0) * ts + 1e-6)) ** 2 / C
    want = (d * cw[None, :]).sum()
    assert abs(float(handler(prd, tar)) - want) < 1e-4 * abs(want)


def test_h1_loss_from_coefficients(fields):
    prd, tar = fields
    handler = LossHandler(_params(loss="absolute squared geometric h1")).eval()
    sht = RealSHT(H, W, grid="equiangular").float()
    c = sht((prd - tar).float())
    c2 = (c.real ** 2 + c.imag ** 2).double().numpy()
    n2 = c2[..., 0] + 2 * c2[..., 1:].sum(axis=-1)                     # [B, C, l]
    l = np.arange(n2.shape[-1])
    want = (0.5 * n2.reshape(B, -1).sum(axis=-1) + 0.5 * (n2 * l * (l + 1)).reshape(B, -1).sum(axis=-1)).sum()
    assert abs(float(handler(prd, tar)) - want) < 1e-3 * abs(want)


def test_loss_is_differentiable_and_zero_at_the_target(fields):
    _, tar = fields
    handler = LossHandler(_params(loss="geometric l1")).eval()
    assert float(handler(tar.clone(), tar)) == 0.0
    prd = (tar + 0.1 * torch.randn_like(tar)).requires_grad_()
    handler(prd, tar).backward()
    assert torch.isfinite(prd.grad).all() and prd.grad.abs().sum() > 0


def test_unknown_loss_is_rejected():
    with pytest.raises(ValueError):
        LossHandler(_params(loss="hinge"))


def test_h1_loss_abs_and_rel_methods():
    """`GeometricH1Loss.abs` / `.rel` (the two entry points of the reference's class) agree with `forward`."""
    import torch

    from makani_b200.utils.losses import GeometricH1Loss

    torch.manual_seed(0)
    prd, tar = torch.randn(2, 3, 16, 32), torch.randn(2, 3, 16, 32)
    for squared in (False, True):
        rel = GeometricH1Loss((16, 32), absolute=False, squared=squared)
        ab = GeometricH1Loss((16, 32), absolute=True, squared=squared)
        assert torch.allclose(rel.rel(prd, tar), rel(prd, tar))
        assert torch.allclose(ab.abs(prd, tar), ab(prd, tar))
        assert float(ab.abs(prd, prd)) == 0.0
