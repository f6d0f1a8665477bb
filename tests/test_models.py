"""Every registered network builds on a 32x64 grid, maps [4,4,32,64] -> [4,2,32,64] and back-propagates to its input
(same checks as the reference's tests/test_models.py:24-69)."""

import pytest
import torch

from makani_b200.models import model_registry
from testutils import get_default_parameters


@pytest.mark.parametrize("nettype", [n for n in model_registry.list_models() if n != "DebugNet"])
def test_model_forward_backward(nettype):
    p = get_default_parameters(nettype=nettype, img_crop_shape_x=32, img_crop_shape_y=64, img_shape_x=32, img_shape_y=64,
                               N_in_channels=4, N_out_channels=2, depth=2, num_heads=4, patch_size=(4, 4), num_blocks=4)
    torch.manual_seed(0)
    model = model_registry.get_model(p)
    x = torch.randn(4, 4, 32, 64, requires_grad=True)
    y = model(x)
    assert y.shape == (4, 2, 32, 64)
    y.sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape
    assert torch.isfinite(x.grad).all()


@pytest.mark.parametrize("kw", [dict(filter_type="non-linear", operator_type="diagonal", spectral_layers=2),
                                dict(operator_type="diagonal"), dict(factorization="cp", rank=0.5),
                                dict(factorization="tucker", rank=0.5), dict(factorization="tt", rank=0.5),
                                dict(pos_embed="frequency"), dict(pos_embed="direct"), dict(normalization_layer="layer_norm"),
                                dict(checkpointing=3), dict(separable=True), dict(nettype="FNO", operator_type="diagonal")])
def test_sfno_variants(kw):
    kw = dict(kw)
    p = get_default_parameters(img_crop_shape_x=32, img_crop_shape_y=64, img_shape_x=32, img_shape_y=64,
                               N_in_channels=3, N_out_channels=3, **kw)
    model = model_registry.get_model(p)
    model.train()
    y = model(torch.randn(2, 3, 32, 64))
    assert y.shape == (2, 3, 32, 64)
    y.square().mean().backward()


def test_registry_register_and_errors():
    class Net(torch.nn.Module):
        def __init__(self, **kw):
            super().__init__()

        def forward(self, x):
            return x

    model_registry.register_model(Net, "MyNetForTest")
    assert "MyNetForTest" in model_registry.list_models()
    with pytest.raises(ValueError):
        model_registry.register_model(Net, "MyNetForTest")
    with pytest.raises(KeyError):
        model_registry.get_model_class("does-not-exist")


def test_state_dict_names_follow_the_checkpoint_contract():
    p = get_default_parameters(img_crop_shape_x=32, img_crop_shape_y=64, img_shape_x=32, img_shape_y=64, N_in_channels=4, N_out_channels=4)
    names = set(model_registry.get_model(p).state_dict().keys())
    for k in ["model.encoder.fwd.0.weight", "model.encoder.fwd.0.bias", "model.encoder.fwd.2.weight",
              "model.blocks.0.filter.filter.weight", "model.blocks.0.norm0.weight", "model.blocks.0.mlp.fwd.0.weight",
              "model.blocks.0.mlp.fwd.3.bias", "model.blocks.1.outer_skip.weight", "model.decoder.fwd.2.weight",
              "model.residual_transform.weight"]:
        assert k in names, k
    assert not any("sht" in k or "weights" == k.split(".")[-1] and "trans" in k for k in names)


def test_contraction_handle_and_parameter_report(capsys):
    """`factorizations.get_contract_fun` (dense tensor, real-view tensor and factorised weight give the same product as
    the dense contraction) and `helpers.check_parameters`."""
    import torch

    from makani_b200.models.common.contractions import get_contract_fun as dense_fun
    from makani_b200.models.common.factorizations import FactorizedWeight, get_contract_fun
    from makani_b200.models.helpers import check_parameters

    torch.manual_seed(0)
    x = torch.randn(2, 3, 5, 6, dtype=torch.complex64)
    for op, shape in (("dhconv", [3, 4, 5]), ("diagonal", [3, 4, 5, 6])):
        w = FactorizedWeight(shape, rank=0.5, factorization="cp")
        want = dense_fun(op, False)(x, w.to_tensor())
        for impl in ("reconstructed", "factorized"):
            assert torch.allclose(get_contract_fun(w, impl, False, op)(x, w), want, atol=1e-6)
        dense = w.to_tensor().detach()
        assert torch.allclose(get_contract_fun(dense, "factorized", False, op)(x, dense), want, atol=1e-6)
        assert torch.allclose(get_contract_fun(dense, "reconstructed", False, op)(torch.view_as_real(x), torch.view_as_real(dense)), want, atol=1e-6)
    check_parameters(torch.nn.Linear(3, 2))
    out = capsys.readouterr().out
    assert "weight (2, 3)" in out and "bias (2,)" in out
