"""MetricsHandler: rollout curves, validation loss / L1 and ACC area under the curve against direct restatements."""

import numpy as np
import torch

from makani_b200.utils.grids import GridQuadrature
from makani_b200.utils.metric import MetricsHandler
from testutils import get_default_parameters

H, W, C, B, STEPS = 13, 24, 4, 3, 2


def test_curves_losses_and_auc():
    p = get_default_parameters(img_shape_x=H, img_shape_y=W, img_crop_shape_x=H, img_crop_shape_y=W, img_crop_offset_x=0,
                               img_crop_offset_y=0, N_out_channels=C, valid_autoreg_steps=STEPS, dt=1, dhours=6)
    torch.manual_seed(4)
    mult = torch.tensor([1.0, 2.0, 3.0, 4.0])
    clim = torch.randn(C, H, W) * 0.1
    mh = MetricsHandler(p, mult, clim, torch.device("cpu"))
    mh.initialize_buffers()
    mh.zero_buffers()
    q = GridQuadrature("naive", (H, W), normalize=True).quad_weight.reshape(H, W).double().numpy()
    nbatches = 2
    acc_ref = np.zeros((C, STEPS + 1))
    rmse_ref = np.zeros((C, STEPS + 1))
    loss_ref, l1_ref = 0.0, 0.0
    for b in range(nbatches):
        for idt in range(STEPS + 1):
            prd, tar = torch.randn(B, C, H, W), torch.randn(B, C, H, W)
            loss = torch.tensor(0.5 + b + idt)
            mh.update(prd, tar, loss, idt)
            pa, ta = (prd - clim).double().numpy(), (tar - clim).double().numpy()
            acc = (pa * ta * q).sum(axis=(-2, -1)) / (np.sqrt((pa ** 2 * q).sum(axis=(-2, -1)) * (ta ** 2 * q).sum(axis=(-2, -1))) + 1e-8)
            acc_ref[:, idt] += acc.sum(axis=0)
            rmse = np.sqrt((((prd - tar).double().numpy()) ** 2 * q).sum(axis=(-2, -1)))
            rmse_ref[:, idt] += mult.numpy() * rmse.sum(axis=0)
            if idt == 0:
                loss_ref += float(loss)
                l1_ref += (np.abs((prd - tar).double().numpy()) * q).sum(axis=(-2, -1)).mean(axis=1).sum()
    logs = mh.finalize()
    assert logs["base"]["validation steps"] == nbatches
    assert abs(logs["base"]["validation loss"] - loss_ref / nbatches) < 1e-5
    assert abs(logs["base"]["validation L1"] - l1_ref / nbatches) < 1e-4
    np.testing.assert_allclose(mh.acc_curve_cpu.numpy(), acc_ref / nbatches, rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(mh.rmse_curve_cpu.numpy(), rmse_ref / nbatches, rtol=1e-4)
    assert abs(logs["metrics"]["validation t2m"] - rmse_ref[1, 0] / nbatches) < 1e-3
    # Simpson's rule over the rollout steps (two intervals of width 1/3)
    a = acc_ref / nbatches
    auc = (a[:, 0] + 4 * a[:, 1] + a[:, 2]) * (1.0 / 3.0) / 3.0
    np.testing.assert_allclose(mh.acc_auc_cpu.numpy(), auc, rtol=1e-3, atol=1e-5)
    assert abs(logs["metrics"]["ACC AUC z500"] - auc[3]) < 1e-4
    # a second epoch starts from zeroed buffers
    mh.zero_buffers()
    assert float(mh.acc_curve.abs().sum()) == 0.0 and float(mh.valid_buffer.abs().sum()) == 0.0
