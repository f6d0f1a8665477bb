"""Preprocessor: history layout, rolling autoregressive window (with unpredicted zenith channels), residual targets,
static features restricted to the local window, per-sample history normalisation round trip."""

import numpy as np
import torch

from makani_b200.models.preprocessor import Preprocessor2D
from testutils import get_default_parameters

H, W, C = 12, 16, 3


def _pp(**over):
    p = get_default_parameters(img_shape_x=H, img_shape_y=W, N_in_channels=C, N_out_channels=C)
    p.update_params(over)
    return Preprocessor2D(p)


def test_flatten_and_expand_history_are_inverse():
    pp = _pp(n_history=2)
    x = torch.randn(2, 3, C, H, W)
    f = pp.flatten_history(x)
    assert f.shape == (2, 3 * C, H, W)
    assert torch.equal(pp.expand_history(f, 3), x)
    assert pp.flatten_history(f) is f


def test_append_history_rolls_the_window():
    pp = _pp(n_history=2)
    steps = [torch.full((1, C, H, W), float(i)) for i in range(4)]
    state = torch.cat(steps[:3], dim=1)                        # history t-2, t-1, t
    nxt = pp.append_history(state, steps[3], 0)
    want = torch.cat(steps[1:4], dim=1)
    assert torch.equal(nxt, want)
    assert torch.equal(_pp(n_history=0).append_history(steps[0], steps[1], 0), steps[1])


def test_unpredicted_channels_follow_the_rollout():
    pp = _pp(n_history=1, add_zenith=True)
    pp.eval()
    inp = torch.randn(2, 2, C, H, W)
    tar = torch.randn(2, 3, C, H, W)
    izen = torch.arange(2, dtype=torch.float32).view(1, 2, 1, 1, 1).expand(2, 2, 1, H, W).clone()
    tzen = (10 + torch.arange(3, dtype=torch.float32)).view(1, 3, 1, 1, 1).expand(2, 3, 1, H, W).clone()
    x, y = pp.cache_unpredicted_features(inp, tar, izen, tzen)
    xa = pp.append_unpredicted_features(pp.flatten_history(x))
    assert xa.shape == (2, 2 * (C + 1), H, W)
    xe = pp.expand_history(xa, 2)
    assert torch.equal(xe[:, :, C], izen[:, :, 0])             # zenith rides behind the prognostic channels of each step
    # after one autoregressive step the zenith history is (old step 1, target step 0)
    pp.append_history(pp.flatten_history(x), tar[:, 0], 0)
    xb = pp.expand_history(pp.append_unpredicted_features(pp.flatten_history(x)), 2)
    assert torch.all(xb[:, 0, C] == 1.0) and torch.all(xb[:, 1, C] == 10.0)
    assert torch.equal(pp.remove_unpredicted_features(xa), pp.flatten_history(x))


def test_residual_target(tmp_path):
    np.save(tmp_path / "tds.npy", np.full((1, C, 1, 1), 2.0, dtype=np.float32))
    pp = _pp(n_history=1, target="residual", normalize_residual=True, time_diff_stds_path=str(tmp_path / "tds.npy"))
    x = torch.randn(2, 2 * C, H, W)
    dx = torch.randn(2, C, H, W)
    out = pp.expand_history(pp.add_residual(x, dx), 2)
    xin = pp.expand_history(x, 2)
    assert torch.equal(out[:, 0], xin[:, 0])
    assert torch.allclose(out[:, 1], xin[:, 1] + 2.0 * dx)
    assert torch.equal(_pp().add_residual(x, dx), dx)          # default target: the model output is the state


def test_static_features_are_cut_to_the_local_window():
    full = _pp(add_grid=True, gridtype="linear")
    part = _pp(add_grid=True, gridtype="linear", img_local_offset_x=4, img_local_shape_x=5, img_local_offset_y=8, img_local_shape_y=8)
    assert full.static_features.shape == (1, 2, H, W) and part.static_features.shape == (1, 2, 5, 8)
    assert torch.equal(part.static_features, full.static_features[:, :, 4:9, 8:16])
    x = torch.randn(3, C, 5, 8)
    xs = part.add_static_features(x)
    assert xs.shape == (3, C + 2, 5, 8) and torch.equal(part.remove_static_features(xs), x)
    sin = _pp(add_grid=True, gridtype="sinusoidal", grid_num_frequencies=3)
    assert sin.static_features.shape == (1, 6, H, W)


def test_history_normalisation_round_trip():
    pp = _pp(n_history=2, history_normalization_mode="mean")
    x = torch.randn(2, 3 * C, H, W) * 3.0 + 1.5
    pp.history_compute_stats(x)
    xn = pp.history_normalize(x)
    assert xn.shape == x.shape
    assert torch.allclose(pp.history_denormalize(xn), x, atol=1e-4)
    y = torch.randn(2, C, H, W)
    assert torch.allclose(pp.history_denormalize(pp.history_normalize(y, target=True), target=True), y, atol=1e-4)
