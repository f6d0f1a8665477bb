"""Visualisation without a plotting stack: colour ramps, Mollweide resampling, comparison frames, curve plots, GIFs."""

import os

import numpy as np
import pytest

from makani_b200.utils import visualize as viz
from testutils import get_default_parameters

PIL = pytest.importorskip("PIL")


def test_colorize_endpoints_and_nan():
    f = np.array([[0.0, 0.5, 1.0, np.nan]])
    rgb = viz.colorize(f, 0.0, 1.0, diverging=True)
    assert rgb.shape == (1, 4, 3) and rgb.dtype == np.uint8
    assert tuple(rgb[0, 0]) == (5, 48, 97) and tuple(rgb[0, 1]) == (247, 247, 247) and tuple(rgb[0, 2]) == (103, 0, 31)
    assert tuple(rgb[0, 3]) == (255, 255, 255)


def test_mollweide_resampling_geometry():
    H, W = 91, 180
    lat = np.linspace(90, -90, H)[:, None] * np.ones((1, W))
    m = viz.mollweide_resample(lat, width=200)
    assert m.shape == (100, 200)
    assert np.isnan(m[0, 0]) and np.isnan(m[-1, -1])                  # corners are outside the ellipse
    mid = m[:, 100]
    assert np.all(np.isfinite(mid)) and mid[0] > 80 and mid[-1] < -80 and abs(mid[50]) < 3     # pole to pole on the meridian
    assert np.nanmax(np.abs(m[50])) < 3                               # the equator is the horizontal axis
    # area fraction of the ellipse inside its bounding box is pi / 4
    assert abs(np.isfinite(m).mean() - np.pi / 4) < 0.02
    lon = np.ones((H, 1)) * np.linspace(-180, 180, W, endpoint=False)[None, :]
    ml = viz.mollweide_resample(lon, width=200)
    assert ml[50, 10] < -150 and ml[50, 190] > 150                    # west on the left, east on the right


def test_comparison_frame_curves_and_gif(tmp_path):
    rng = np.random.default_rng(0)
    pred, truth = rng.standard_normal((33, 64)), rng.standard_normal((33, 64))
    img = viz.plot_comparison(pred, truth, diverging=True)
    assert img.size[0] > 100 and img.size[1] > 100
    p = get_default_parameters(experiment_dir=str(tmp_path), dt=1, dhours=6)
    acc = np.linspace(1.0, 0.2, 5)[None, :].repeat(4, 0)
    viz.plot_rollout_metrics(acc, 1 - acc, p, epoch=0, model_name="tiny")
    assert os.path.isfile(tmp_path / "acc_t2m.png") and os.path.isfile(tmp_path / "rmse_z500.png")
    w = viz.VisualizationWrapper(False, str(tmp_path), "viz", [{"name": "ch0", "functor": "lambda x: x[0]", "diverging": True}])
    for step in range(3):
        w.add(f"step{step}", rng.standard_normal((2, 17, 32)), rng.standard_normal((2, 17, 32)))
    out = w.finalize()
    assert os.path.isfile(out["ch0"])


def test_visualize_field_applies_the_functor_to_unscaled_fields():
    import numpy as np

    from makani_b200.utils.visualize import visualize_field

    rng = np.random.default_rng(0)
    pred, targ = rng.normal(size=(2, 16, 32)), rng.normal(size=(2, 16, 32))
    tag, image = visualize_field("wind", "lambda x: np.sqrt(np.square(x[0]) + np.square(x[1]))", pred, targ, None, None, 2.0, 1.0, False)
    assert tag == "wind" and image is not None and image.size[0] > 0 and image.size[1] > 0
