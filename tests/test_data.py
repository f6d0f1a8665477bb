"""Data path: loaders, metrics against direct numpy restatements, data tools (CPU)."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from makani_b200.utils.YParams import ParamsBase

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stats(tmp_path, C):
    np.save(tmp_path / "m.npy", np.arange(C, dtype=np.float32).reshape(1, C, 1, 1))
    np.save(tmp_path / "s.npy", (1.0 + np.arange(C, dtype=np.float32)).reshape(1, C, 1, 1))
    return str(tmp_path / "m.npy"), str(tmp_path / "s.npy")


def test_zarr_style_loader_pairs_and_normalisation(tmp_path):
    from makani_b200.utils.dataloaders.zarr_helper import get_data_loader
    C = 5
    m, s = _stats(tmp_path, C)
    p = ParamsBase()
    p.update_params(dict(global_means_path=m, global_stds_path=s, in_channels=[0, 1, 2], out_channels=[1, 2], dt=2, batch_size=2))
    f = np.random.RandomState(0).rand(9, C, 6, 8).astype(np.float32)
    loader, meta, sampler = get_data_loader(p, None, True, store=f)
    assert sampler is None and len(loader.dataset) == 7 and (meta.img_shape_x, meta.img_shape_y) == (6, 8)
    x, y = next(iter(loader))
    mean, std = np.load(m)[0], np.load(s)[0]
    np.testing.assert_allclose(x[1].numpy(), (f[1][[0, 1, 2]] - mean[[0, 1, 2]]) / std[[0, 1, 2]], rtol=1e-6)
    np.testing.assert_allclose(y[1].numpy(), (f[3][[1, 2]] - mean[[1, 2]]) / std[[1, 2]], rtol=1e-6)
    im, istd = loader.get_input_normalization()
    assert im.shape == (1, 3, 1, 1) and istd.shape == (1, 3, 1, 1)


def test_synthetic_loader_is_seeded_and_shaped():
    from makani_b200.utils.dataloader import get_dataloader
    p = ParamsBase()
    p.update_params(dict(enable_synthetic_data=True, batch_size=2, in_channels=[0, 1, 2], out_channels=[0, 1], n_history=0,
                         n_future=0, img_shape_x=16, img_shape_y=32, n_train_samples_per_epoch=6, dt=1, dhours=6,
                         data_num_shards=1, data_shard_id=0, seed=3))
    batches = []
    for _ in range(2):
        loader, dataset, _ = get_dataloader(p, None, torch.device("cpu"), train=True)
        batches.append([tuple(t.clone() for t in b) for b in loader])
    assert len(batches[0]) == 3
    for a, b in zip(*batches):
        assert a[0].shape[0] == 2 and a[0].shape[-2:] == (16, 32)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_weighted_metrics_match_numpy():
    from makani_b200.utils.grids import GridQuadrature
    from makani_b200.utils.metrics import functions as F
    torch.manual_seed(0)
    H, W = 19, 36
    quad = GridQuadrature("naive", (H, W), normalize=True)
    q = quad.quad_weight.reshape(H, W).double().numpy()
    assert abs(q.sum() - 1.0) < 1e-5
    x, y = torch.randn(3, 4, H, W), torch.randn(3, 4, H, W)
    rmse_ref = np.sqrt(((x - y).double().numpy() ** 2 * q).sum(axis=(-2, -1)))
    rmse = F.GeometricRMSE("naive", (H, W), normalize=True, channel_reduction="none", batch_reduction="none")(x, y)
    np.testing.assert_allclose(rmse.double().numpy(), rmse_ref, rtol=1e-4)
    l1_ref = (np.abs((x - y).double().numpy()) * q).sum(axis=(-2, -1))
    l1 = F.GeometricL1("naive", (H, W), normalize=True, channel_reduction="none", batch_reduction="none")(x, y)
    np.testing.assert_allclose(l1.double().numpy(), l1_ref, rtol=1e-4)
    # anomaly correlation of fields that are already anomalies: no re-centring (makani/utils/metrics/functions.py:87-92)
    xa, ya = x.double().numpy(), y.double().numpy()
    acc_ref = (xa * ya * q).sum(axis=(-2, -1)) / np.sqrt((xa ** 2 * q).sum(axis=(-2, -1)) * (ya ** 2 * q).sum(axis=(-2, -1)))
    acc = F.GeometricACC("naive", (H, W), normalize=True, channel_reduction="none", batch_reduction="none")(x, y)
    np.testing.assert_allclose(acc.double().numpy(), acc_ref, rtol=1e-4, atol=1e-6)


def test_parallel_copy_tool(tmp_path):
    src, dst = tmp_path / "in", tmp_path / "out"
    src.mkdir()
    for y in (2017, 2018, 2019):
        (src / f"{y}.h5").write_bytes(os.urandom(1000 + y))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "data_process", "parallel_copy.py"), "--input_dir", str(src),
                        "--output_dir", str(dst), "--workers", "2"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    for y in (2017, 2018, 2019):
        assert (dst / f"{y}.h5").read_bytes() == (src / f"{y}.h5").read_bytes()


def test_h5_convert_chunk_parser():
    sys.path.insert(0, os.path.join(ROOT, "data_process"))
    import h5_convert
    assert h5_convert.parse_chunks("auto", (10, 4, 8, 8), 4) is True
    assert h5_convert.parse_chunks("none", (10, 4, 8, 8), 4) is None
    assert h5_convert.parse_chunks("1MB", (2000, 4, 8, 8), 4) == (1024, 4, 8, 8)
    with pytest.raises(ValueError):
        h5_convert.parse_chunks("7", (1, 1, 1, 1), 4)


@pytest.mark.parametrize("shape", [(20, 101), (721, 1440)])
@pytest.mark.parametrize("rule", ["naive", "clenshaw-curtiss", "legendre-gauss"])
def test_quadrature_weights_integrate_to_one(rule, shape):
    from makani_b200.utils.grids import GridQuadrature
    quad = GridQuadrature(rule, shape, normalize=True)
    ones = torch.ones(1, 1, *shape)
    assert abs(float(quad(ones)) - 1.0) < 1e-5


def test_registry_lists_every_network_family_and_registers_custom_models():
    from makani_b200.models import model_registry as reg
    names = set(reg.list_models())
    assert {"AFNOv1", "AFNO", "FNO", "SFNO", "DebugNet", "ViT"} <= names

    class Tiny(torch.nn.Module):
        def __init__(self, inp_shape=(8, 16), inp_chans=2, out_chans=2, **kw):
            super().__init__()
            self.c = torch.nn.Conv2d(inp_chans, out_chans, 1)

        def forward(self, x):
            return self.c(x)

    reg.register_model(Tiny, "TinyTestNet")
    assert "TinyTestNet" in reg.list_models()
    with pytest.raises(Exception):
        reg.register_model(Tiny, "TinyTestNet")      # names are unique


def test_era5_time_axis_and_labelled_year(tmp_path):
    import datetime
    sys.path.insert(0, ROOT)
    from datasets.era5 import open_year, time as era5_time
    assert era5_time.filename_to_year("/data/out_of_sample/2018.h5") == 2018
    rng = era5_time.datetime_range(2018, datetime.timedelta(hours=6), 5)
    assert rng[0] == datetime.datetime(2018, 1, 1, tzinfo=datetime.timezone.utc) and (rng[4] - rng[0]).total_seconds() == 24 * 3600
    arr = np.random.rand(6, 3, 5, 8).astype(np.float32)
    np.save(tmp_path / "2017.npy", arr)
    meta = tmp_path / "data.json"
    meta.write_text('{"h5_path": "fields", "dhours": 6, "attrs": {"description": "t"}, "coords": {"grid_type": "equiangular", '
                    '"lat": [2, 1, 0, -1, -2], "lon": [0, 1, 2, 3, 4, 5, 6, 7], "channel": ["a", "b", "c"]}}')
    ya = open_year(str(tmp_path / "2017.npy"), metadata_path=str(meta))
    assert tuple(ya.shape) == arr.shape and tuple(ya.dims) == ("time", "channel", "lat", "lon")
    np.testing.assert_array_equal(np.asarray(ya[2]), arr[2])
    assert len(ya.coords["time"]) == 6 and list(ya.coords["channel"]) == ["a", "b", "c"]


def test_copernicus_request_plan():
    sys.path.insert(0, ROOT)
    from datasets.copernicus import get_data
    jobs = get_data.plan("/out", [2019], [500, 850], 0.25, 6)
    assert len(jobs) == 12 * 3
    fname, req = jobs[0]
    assert fname == "/out/raw/pl_500_2019-01.nc" and req["levtype"] == "pl" and req["levelist"] == "500"
    assert req["time"] == ["00:00", "06:00", "12:00", "18:00"] and req["date"] == "2019-01-01/to/2019-01-31"
    assert jobs[2][0] == "/out/raw/sfc_2019-01.nc" and jobs[2][1]["param"] == get_data.SFC_PARAMS
    feb = [r for f, r in jobs if f.endswith("sfc_2019-02.nc")][0]
    assert feb["date"].endswith("2019-02-28")


def _run_tool(name, *args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "data_process", name), *args], capture_output=True, text=True,
                       cwd=os.path.join(ROOT, "data_process"), env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_statistics_and_histogram_tools(tmp_path):
    rng = np.random.default_rng(3)
    src = tmp_path / "train"
    src.mkdir()
    years = {2016: rng.standard_normal((10, 3, 9, 16)) * np.array([1.0, 2.0, 0.5])[None, :, None, None] + np.array([0.0, 3.0, -1.0])[None, :, None, None],
             2017: rng.standard_normal((7, 3, 9, 16)) + 0.25}
    for y, a in years.items():
        np.save(src / f"{y}.npy", a.astype(np.float32))
    out = tmp_path / "stats"
    _run_tool("get_stats.py", "--input_path", str(src), "--output_path", str(out), "--batch", "4", "--dt", "2")
    full = np.concatenate([years[2016], years[2017]]).astype(np.float32).astype(np.float64)
    lat = np.linspace(0, np.pi, 9)
    q = np.clip(np.sin(lat), 0, None)[:, None] * np.ones((1, 16))
    q = q / q.sum()
    mean = (full * q).sum(axis=(2, 3)).mean(axis=0)
    std = np.sqrt((((full - mean[None, :, None, None]) ** 2) * q).sum(axis=(2, 3)).mean(axis=0))
    np.testing.assert_allclose(np.load(out / "global_means.npy").reshape(-1), mean, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(np.load(out / "global_stds.npy").reshape(-1), std, rtol=1e-4)
    np.testing.assert_allclose(np.load(out / "mins.npy").reshape(-1), full.min(axis=(0, 2, 3)), rtol=1e-6)
    np.testing.assert_allclose(np.load(out / "maxs.npy").reshape(-1), full.max(axis=(0, 2, 3)), rtol=1e-6)
    np.testing.assert_allclose(np.load(out / "time_means.npy")[0], full.mean(axis=0), rtol=1e-4, atol=1e-5)
    # differences x[t+dt] - x[t] never cross a file boundary
    diffs = np.concatenate([a[2:] - a[:-2] for a in (years[2016].astype(np.float32).astype(np.float64), years[2017].astype(np.float32).astype(np.float64))])
    dmean = (diffs * q).sum(axis=(2, 3)).mean(axis=0)
    dstd = np.sqrt((((diffs - dmean[None, :, None, None]) ** 2) * q).sum(axis=(2, 3)).mean(axis=0))
    np.testing.assert_allclose(np.load(out / "time_diff_means.npy").reshape(-1), dmean, rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(np.load(out / "time_diff_stds.npy").reshape(-1), dstd, rtol=1e-4)
    hist = tmp_path / "hist"
    _run_tool("get_histograms.py", "--input_path", str(src), "--output_path", str(hist), "--stats_path", str(out), "--nbins", "20")
    h = np.load(hist / "histograms.npz")
    assert h["counts"].shape == (3, 20) and h["edges"].shape == (3, 21)
    assert np.all(h["counts"].sum(axis=1) == 17 * 9 * 16)
