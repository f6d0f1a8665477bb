"""`MultifilesDataset` against direct reads of the files: shapes, sample counts, history / future windows, evaluation
roll-out targets, and spatial sharding emulated in one process through `io_grid` / `io_rank`
(test plan of the reference: tests/test_dataloader.py:83-261)."""

import os

import numpy as np
import pytest
import torch

from makani_b200.utils.dataloaders.data_loader_multifiles import MultifilesDataset
from testutils import get_default_parameters, init_dataset

NLAT, NLON, NCHAN, NDAYS = 33, 64, 4, 24


@pytest.fixture()
def data(tmp_path):
    paths = init_dataset(str(tmp_path), nlat=NLAT, nlon=NLON, nchan=NCHAN, ndays=NDAYS)
    return paths


def _params(paths, **over):
    p = get_default_parameters(**paths)
    p.update_params(over)
    return p


def _raw(paths, sub, year):
    return np.load(os.path.join(paths["train_data_path" if sub == "train" else "valid_data_path"], f"{year}.npy"))


def _norm(a, chans):
    return (a[:, chans] - 0.5) / 1.5


def _unpack(item):
    inp, tar = item[0], item[1]
    return np.asarray(inp), np.asarray(tar)


def test_shapes_counts_and_content(data):
    p = _params(data, n_history=0, n_future=0, dt=1)
    ds = MultifilesDataset(p, data["train_data_path"], train=True)
    assert len(ds) == 2 * NDAYS - p.dt * (p.n_history + p.n_future + 1)     # samples index one time axis across both years
    inp, tar = _unpack(ds[3])
    assert inp.shape == (1, NCHAN, NLAT, NLON) and tar.shape == (1, NCHAN, NLAT, NLON)
    raw = _raw(data, "train", 2016)
    np.testing.assert_allclose(inp[0], _norm(raw[3:4], p.in_channels)[0], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(tar[0], _norm(raw[4:5], p.out_channels)[0], rtol=1e-5, atol=1e-6)


def test_history_and_future_windows(data):
    p = _params(data, n_history=2, n_future=1, dt=2)
    ds = MultifilesDataset(p, data["train_data_path"], train=True)
    assert len(ds) == 2 * NDAYS - 2 * (2 + 1 + 1)
    inp, tar = _unpack(ds[0])
    assert inp.shape == (3, NCHAN, NLAT, NLON) and tar.shape == (2, NCHAN, NLAT, NLON)
    raw = _raw(data, "train", 2016)
    # first sample starts where a full history fits: input steps t-2dt, t-dt, t; targets t+dt, t+2dt
    t = 2 * 2
    want_in = _norm(raw[[t - 4, t - 2, t]], p.in_channels)
    want_tar = _norm(raw[[t + 2, t + 4]], p.out_channels)
    np.testing.assert_allclose(inp, want_in, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(tar, want_tar, rtol=1e-5, atol=1e-6)


def test_eval_targets_follow_valid_autoreg_steps(data):
    p = _params(data, n_history=0, n_future=0, valid_autoreg_steps=3, dt=1)
    ds = MultifilesDataset(p, data["valid_data_path"], train=False)
    inp, tar = _unpack(ds[5])
    assert tar.shape == (4, NCHAN, NLAT, NLON)
    raw = _raw(data, "test", 2019)
    np.testing.assert_allclose(tar, _norm(raw[6:10], p.out_channels), rtol=1e-5, atol=1e-6)


def test_channel_subsets(data):
    p = _params(data, in_channels=[0, 2], out_channels=[1, 3])
    ds = MultifilesDataset(p, data["train_data_path"], train=True)
    inp, tar = _unpack(ds[1])
    raw = _raw(data, "train", 2016)
    np.testing.assert_allclose(inp[0], _norm(raw[1:2], [0, 2])[0], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(tar[0], _norm(raw[2:3], [1, 3])[0], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("grid,rank", [([1, 2, 1], [0, 1, 0]), ([1, 1, 2], [0, 0, 1]), ([1, 2, 2], [0, 1, 0])])
def test_spatial_sharding_matches_slices_of_the_full_sample(data, grid, rank):
    from makani_b200.parallel.helpers import compute_split_shapes
    full = MultifilesDataset(_params(data), data["train_data_path"], train=True)
    part = MultifilesDataset(_params(data, io_grid=grid, io_rank=rank), data["train_data_path"], train=True)
    assert len(full) == len(part)
    fi, ft = _unpack(full[7])
    pi, pt = _unpack(part[7])
    hs, ws = compute_split_shapes(NLAT, grid[1]), compute_split_shapes(NLON, grid[2])
    h0, w0 = sum(hs[: rank[1]]), sum(ws[: rank[2]])
    sl = (Ellipsis, slice(h0, h0 + hs[rank[1]]), slice(w0, w0 + ws[rank[2]]))
    np.testing.assert_array_equal(pi, fi[sl])
    np.testing.assert_array_equal(pt, ft[sl])
    assert part.img_local_shape_x == hs[rank[1]] and part.img_local_shape_y == ws[rank[2]]
    assert part.img_local_offset_x == h0 and part.img_local_offset_y == w0


def test_minmax_normalisation(data):
    p = _params(data, normalization="minmax")
    ds = MultifilesDataset(p, data["train_data_path"], train=True)
    inp, _ = _unpack(ds[0])
    raw = _raw(data, "train", 2016)
    np.testing.assert_allclose(inp[0], (raw[0] + 5.0) / 10.0, rtol=1e-5, atol=1e-6)
    bias, scale = ds.get_input_normalization()
    assert bias.shape == (1, NCHAN, 1, 1) and scale.shape == (1, NCHAN, 1, 1)
