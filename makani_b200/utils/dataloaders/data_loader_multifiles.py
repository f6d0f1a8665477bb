"""Map-style dataset over yearly files holding `[time, channel, lat, lon]` arrays.

Behaviour contract: makani/utils/dataloaders/data_loader_multifiles.py:38-289 — samples index a global time
axis across years; each item returns `n_history+1` input steps and `n_future+1` (train) or
`valid_autoreg_steps+1` (eval) target steps spaced `dt` apart, restricted to this rank's lat/lon window
(`io_grid`, `io_rank`), normalised with z-score or min-max statistics, optionally with the cosine of the solar
zenith angle, and passed through the grid converter.

Files: `????.h5` (dataset `params.h5_path`, needs h5py) or `????.npy` (memory-mapped, no extra dependency).
Targets are read with `out_channels` (the reference reads them with `in_channels`, line 260).
"""

from __future__ import annotations

import datetime
import glob
import logging
import os
from bisect import bisect_right
from itertools import accumulate

import numpy as np
import torch
from torch.utils.data import Dataset

from ...parallel.helpers import compute_split_shapes
from ..grids import GridConverter


class MultifilesDataset(Dataset):
    def __init__(self, params, location, train, enable_logging=True):
        self.params, self.location, self.train = params, location, train
        g = params.get
        self.dt, self.dhours = params.dt, params.dhours
        self.n_history = g("n_history", 0)
        self.n_future = g("valid_autoreg_steps", 0) if not train else g("n_future", 0)
        self.in_channels = np.array(params.in_channels)
        self.out_channels = np.array(params.out_channels)
        self.n_in_channels, self.n_out_channels = len(self.in_channels), len(self.out_channels)
        self.add_zenith = g("add_zenith", False)
        self.dataset_path = g("h5_path", "fields")
        self.lat_lon = (params.lat, params.lon) if (g("lat") is not None and g("lon") is not None) else None
        io_grid, io_rank = g("io_grid", [1, 1, 1]), g("io_rank", [0, 0, 0])
        assert io_grid[0] == 1, "channel-parallel IO is not supported"
        self.io_grid, self.io_rank = io_grid[1:], io_rank[1:]
        self.crop_size = [g("crop_size_x"), g("crop_size_y")]
        self.crop_anchor = [g("crop_anchor_x", 0) or 0, g("crop_anchor_y", 0) or 0]
        self._get_files_stats(enable_logging)

        self.normalize = True
        norm = g("normalization", "zscore")
        if norm == "minmax":
            mn, mx = np.load(params.min_path), np.load(params.max_path)
            self.in_bias, self.in_scale = mn[:, self.in_channels], mx[:, self.in_channels] - mn[:, self.in_channels]
            self.out_bias, self.out_scale = mn[:, self.out_channels], mx[:, self.out_channels] - mn[:, self.out_channels]
        elif norm == "zscore":
            m, s = np.load(params.global_means_path), np.load(params.global_stds_path)
            self.in_bias, self.in_scale = m[:, self.in_channels], s[:, self.in_channels]
            self.out_bias, self.out_scale = m[:, self.out_channels], s[:, self.out_channels]
        else:
            self.normalize = False
            self.in_bias = np.zeros((1, self.n_in_channels, 1, 1), np.float32)
            self.in_scale = np.ones((1, self.n_in_channels, 1, 1), np.float32)
            self.out_bias = np.zeros((1, self.n_out_channels, 1, 1), np.float32)
            self.out_scale = np.ones((1, self.n_out_channels, 1, 1), np.float32)

        if self.lat_lon is None:
            res = 360.0 / float(self.img_shape[1])
            lon = np.arange(0, 360, res)
            lat = np.arange(-90, 90 + res, res)[::-1]
            self.lat_lon = (lat.tolist(), lon.tolist())
        if self.add_zenith:
            lon_g, lat_g = np.meshgrid(np.array(self.lat_lon[1]), np.array(self.lat_lon[0]))
            sl = (slice(self.read_anchor[0], self.read_anchor[0] + self.read_shape[0]),
                  slice(self.read_anchor[1], self.read_anchor[1] + self.read_shape[1]))
            self.lat_grid_local, self.lon_grid_local = lat_g[sl], lon_g[sl]
        self.grid_converter = GridConverter(g("data_grid_type", "equiangular"), g("model_grid_type", "equiangular"),
                                            torch.deg2rad(torch.tensor(self.lat_lon[0], dtype=torch.float32)),
                                            torch.deg2rad(torch.tensor(self.lat_lon[1], dtype=torch.float32)))

    # ---- files ------------------------------------------------------------------------------------
    def _open(self, path):
        if path.endswith(".npy"):
            return np.load(path, mmap_mode="r")
        import h5py
        return h5py.File(path, "r")[self.dataset_path]

    def _get_files_stats(self, enable_logging):
        locs = self.location if isinstance(self.location, list) else [self.location]
        paths = []
        for loc in locs:
            paths += glob.glob(os.path.join(loc, "????.h5")) + glob.glob(os.path.join(loc, "????.npy"))
        if not paths:
            raise IOError(f"Error, the specified file path {self.location} does not contain ????.h5 or ????.npy files.")
        self.files_paths = sorted(paths, key=lambda p: os.path.basename(p))
        self.years = [int(os.path.splitext(os.path.basename(x))[0]) for x in self.files_paths]
        self.files = [None] * len(self.files_paths)
        self.n_years = len(self.files_paths)
        first = self._open(self.files_paths[0])
        self.img_shape = tuple(first.shape[2:4])
        self.total_channels = first.shape[1]
        self.n_samples_year = [self._open(p).shape[0] for p in self.files_paths]
        if self.crop_size[0] is None:
            self.crop_size[0] = self.img_shape[0]
        if self.crop_size[1] is None:
            self.crop_size[1] = self.img_shape[1]
        assert self.crop_anchor[0] + self.crop_size[0] <= self.img_shape[0]
        assert self.crop_anchor[1] + self.crop_size[1] <= self.img_shape[1]
        sx = compute_split_shapes(self.crop_size[0], self.io_grid[0])
        sy = compute_split_shapes(self.crop_size[1], self.io_grid[1])
        self.read_shape = [sx[self.io_rank[0]], sy[self.io_rank[1]]]
        self.read_anchor = [self.crop_anchor[0] + sum(sx[: self.io_rank[0]]), self.crop_anchor[1] + sum(sy[: self.io_rank[1]])]
        self.year_offsets = [0] + list(accumulate(self.n_samples_year))[:-1]
        self.n_samples_available = self.n_samples_total = sum(self.n_samples_year)
        if enable_logging:
            logging.info(f"Found data at path {self.location}. Number of examples: {self.n_samples_available}. "
                         f"Full image shape: {self.img_shape[0]} x {self.img_shape[1]} x {self.total_channels}. "
                         f"Read shape: {self.read_shape[0]} x {self.read_shape[1]} x {self.n_in_channels}")
        self.img_shape_x, self.img_shape_y = self.img_shape
        self.img_crop_shape_x, self.img_crop_shape_y = self.crop_size
        self.img_crop_offset_x, self.img_crop_offset_y = self.crop_anchor
        self.img_local_shape_x, self.img_local_shape_y = self.read_shape
        self.img_local_offset_x, self.img_local_offset_y = self.read_anchor

    def _compute_zenith_angle(self, local_idx, year_idx):
        from ..zenith_angle import cos_zenith_angle
        jan1 = datetime.datetime(self.years[year_idx], 1, 1, 0, 0, 0, tzinfo=datetime.timezone.utc)
        it = [jan1 + datetime.timedelta(hours=i * self.dhours) for i in range(local_idx - self.dt * self.n_history, local_idx + 1, self.dt)]
        tt = [jan1 + datetime.timedelta(hours=i * self.dhours)
              for i in range(local_idx + self.dt, local_idx + self.dt * (self.n_future + 1) + 1, self.dt)]
        zi = np.expand_dims(cos_zenith_angle(it, self.lon_grid_local, self.lat_grid_local).astype(np.float32), axis=1)
        zt = np.expand_dims(cos_zenith_angle(tt, self.lon_grid_local, self.lat_grid_local).astype(np.float32), axis=1)
        return zi, zt

    def __len__(self):
        return self.n_samples_total - self.dt * (self.n_history + self.n_future + 1)

    def _read(self, global_idx, channels):
        yi = bisect_right(self.year_offsets, global_idx) - 1
        li = global_idx - self.year_offsets[yi]
        if self.files[yi] is None:
            self.files[yi] = self._open(self.files_paths[yi])
        sx, sy = self.read_anchor
        ex, ey = sx + self.read_shape[0], sy + self.read_shape[1]
        # channel fancy-index first (h5py needs increasing indices; numpy memmaps do not care), then the window
        arr = np.asarray(self.files[yi][li: li + 1, :, sx:ex, sy:ey])[:, channels]
        return arr.astype(np.float32, copy=False)

    def __getitem__(self, global_idx):
        inp = [self._read(global_idx + self.dt * o, self.in_channels) for o in range(self.n_history + 1)]
        tar = [self._read(global_idx + self.dt * o, self.out_channels)
               for o in range(self.n_history + 1, self.n_history + self.n_future + 2)]
        inp, tar = np.concatenate(inp, axis=0), np.concatenate(tar, axis=0)
        if self.normalize:
            inp = (inp - self.in_bias) / self.in_scale
            tar = (tar - self.out_bias) / self.out_scale
        result = (inp.astype(np.float32), tar.astype(np.float32))
        if self.add_zenith:
            yi = bisect_right(self.year_offsets, global_idx + self.dt * self.n_history) - 1
            li = global_idx + self.dt * self.n_history - self.year_offsets[yi]
            result = result + self._compute_zenith_angle(li, yi)
        return tuple(self.grid_converter(torch.as_tensor(np.ascontiguousarray(a))) for a in result)

    def get_output_normalization(self):
        return self.out_bias, self.out_scale

    def get_input_normalization(self):
        return self.in_bias, self.in_scale
