"""Seeded synthetic data source: N(0,1) fields of the configured grid and channel shape, generated on the device.

Stands in for the reference's DALI/HDF5 pipeline (makani/utils/dataloaders/data_loader_dali_2d.py:42-332) and
replaces its `DummyLoader` (data_loader_dummy.py:35-190, which returns one fixed batch).  Every batch is a
pure function of (seed, epoch, step, data shard, spatial tile), so runs are reproducible across restarts and
across different model-parallel layouts; each rank generates only its own lat/lon tile.

Batch layout: `inp [B, n_history+1, C_in, H_loc, W_loc]`, `tar [B, T_out, C_out, H_loc, W_loc]` with
`T_out = n_future+1` (train) or `valid_autoreg_steps+1` (eval); with `add_zenith` also `izen`, `tzen` with one
channel.  Identity input/output normalisation.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ...parallel.helpers import compute_split_shapes
from ..grids import GridConverter


class SyntheticLoader:
    def __init__(self, params, location, train, device):
        self.params = params
        self.train = train
        self.device = torch.device(device)
        g = params.get
        self.dhours = g("dhours", 6)
        self.dt = g("dt", 1)
        self.batch_size = int(params.batch_size)
        self.n_history = g("n_history", 0)
        self.n_future = g("n_future", 0) if train else g("valid_autoreg_steps", 0)
        self.in_channels = list(g("in_channels", list(range(g("N_in_channels", 2)))))
        self.out_channels = list(g("out_channels", list(range(g("N_out_channels", 2)))))
        self.n_in_channels, self.n_out_channels = len(self.in_channels), len(self.out_channels)
        self.add_zenith = g("add_zenith", False)
        self.seed = int(g("synthetic_seed", g("seed", 333)))
        self.img_shape_x = g("img_shape_x", 721)
        self.img_shape_y = g("img_shape_y", 1440)
        self.img_crop_shape_x = g("crop_size_x") or self.img_shape_x
        self.img_crop_shape_y = g("crop_size_y") or self.img_shape_y
        self.img_crop_offset_x = g("crop_anchor_x", 0) or 0
        self.img_crop_offset_y = g("crop_anchor_y", 0) or 0
        io_grid = g("io_grid", [1, 1, 1])
        io_rank = g("io_rank", [0, 0, 0])
        sx = compute_split_shapes(self.img_crop_shape_x, io_grid[1])
        sy = compute_split_shapes(self.img_crop_shape_y, io_grid[2])
        self.img_local_shape_x, self.img_local_shape_y = sx[io_rank[1]], sy[io_rank[2]]
        self.img_local_offset_x = self.img_crop_offset_x + sum(sx[: io_rank[1]])
        self.img_local_offset_y = self.img_crop_offset_y + sum(sy[: io_rank[2]])
        self.tile_id = io_rank[1] * io_grid[2] + io_rank[2]
        self.shard_id = g("data_shard_id", 0)
        self.num_shards = g("data_num_shards", 1)
        n = g("n_train_samples_per_epoch" if train else "n_eval_samples_per_epoch") or g("n_train_samples" if train else "n_eval_samples") or (8 * self.batch_size * self.num_shards)
        self.num_steps_per_epoch = max(1, int(n) // (self.batch_size * self.num_shards))
        self.epoch = 0
        self.dtype = torch.float32
        if g("lat") is not None and g("lon") is not None:
            lat = torch.tensor(params.lat, dtype=torch.float32)
            lon = torch.tensor(params.lon, dtype=torch.float32)
        else:
            lat = torch.linspace(90.0, -90.0, self.img_shape_x)
            lon = torch.arange(self.img_shape_y, dtype=torch.float32) * (360.0 / self.img_shape_y)
        self.grid_converter = GridConverter(g("data_grid_type", "equiangular"), g("model_grid_type", "equiangular"),
                                            torch.deg2rad(lat), torch.deg2rad(lon))
        self.in_bias = np.zeros((1, self.n_in_channels, 1, 1), dtype=np.float32)
        self.in_scale = np.ones((1, self.n_in_channels, 1, 1), dtype=np.float32)
        self.out_bias = np.zeros((1, self.n_out_channels, 1, 1), dtype=np.float32)
        self.out_scale = np.ones((1, self.n_out_channels, 1, 1), dtype=np.float32)

    def get_input_normalization(self):
        return self.in_bias, self.in_scale

    def get_output_normalization(self):
        return self.out_bias, self.out_scale

    def __len__(self):
        return self.num_steps_per_epoch

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def _generator(self, step: int) -> torch.Generator:
        g = torch.Generator(device=self.device)
        mix = (self.seed * 1000003 + self.epoch * 7919 + step) * 4099 + self.shard_id * 131 + self.tile_id
        mix = mix * 2 + (1 if self.train else 0)
        g.manual_seed(mix % (2 ** 63 - 1))
        return g

    def __iter__(self):
        hl, wl = self.img_local_shape_x, self.img_local_shape_y
        B = self.batch_size
        for step in range(self.num_steps_per_epoch):
            g = self._generator(step)
            inp = torch.randn(B, self.n_history + 1, self.n_in_channels, hl, wl, device=self.device, generator=g, dtype=self.dtype)
            tar = torch.randn(B, self.n_future + 1, self.n_out_channels, hl, wl, device=self.device, generator=g, dtype=self.dtype)
            if self.add_zenith:
                izen = torch.rand(B, self.n_history + 1, 1, hl, wl, device=self.device, generator=g, dtype=self.dtype)
                tzen = torch.rand(B, self.n_future + 1, 1, hl, wl, device=self.device, generator=g, dtype=self.dtype)
                yield inp, tar, izen, tzen
            else:
                yield inp, tar
