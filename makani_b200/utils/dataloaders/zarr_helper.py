"""Loader over a zarr store holding one `fields[time, channel, lat, lon]` array (e.g. an ARCO-style ERA5 cube).

Behaviour contract: makani/utils/dataloaders/zarr_helper.py:60-184 — samples are consecutive (input, target) pairs
`dt` steps apart, z-score normalised with `global_means_path` / `global_stds_path` of shape `[1, C, 1, 1]`, sharded
over the data group with a `DistributedSampler`; the returned loader carries `get_input_normalization`,
`get_output_normalization` and `reset_pipeline`, and the second return value describes the geometry.

`xarray` / `zarr` are optional: when they are absent (they are not part of the base image) an array-like opened by
the caller can be passed as `store` instead, e.g. a numpy memory map, which is also how the unit test drives it.
"""

from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset


def _open_fields(files_pattern):
    try:
        import xarray
        ds = xarray.open_zarr(files_pattern)
        return ds["fields"], getattr(ds, "time", None)
    except ImportError:
        pass
    try:
        import zarr
        return zarr.open(files_pattern, mode="r")["fields"], None
    except ImportError as e:
        raise ImportError("reading a zarr store needs `xarray` or `zarr`; pass an opened array as `store=` instead") from e


class ZarrPairs(Dataset):
    def __init__(self, fields, in_channels, out_channels, dt, mean, std, n_samples=None):
        self.fields, self.dt = fields, int(dt)
        self.in_channels, self.out_channels = np.asarray(in_channels), np.asarray(out_channels)
        self.in_mean, self.in_std = mean[0, self.in_channels], std[0, self.in_channels]
        self.out_mean, self.out_std = mean[0, self.out_channels], std[0, self.out_channels]
        n = int(fields.shape[0]) - self.dt
        self.n = n if n_samples is None else min(n, int(n_samples))

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        x = np.asarray(self.fields[i])[self.in_channels]
        y = np.asarray(self.fields[i + self.dt])[self.out_channels]
        x = (x - self.in_mean) / self.in_std
        y = (y - self.out_mean) / self.out_std
        return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)), torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32))


def get_data_loader(params, files_pattern, train: bool, store=None):
    fields = store if store is not None else _open_fields(files_pattern)[0]
    mean, std = np.load(params.global_means_path), np.load(params.global_stds_path)
    nchan = int(fields.shape[1])
    assert mean.shape == (1, nchan, 1, 1) and std.shape == (1, nchan, 1, 1), (mean.shape, std.shape)
    assert not np.isnan(mean).any() and not np.isnan(std).any()
    g = params.get
    dataset = ZarrPairs(fields, params.in_channels, params.out_channels, g("dt", 1), mean, std,
                        g("n_train_samples") if train else g("n_eval_samples"))
    sampler = None
    if g("data_num_shards", 1) > 1:
        from torch.utils.data.distributed import DistributedSampler
        sampler = DistributedSampler(dataset, shuffle=train, num_replicas=params.data_num_shards, rank=params.data_shard_id)
    loader = DataLoader(dataset, batch_size=int(params.batch_size), num_workers=g("num_data_workers", 0), shuffle=False,
                        sampler=sampler if train else None, drop_last=True, pin_memory=torch.cuda.is_available())
    loader.get_input_normalization = lambda: (mean[:, dataset.in_channels], std[:, dataset.in_channels])
    loader.get_output_normalization = lambda: (mean[:, dataset.out_channels], std[:, dataset.out_channels])
    loader.reset_pipeline = lambda: None
    nlat, nlon = int(fields.shape[-2]), int(fields.shape[-1])
    meta = SimpleNamespace(img_shape_x=nlat, img_shape_y=nlon, img_crop_shape_x=nlat, img_crop_shape_y=nlon,
                           img_crop_offset_x=0, img_crop_offset_y=0, img_local_shape_x=nlat, img_local_shape_y=nlon,
                           img_local_offset_x=0, img_local_offset_y=0, in_channels=list(params.in_channels),
                           out_channels=list(params.out_channels))
    if train:
        return loader, meta, sampler
    return loader, meta
