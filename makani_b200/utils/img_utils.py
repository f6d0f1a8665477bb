"""Image helpers (behaviour of makani/utils/img_utils.py:34-110): periodic padding in longitude, and the sample
preparation of the numpy data path (normalise, grid channels, roll, crop, flatten the history)."""

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F


class PeriodicPad2d(nn.Module):
    """Circular padding in the last (longitude) dimension, zero padding in latitude."""

    def __init__(self, pad_width):
        super().__init__()
        self.pad_width = pad_width

    def forward(self, x):
        out = F.pad(x, (self.pad_width, self.pad_width, 0, 0), mode="circular")
        return F.pad(out, (0, 0, self.pad_width, self.pad_width), mode="constant", value=0)


def reshape_fields(img, inp_or_tar, crop_size_x, crop_size_y, rnd_x, rnd_y, params, y_roll, train, normalize=True):
    """Turn a numpy sample `[n_history + 1, C, H, W]` (or `[C, H, W]`) into the tensor the networks take:
    `[(n_history + 1) * C, h, w]` for an input, `[C, h, w]` for a target.

    Steps, in the order of makani/utils/img_utils.py:51-110: drop columns beyond 720 (the legacy 721 x 1440 -> 720 x 1440
    crop acts on the latitude axis of those files), normalise with the statistics files named in `params` ("minmax" or
    "zscore"), append the grid channels to an input when `params.add_grid` ("linear": 2 channels, "sinusoidal": 4),
    roll in longitude by `y_roll`, crop a `crop_size_x x crop_size_y` window at (`rnd_x`, `rnd_y`) when training."""
    img = np.asarray(img)
    if img.ndim == 3:
        img = img[None]
    img = img[:, :, 0:720]
    n_history, n_channels = img.shape[0] - 1, img.shape[1]
    H, W = img.shape[-2], img.shape[-1]
    channels = params.in_channels if inp_or_tar == "inp" else params.out_channels
    crop_size_x = H if crop_size_x is None else crop_size_x
    crop_size_y = W if crop_size_y is None else crop_size_y
    if normalize:
        if params.normalization == "minmax":
            lo, hi = np.load(params.min_path)[:, channels], np.load(params.max_path)[:, channels]
            img = (img - lo) / (hi - lo)
        elif params.normalization == "zscore":
            mu, sd = np.load(params.global_means_path)[:, channels], np.load(params.global_stds_path)[:, channels]
            img = (img - mu) / sd
    if params.add_grid and inp_or_tar == "inp":
        if params.gridtype == "linear":
            assert params.n_grid_channels == 2, "n_grid_channels must be set to 2 for gridtype linear"
            gy, gx = np.meshgrid(np.linspace(-1, 1, W), np.linspace(-1, 1, H))
            grid = np.stack((gy, gx), axis=0)[None]
        elif params.gridtype == "sinusoidal":
            assert params.n_grid_channels == 4, "n_grid_channels must be set to 4 for gridtype sinusoidal"
            ax, ay = np.linspace(0, 2 * np.pi, H), np.linspace(0, 2 * np.pi, W)
            sy, sx = np.meshgrid(np.sin(ay), np.sin(ax))
            cy, cx = np.meshgrid(np.cos(ay), np.cos(ax))
            grid = np.stack((sy, sx, cy, cx), axis=0)[None]
        else:
            raise ValueError(f"unknown gridtype {params.gridtype}")
        img = np.concatenate((img, np.broadcast_to(grid, (img.shape[0],) + grid.shape[1:])), axis=1)
        n_channels = img.shape[1]
    if params.roll:
        img = np.roll(img, y_roll, axis=-1)
    if train and (crop_size_x or crop_size_y):
        img = img[:, :, rnd_x: rnd_x + crop_size_x, rnd_y: rnd_y + crop_size_y]
    if inp_or_tar == "inp":
        img = np.reshape(img, (n_channels * (n_history + 1), crop_size_x, crop_size_y))
    elif inp_or_tar == "tar":
        img = np.reshape(img, (n_channels, crop_size_x, crop_size_y))
    return torch.as_tensor(np.ascontiguousarray(img))
