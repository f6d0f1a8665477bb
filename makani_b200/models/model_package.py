"""Self-contained model packages: everything beyond the checkpoint that inference outside the trainer needs.

Contract: makani/models/model_package.py:36-268 — `save_model_package(params)` writes `config.json` (the
parameter dict), copies normalisation statistics and invariant fields, and writes `metadata.json` with the
entry point of `load_time_loop`; `load_model_package(package)` rebuilds the single-GPU model from those files and
`training_checkpoints/best_ckpt_mp0.tar`; `ModelWrapper.forward(x, time)` appends the cosine of the solar
zenith angle when the model was trained with it.
"""

from __future__ import annotations

import json
import logging
import os
import shutil

import numpy as np
import torch

from ..utils.checkpoint import load_file
from ..utils.YParams import ParamsBase
from ..utils.zenith_angle import cos_zenith_angle
from . import model_registry

logger = logging.getLogger(__name__)

THIS_MODULE = "makani_b200.models.model_package"
MODEL_PACKAGE_CHECKPOINT_PATH = "training_checkpoints/best_ckpt_mp0.tar"
MINS_FILE, MAXS_FILE = "mins.npy", "maxs.npy"
MEANS_FILE, STDS_FILE = "global_means.npy", "global_stds.npy"
OROGRAPHY_FILE, LANDMASK_FILE = "orography.nc", "land_mask.nc"


class LocalPackage:
    """Directory-backed package (the `get(path)` interface earth2mip packages expose)."""

    def __init__(self, root):
        self.root = root

    def get(self, path):
        return os.path.join(self.root, path)


class ModelWrapper(torch.nn.Module):
    """Single prediction step `forward(x, time)` for use outside the trainer."""

    def __init__(self, model, params):
        super().__init__()
        self.model, self.params = model, params
        nlat, nlon = params.img_shape_x, params.img_shape_y
        self.lats = 90 - 180 * np.arange(nlat) / (nlat - 1)
        self.lons = 360 * np.arange(nlon) / nlon
        self.add_zenith = params.get("add_zenith", False)

    def forward(self, x, time):
        if self.add_zenith:
            lon_grid, lat_grid = np.meshgrid(self.lons, self.lats)
            cosz = cos_zenith_angle(time, lon_grid, lat_grid).astype(np.float32)
            z = torch.from_numpy(cosz).to(device=x.device)
            while z.ndim != x.ndim:
                z = z[None]
            x = torch.cat([x, z.expand(x.shape[0], *z.shape[1:])], dim=1)
        return self.model(x)


def _jsonable(v):
    if isinstance(v, (np.integer,)):
        return int(v)
    if isinstance(v, (np.floating,)):
        return float(v)
    if isinstance(v, np.ndarray):
        return v.tolist()
    if isinstance(v, (list, tuple)):
        return [_jsonable(x) for x in v]
    if isinstance(v, dict):
        return {k: _jsonable(x) for k, x in v.items()}
    if isinstance(v, (str, int, float, bool)) or v is None:
        return v
    return str(v)


def save_model_package(params):
    exp = params.experiment_dir
    os.makedirs(exp, exist_ok=True)
    with open(os.path.join(exp, "config.json"), "w") as f:
        json.dump(_jsonable(params.to_dict()), f, indent=2)

    def cp(src, name):
        if src is not None and os.path.exists(src):
            shutil.copy(src, os.path.join(exp, name))

    g = params.get
    if g("add_orography", False):
        cp(g("orography_path"), OROGRAPHY_FILE if str(g("orography_path")).endswith(".nc") else "orography.npy")
    if g("add_landmask", False):
        cp(g("landmask_path"), LANDMASK_FILE if str(g("landmask_path")).endswith(".nc") else "land_mask.npy")
    cp(g("global_means_path"), MEANS_FILE)
    cp(g("global_stds_path"), STDS_FILE)
    if g("normalization") == "minmax":
        cp(g("min_path"), MINS_FILE)
        cp(g("max_path"), MAXS_FILE)
    with open(os.path.join(exp, "metadata.json"), "w") as f:
        json.dump({"entrypoint": {"name": f"{THIS_MODULE}:load_time_loop"}}, f, indent=2)


def _load_static_data(package, params):
    g = params.get
    if g("add_orography", False):
        name = OROGRAPHY_FILE if os.path.exists(package.get(OROGRAPHY_FILE)) else "orography.npy"
        params.orography_path = package.get(name)
    if g("add_landmask", False):
        name = LANDMASK_FILE if os.path.exists(package.get(LANDMASK_FILE)) else "land_mask.npy"
        params.landmask_path = package.get(name)
    if g("normalization") == "zscore":
        params.global_means_path = package.get(MEANS_FILE)
        params.global_stds_path = package.get(STDS_FILE)
    elif g("normalization") == "minmax":
        params.min_path = package.get(MINS_FILE)
        params.max_path = package.get(MAXS_FILE)


def load_model_package(package, pretrained=True, device="cpu"):
    """Rebuild the (single-GPU) model described by `config.json` of the package and load its best checkpoint."""
    params = ParamsBase.from_json(package.get("config.json"))
    _load_static_data(package, params)
    # the package is always evaluated on one device with the full grid
    params.img_local_offset_x = params.img_local_offset_y = 0
    params.img_local_shape_x = params.get("img_crop_shape_x", params.img_shape_x)
    params.img_local_shape_y = params.get("img_crop_shape_y", params.img_shape_y)
    params.n_future = 0
    model = model_registry.get_model(params).to(device)
    if pretrained:
        ckpt = load_file(package.get(MODEL_PACKAGE_CHECKPOINT_PATH))
        state = ckpt["model_state"]
        torch.nn.modules.utils.consume_prefix_in_state_dict_if_present(state, "module.")
        model.load_state_dict(state, strict=True)
    model = ModelWrapper(model, params=params)
    model.eval()
    return model


def load_time_loop(package, device=None, time_step_hours=None):
    """Entry point for earth2mip: wraps the packaged model in its `Inference` time loop (needs earth2mip)."""
    try:
        from earth2mip.networks import Inference
        from earth2mip.grid import equiangular_lat_lon_grid
    except ImportError as e:
        raise ImportError("load_time_loop needs the earth2mip package") from e
    import datetime

    config = ParamsBase.from_json(package.get("config.json"))
    model = load_model_package(package, pretrained=True, device=device or "cpu")
    names = [config.channel_names[i] for i in config.out_channels] if config.get("out_channels") else config.channel_names
    center = np.load(package.get(MEANS_FILE))[0, config.out_channels, 0, 0]
    scale = np.load(package.get(STDS_FILE))[0, config.out_channels, 0, 0]
    grid = equiangular_lat_lon_grid(config.img_shape_x, config.img_shape_y, includes_south_pole=True)
    dt = datetime.timedelta(hours=time_step_hours or config.get("dt", 1) * config.get("dhours", 6))
    inference = Inference(model, channel_names=names, center=center, scale=scale, grid=grid,
                          n_history=config.get("n_history", 0), time_step=dt)
    inference.to(device)
    return inference
