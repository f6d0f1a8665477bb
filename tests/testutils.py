"""Shared fixtures: default parameter bags and tiny on-disk datasets (yearly .npy files + statistics)."""

import json
import os

import numpy as np

from makani_b200.utils.YParams import ParamsBase


def get_default_parameters(**over):
    p = ParamsBase()
    d = dict(
        dt=1, dhours=24, n_history=0, n_future=0, valid_autoreg_steps=2, batch_size=2, num_data_workers=0,
        in_channels=[0, 1, 2, 3], out_channels=[0, 1, 2, 3], channel_names=["u10m", "t2m", "u500", "z500"],
        normalization="zscore", add_zenith=False, add_grid=False, add_orography=False, add_landmask=False,
        data_grid_type="equiangular", model_grid_type="equiangular", sht_grid_type="legendre-gauss",
        io_grid=[1, 1, 1], io_rank=[0, 0, 0], enable_synthetic_data=False, h5_path="fields",
        nettype="SFNO", scale_factor=2, embed_dim=16, num_layers=2, filter_type="linear", operator_type="dhconv",
        use_mlp=True, mlp_ratio=2, activation_function="gelu", normalization_layer="instance_norm", pos_embed="none",
        hard_thresholding_fraction=1.0, complex_activation="real", separable=False,
        loss="absolute squared geometric l2", channel_weights="auto", lr=1e-3, weight_decay=0.0, max_epochs=1,
        optimizer_type="AdamW", optimizer_beta1=0.9, optimizer_beta2=0.999, scheduler="StepLR", scheduler_step_size=10,
        scheduler_gamma=0.5, lr_warmup_steps=0, lr_start=1e-3, amp_mode="none", cuda_graph_mode="none",
        skip_validation=False, log_to_screen=False, log_to_wandb=False, save_checkpoint="legacy", load_checkpoint="legacy",
        target="default", normalize_residual=False, finetune=False, resuming=False, checkpointing=0, disable_ddp=False,
        split_data_channels=False, print_timings_frequency=-1, history_normalization_mode="none",
    )
    d.update(over)
    p.update_params(d)
    return p


def init_dataset(path, nlat=33, nlon=64, nchan=4, ndays=24, years=(2016, 2017), test_years=(2019,), seed=0):
    """Writes train/<year>.npy, test/<year>.npy ([T, C, H, W] float32), stats/*.npy and metadata/data.json."""
    rng = np.random.default_rng(seed)
    for sub, ys in (("train", years), ("test", test_years)):
        os.makedirs(os.path.join(path, sub), exist_ok=True)
        for y in ys:
            arr = rng.standard_normal((ndays, nchan, nlat, nlon)).astype(np.float32) + 0.5
            np.save(os.path.join(path, sub, f"{y}.npy"), arr)
    st = os.path.join(path, "stats")
    os.makedirs(st, exist_ok=True)
    np.save(os.path.join(st, "global_means.npy"), np.full((1, nchan, 1, 1), 0.5, dtype=np.float32))
    np.save(os.path.join(st, "global_stds.npy"), np.full((1, nchan, 1, 1), 1.5, dtype=np.float32))
    np.save(os.path.join(st, "mins.npy"), np.full((1, nchan, 1, 1), -5.0, dtype=np.float32))
    np.save(os.path.join(st, "maxs.npy"), np.full((1, nchan, 1, 1), 5.0, dtype=np.float32))
    np.save(os.path.join(st, "time_means.npy"), np.full((1, nchan, nlat, nlon), 0.5, dtype=np.float32))
    np.save(os.path.join(st, "time_diff_means.npy"), np.zeros((1, nchan, 1, 1), dtype=np.float32))
    np.save(os.path.join(st, "time_diff_stds.npy"), np.ones((1, nchan, 1, 1), dtype=np.float32))
    md = os.path.join(path, "metadata")
    os.makedirs(md, exist_ok=True)
    lat = np.linspace(90, -90, nlat).tolist()
    lon = (np.arange(nlon) * 360.0 / nlon).tolist()
    meta = dict(dataset_name="testset", h5_path="fields", dhours=24, attrs=dict(description="random test data"),
                coords=dict(grid_type="equiangular", lat=lat, lon=lon, channel=["u10m", "t2m", "u500", "z500"][:nchan]))
    with open(os.path.join(md, "data.json"), "w") as f:
        json.dump(meta, f)
    paths = dict(train_data_path=os.path.join(path, "train"), valid_data_path=os.path.join(path, "test"),
                 inf_data_path=os.path.join(path, "test"), global_means_path=os.path.join(st, "global_means.npy"),
                 global_stds_path=os.path.join(st, "global_stds.npy"), min_path=os.path.join(st, "mins.npy"),
                 max_path=os.path.join(st, "maxs.npy"), time_means_path=os.path.join(st, "time_means.npy"),
                 time_diff_means_path=os.path.join(st, "time_diff_means.npy"),
                 time_diff_stds_path=os.path.join(st, "time_diff_stds.npy"), metadata_json_path=os.path.join(md, "data.json"),
                 lat=lat, lon=lon)
    return paths
