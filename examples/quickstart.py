"""Quick start: train a tiny SFNO on an on-disk toy dataset, then use the two inference routes.

    python examples/quickstart.py [--workdir /tmp/makani_b200_quickstart] [--epochs 1]

1. writes a toy dataset (yearly `.npy` files, statistics, `data.json`) — replace with your own paths;
2. trains with `Trainer` (the same object `python -m makani_b200.train` drives);
3. route A — *model package*: reload the trained model from the experiment directory alone and call it with a time stamp;
4. route B — *Inferencer*: autoregressive rollout of one initial condition with ACC / RMSE curves, an
   initial-condition ensemble, and the scoring pass over the evaluation set.

Runs on CPU in well under a minute; on a B200 the same script uses the sm_100a kernels (`--amp_mode bf16`).
The flow mirrors notebooks/inference.ipynb of the reference.
"""

import argparse
import datetime
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from makani_b200 import Inferencer, Trainer  # noqa: E402
from makani_b200.models.model_package import LocalPackage, load_model_package  # noqa: E402
from makani_b200.utils.YParams import ParamsBase  # noqa: E402

CHANNELS = ["u10m", "t2m", "u500", "z500"]


def make_toy_dataset(root, nlat=33, nlon=64, days=16, seed=0):
    rng = np.random.default_rng(seed)
    lat = np.linspace(90, -90, nlat)
    lon = np.arange(nlon) * 360.0 / nlon
    base = np.cos(np.deg2rad(lat))[None, None, :, None] * np.sin(np.deg2rad(lon))[None, None, None, :]
    for sub, years in (("train", (2016, 2017)), ("test", (2019,))):
        os.makedirs(os.path.join(root, sub), exist_ok=True)
        for y in years:
            t = np.arange(days)[:, None, None, None]
            field = base * np.cos(0.3 * t) + 0.1 * rng.standard_normal((days, len(CHANNELS), nlat, nlon))
            np.save(os.path.join(root, sub, f"{y}.npy"), field.astype(np.float32))
    stats = os.path.join(root, "stats")
    os.makedirs(stats, exist_ok=True)
    c = len(CHANNELS)
    np.save(os.path.join(stats, "global_means.npy"), np.zeros((1, c, 1, 1), np.float32))
    np.save(os.path.join(stats, "global_stds.npy"), np.full((1, c, 1, 1), 0.5, np.float32))
    np.save(os.path.join(stats, "time_means.npy"), np.zeros((1, c, nlat, nlon), np.float32))
    os.makedirs(os.path.join(root, "metadata"), exist_ok=True)
    meta = dict(dataset_name="toy", h5_path="fields", dhours=24, attrs=dict(description="quick-start toy data"),
                coords=dict(grid_type="equiangular", lat=lat.tolist(), lon=lon.tolist(), channel=CHANNELS))
    with open(os.path.join(root, "metadata", "data.json"), "w") as f:
        json.dump(meta, f)
    return dict(train_data_path=os.path.join(root, "train"), valid_data_path=os.path.join(root, "test"),
                inf_data_path=os.path.join(root, "test"), global_means_path=os.path.join(stats, "global_means.npy"),
                global_stds_path=os.path.join(stats, "global_stds.npy"), time_means_path=os.path.join(stats, "time_means.npy"),
                metadata_json_path=os.path.join(root, "metadata", "data.json"), lat=lat.tolist(), lon=lon.tolist())


def make_params(paths, workdir, epochs):
    exp = os.path.join(workdir, "runs", "tiny_sfno", "0")
    os.makedirs(os.path.join(exp, "training_checkpoints"), exist_ok=True)
    p = ParamsBase()
    p.update_params(dict(
        paths, exp_dir=os.path.join(workdir, "runs"), experiment_dir=exp,
        checkpoint_path=os.path.join(exp, "training_checkpoints/ckpt_mp{mp_rank}.tar"),
        best_checkpoint_path=os.path.join(exp, "training_checkpoints/best_ckpt_mp{mp_rank}.tar"),
        # data
        dt=1, dhours=24, n_history=0, n_future=0, valid_autoreg_steps=4, batch_size=2, num_data_workers=0,
        in_channels=[0, 1, 2, 3], out_channels=[0, 1, 2, 3], channel_names=CHANNELS, normalization="zscore", h5_path="fields",
        add_zenith=False, add_grid=False, add_orography=False, add_landmask=False, io_grid=[1, 1, 1], io_rank=[0, 0, 0],
        data_grid_type="equiangular", model_grid_type="equiangular", sht_grid_type="legendre-gauss", enable_synthetic_data=False,
        # model
        nettype="SFNO", scale_factor=2, embed_dim=16, num_layers=2, filter_type="linear", operator_type="dhconv", use_mlp=True,
        mlp_ratio=2, activation_function="gelu", normalization_layer="instance_norm", pos_embed="none",
        hard_thresholding_fraction=1.0, complex_activation="real", separable=False,
        # optimisation
        loss="absolute squared geometric l2", channel_weights="auto", lr=2e-3, weight_decay=0.0, max_epochs=epochs,
        optimizer_type="AdamW", optimizer_beta1=0.9, optimizer_beta2=0.95, scheduler="StepLR", scheduler_step_size=10,
        scheduler_gamma=0.5, lr_warmup_steps=0, lr_start=2e-3, amp_mode="none", cuda_graph_mode="none",
        # bookkeeping
        skip_validation=False, log_to_screen=False, log_to_wandb=False, save_checkpoint="legacy", load_checkpoint="legacy",
        target="default", normalize_residual=False, finetune=False, resuming=False, checkpointing=0, disable_ddp=False,
        split_data_channels=False, print_timings_frequency=-1, history_normalization_mode="none"))
    return p


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--workdir", default="/tmp/makani_b200_quickstart")
    ap.add_argument("--epochs", type=int, default=1)
    args = ap.parse_args(argv)
    paths = make_toy_dataset(os.path.join(args.workdir, "data"))
    params = make_params(paths, args.workdir, args.epochs)

    trainer = Trainer(params, 0)
    trainer.train()
    print("validation loss after training:", trainer.metrics.logs["base"]["validation loss"])

    # route A: the model package (config.json + statistics + best checkpoint in the experiment directory)
    model = load_model_package(LocalPackage(params.experiment_dir), pretrained=True, device="cpu")
    x = torch.randn(1, len(CHANNELS), params.img_shape_x, params.img_shape_y)
    y = model(x, datetime.datetime(2019, 1, 1, tzinfo=datetime.timezone.utc))
    print("model package output:", tuple(y.shape))

    # route B: the Inferencer
    inf = Inferencer(params, 0)
    truth, pred, logs, acc, rmse = inf.inference_single(ic=0, compute_metrics=True, output_data=True, output_channels=[1, 3])
    lead = torch.arange(params.valid_autoreg_steps + 1) * params.dhours
    print("lead times [h]:", lead.tolist())
    print("ACC  t2m:", [round(float(v), 3) for v in acc[1]])
    print("RMSE z500:", [round(float(v), 3) for v in rmse[3]])
    ens = inf.inference_ensemble(ic=0, n_members=4, noise_std=0.05)
    print("ensemble spread/skill t2m:", [round(float(v), 3) for v in ens["spread_skill_ratio"][1]])
    scores = inf.score_model()
    print("scoring metrics:", {k: round(v, 4) for k, v in scores["metrics"].items() if isinstance(v, float)})
    return dict(trainer=trainer, inferencer=inf, truth=truth, pred=pred, acc=acc, rmse=rmse, ensemble=ens, scores=scores)


if __name__ == "__main__":
    main()
