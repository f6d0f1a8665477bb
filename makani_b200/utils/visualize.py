"""Optional CPU plotting of fields and rollout metrics (matplotlib, Agg backend), off the timed path.

Behaviour contract: makani/utils/visualize.py:27-235 — Mollweide maps of prediction vs target rendered to
in-memory PNGs, line plots of ACC / RMSE rollout curves saved as `acc_*.png` / `rmse_*.png`, and a wrapper that
renders frames in a process pool and assembles them into a GIF.  Everything degrades to a no-op when matplotlib
(or PIL) is not installed.
"""

from __future__ import annotations

import io
import logging
import os
from concurrent.futures import ProcessPoolExecutor

import numpy as np


def _plt():
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    return plt


def plot_comparison(pred, truth, lat=None, lon=None, pred_title="Prediction", truth_title="Ground truth", cmap="twilight_shifted",
                    projection="mollweide", diverging=False, figsize=(4, 6), vmax=None):
    """Render prediction and target side by side (stacked) and return a PIL image."""
    plt = _plt()
    from PIL import Image
    H, W = pred.shape
    if lon is None:
        lon = np.linspace(-np.pi, np.pi, W)
    if lat is None:
        lat = np.linspace(np.pi / 2.0, -np.pi / 2.0, H)
    Lon, Lat = np.meshgrid(lon, lat)
    vmax = vmax or max(np.abs(pred).max(), np.abs(truth).max())
    vmin = -vmax if diverging else min(pred.min(), truth.min())
    fig = plt.figure(figsize=figsize)
    for k, (field, title) in enumerate(((pred, pred_title), (truth, truth_title))):
        ax = fig.add_subplot(2, 1, k + 1, projection=projection)
        ax.pcolormesh(Lon, Lat, field, cmap=cmap, vmax=vmax, vmin=vmin)
        ax.set_title(title)
        ax.grid(True)
        ax.set_xticklabels([])
        ax.set_yticklabels([])
    fig.tight_layout()
    buf = io.BytesIO()
    fig.savefig(buf, format="png")
    plt.close(fig)
    buf.seek(0)
    return Image.open(buf)


def plot_rollout_metrics(acc_curves, rmse_curves, params, epoch, model_name, comparison_channels=("u10m", "t2m", "u500", "z500", "r500", "q500")):
    """Line plots of the ACC and RMSE rollout curves of selected variables into the experiment directory."""
    plt = _plt()
    acc = np.asarray(acc_curves.cpu() if hasattr(acc_curves, "cpu") else acc_curves)
    rmse = np.asarray(rmse_curves.cpu() if hasattr(rmse_curves, "cpu") else rmse_curves)
    dtxdh = params.get("dt", 1) * params.get("dhours", 6)
    t = np.arange(1, acc.shape[1] + 1) * dtxdh
    names = list(params.get("channel_names", []))
    for ch in comparison_channels:
        if ch not in names:
            continue
        idx = names.index(ch)
        for kind, curve in (("acc", acc), ("rmse", rmse)):
            fig = plt.figure(figsize=(8, 6))
            plt.plot(t, curve[idx], ".-", label=model_name)
            plt.xlabel("lead time [h]")
            plt.ylabel(kind.upper())
            plt.title(f"{kind.upper()} {ch}")
            plt.legend()
            plt.grid(True)
            fig.savefig(os.path.join(params.experiment_dir, f"{kind}_{ch}.png"))
            plt.close(fig)


def _render(args):
    pred, targ, lat, lon, title = args
    try:
        return plot_comparison(pred, targ, lat, lon, pred_title=title + " prediction", truth_title=title + " target")
    except Exception as e:  # plotting must never take a training run down
        logging.getLogger().info(f"visualisation frame skipped: {e}")
        return None


class VisualizationWrapper:
    """Collects (prediction, target) frames, renders them in worker processes and writes a GIF per plotted field."""

    def __init__(self, log_to_wandb, path, prefix, plot_list, lat=None, lon=None, scale=1.0, bias=0.0, num_workers=1):
        self.log_to_wandb, self.path, self.prefix = log_to_wandb, path, prefix or "viz"
        self.plot_list = plot_list or [{"name": "channel0", "functor": "lambda x: x[0]", "diverging": False}]
        self.lat, self.lon = lat, lon
        self.scale = np.asarray(scale, dtype=np.float32).reshape(-1, 1, 1) if np.ndim(scale) else scale
        self.bias = np.asarray(bias, dtype=np.float32).reshape(-1, 1, 1) if np.ndim(bias) else bias
        self.executor = ProcessPoolExecutor(max_workers=max(1, num_workers))
        self.requests = []

    def reset(self):
        self.requests = []

    def add(self, tag, prediction, target):
        pred = prediction * self.scale + self.bias
        targ = target * self.scale + self.bias
        for item in self.plot_list:
            fn = eval(item["functor"]) if isinstance(item["functor"], str) else item["functor"]
            self.requests.append((item["name"], tag, self.executor.submit(_render, (fn(pred), fn(targ), self.lat, self.lon, item["name"]))))

    def finalize(self):
        frames = {}
        for name, tag, fut in self.requests:
            img = fut.result()
            if img is not None:
                frames.setdefault(name, []).append(img)
        out = {}
        for name, imgs in frames.items():
            if self.path is not None and imgs:
                fname = os.path.join(self.path, f"{self.prefix}_{name}.gif")
                imgs[0].save(fname, save_all=True, append_images=imgs[1:], duration=400, loop=0)
                out[name] = fname
        if self.log_to_wandb and out:
            try:
                import wandb
                wandb.log({name: wandb.Video(f) for name, f in out.items()})
            except Exception:
                pass
        self.reset()
        return out
