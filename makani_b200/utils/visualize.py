"""Optional CPU plotting of fields and rollout metrics (matplotlib, Agg backend), off the timed path.

Behaviour contract: makani/utils/visualize.py:27-235 — Mollweide maps of prediction vs target rendered to
in-memory PNGs, line plots of ACC / RMSE rollout curves saved as `acc_*.png` / `rmse_*.png`, and a wrapper that
renders frames in a process pool and assembles them into a GIF.  Without matplotlib the maps and curves are drawn by
the small numpy + PIL rasteriser below (Mollweide resampling, built-in colour ramps, polyline plots); without PIL
everything degrades to a no-op.
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


def _have_matplotlib() -> bool:
    try:
        import matplotlib  # noqa: F401
        return True
    except ImportError:
        return False


# ------------------------------------------------------------------------------------------------ raster fallback

_RAMPS = {
    # piecewise-linear colour ramps as (position, r, g, b)
    "sequential": [(0.0, 68, 1, 84), (0.25, 59, 82, 139), (0.5, 33, 145, 140), (0.75, 94, 201, 98), (1.0, 253, 231, 37)],
    "diverging": [(0.0, 5, 48, 97), (0.25, 67, 147, 195), (0.5, 247, 247, 247), (0.75, 214, 96, 77), (1.0, 103, 0, 31)],
}


def colorize(field: np.ndarray, vmin: float, vmax: float, diverging: bool = False) -> np.ndarray:
    """[H, W] float -> [H, W, 3] uint8 through a built-in colour ramp; NaNs become white."""
    ramp = np.array(_RAMPS["diverging" if diverging else "sequential"], dtype=np.float64)
    x = (np.asarray(field, dtype=np.float64) - vmin) / max(vmax - vmin, 1e-30)
    nan = ~np.isfinite(x)
    x = np.clip(np.where(nan, 0.0, x), 0.0, 1.0)
    rgb = np.stack([np.interp(x, ramp[:, 0], ramp[:, c]) for c in (1, 2, 3)], axis=-1)
    rgb[nan] = 255.0
    return rgb.astype(np.uint8)


def mollweide_resample(field: np.ndarray, width: int = 360) -> np.ndarray:
    """Equirectangular [H, W] field (north at row 0, longitudes 0..360 or -180..180) -> Mollweide raster
    [width / 2, width] with NaN outside the ellipse (nearest-neighbour lookup through the inverse projection)."""
    H, W = field.shape
    h = width // 2
    xs = (np.arange(width) + 0.5) / width * 2.0 - 1.0          # x / (2 sqrt 2) in [-1, 1]
    ys = 1.0 - (np.arange(h) + 0.5) / h * 2.0                  # y / sqrt 2 in [1, -1]
    X, Y = np.meshgrid(xs, ys)
    theta = np.arcsin(np.clip(Y, -1.0, 1.0))
    inside = X ** 2 + Y ** 2 <= 1.0
    lat = np.arcsin(np.clip((2.0 * theta + np.sin(2.0 * theta)) / np.pi, -1.0, 1.0))
    cos_t = np.maximum(np.cos(theta), 1e-12)
    lon = np.pi * X / cos_t                                     # [-pi, pi]
    rows = np.clip(np.round((np.pi / 2.0 - lat) / np.pi * (H - 1)).astype(int), 0, H - 1)
    cols = np.round((lon + np.pi) / (2.0 * np.pi) * W).astype(int) % W
    out = np.full((h, width), np.nan)
    out[inside] = np.asarray(field, dtype=np.float64)[rows[inside], cols[inside]]
    return out


def _raster_comparison(pred, truth, diverging, vmax, projection, width=360):
    from PIL import Image
    pred, truth = np.asarray(pred, dtype=np.float64), np.asarray(truth, dtype=np.float64)
    vmax = vmax or max(np.abs(pred).max(), np.abs(truth).max())
    vmin = -vmax if diverging else min(pred.min(), truth.min())
    frames = []
    for f in (pred, truth):
        g = mollweide_resample(f, width) if projection == "mollweide" else f
        frames.append(colorize(g, vmin, vmax, diverging))
    gap = np.full((8, frames[0].shape[1], 3), 255, dtype=np.uint8)
    return Image.fromarray(np.concatenate([frames[0], gap, frames[1]], axis=0))


def _raster_curve(t, y, title, size=(480, 320)):
    """Polyline plot of one curve with axis box and min / max labels (PIL only)."""
    from PIL import Image, ImageDraw
    Wp, Hp = size
    img = Image.new("RGB", size, (255, 255, 255))
    d = ImageDraw.Draw(img)
    l, r, tp, b = 50, Wp - 15, 30, Hp - 35
    d.rectangle([l, tp, r, b], outline=(0, 0, 0))
    y = np.asarray(y, dtype=np.float64)
    t = np.asarray(t, dtype=np.float64)
    lo, hi = float(np.nanmin(y)), float(np.nanmax(y))
    if hi - lo < 1e-12:
        hi = lo + 1.0
    px = l + (t - t.min()) / max(t.max() - t.min(), 1e-12) * (r - l)
    py = b - (y - lo) / (hi - lo) * (b - tp)
    pts = list(zip(px.tolist(), py.tolist()))
    if len(pts) > 1:
        d.line(pts, fill=(31, 119, 180), width=2)
    for x_, y_ in pts:
        d.ellipse([x_ - 3, y_ - 3, x_ + 3, y_ + 3], fill=(31, 119, 180))
    d.text((l, 8), title, fill=(0, 0, 0))
    d.text((4, tp - 5), f"{hi:.3g}", fill=(0, 0, 0))
    d.text((4, b - 8), f"{lo:.3g}", fill=(0, 0, 0))
    d.text((l, b + 8), f"{t.min():g} h", fill=(0, 0, 0))
    d.text((r - 40, b + 8), f"{t.max():g} h", fill=(0, 0, 0))
    return img


def plot_comparison(pred, truth, lat=None, lon=None, pred_title="Prediction", truth_title="Ground truth", cmap="twilight_shifted",
                    projection="mollweide", diverging=False, figsize=(4, 6), vmax=None):
    """Render prediction and target side by side (stacked) and return a PIL image."""
    if not _have_matplotlib():
        return _raster_comparison(pred, truth, diverging, vmax, projection)
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
    plt = _plt() if _have_matplotlib() else None
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
            if plt is None:
                _raster_curve(t, curve[idx], f"{kind.upper()} {ch} ({model_name})").save(
                    os.path.join(params.experiment_dir, f"{kind}_{ch}.png"))
                continue
            fig = plt.figure(figsize=(8, 6))
            plt.plot(t, curve[idx], ".-", label=model_name)
            plt.xlabel("lead time [h]")
            plt.ylabel(kind.upper())
            plt.title(f"{kind.upper()} {ch}")
            plt.legend()
            plt.grid(True)
            fig.savefig(os.path.join(params.experiment_dir, f"{kind}_{ch}.png"))
            plt.close(fig)


def visualize_field(tag, func_string, prediction, target, lat, lon, scale, bias, diverging):
    """One comparison frame: un-normalise (`scale * x + bias`), apply the functor given as source text (e.g.
    `"lambda x: np.sqrt(np.square(x[0]) + np.square(x[1]))"`, as in makani/utils/visualize.py:135-154) and plot
    prediction beside target.  Returns `(tag, image)`."""
    func = eval(func_string)      # the plot list of a recipe is trusted configuration, exactly as upstream
    pred, targ = func(scale * prediction + bias), func(scale * target + bias)
    image = plot_comparison(pred, targ, lat, lon, pred_title="Prediction", truth_title="Ground truth", projection="mollweide",
                            diverging=diverging)
    return tag, image


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
        # spawned (not forked) workers: the parent is multi-threaded and usually holds a CUDA context
        import multiprocessing
        self.executor = ProcessPoolExecutor(max_workers=max(1, num_workers), mp_context=multiprocessing.get_context("spawn"))
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
