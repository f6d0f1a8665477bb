"""Input/target pre- and post-processing around the network.

Responsibilities (behavioural contract: makani/models/preprocessor.py:30-426):
  * static features built once and cut to the rank's local lat/lon window: coordinate grid (optionally
    sin(k * grid), k = 1..grid_num_frequencies), z-scored orography, one-hot land-sea mask;
  * history handling: flatten [B,T,C,H,W] <-> [B,T*C,H,W], rolling window for autoregressive steps;
  * "unpredicted" channels (e.g. solar zenith angle) cached per train/eval mode, appended to every input and
    advanced from the target's copy during rollouts;
  * optional per-sample history normalisation (weighted mean/std over time and the global grid, reduced over
    the `spatial` group) and residual targets.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn as nn

from ..parallel.mappings import copy_to_parallel_region, reduce_from_parallel_region
from ..utils import comm
from ..utils.grids import GridConverter


class Preprocessor2D(nn.Module):
    def __init__(self, params):
        super().__init__()
        g = params.get
        self.n_history = g("n_history", 0)
        self.history_normalization_mode = g("history_normalization_mode", "none")
        nh = self.n_history
        if self.history_normalization_mode == "exponential":
            decay = params.history_normalization_decay
            w = torch.exp(-decay * torch.arange(start=nh, end=-1, step=-1, dtype=torch.float32))
            w = (w / w.sum()).reshape(1, -1, 1, 1, 1)
        elif self.history_normalization_mode == "mean":
            w = torch.full((nh + 1,), 1.0 / float(nh + 1), dtype=torch.float32).reshape(1, -1, 1, 1, 1)
        else:
            w = torch.ones(nh + 1, dtype=torch.float32)
        self.register_buffer("history_normalization_weights", w, persistent=False)
        self.history_mean = self.history_std = None
        self.history_diff_mean = self.history_diff_var = None
        self.history_eps = 1e-6

        self.learn_residual = g("target", "default") == "residual"
        if self.learn_residual and g("normalize_residual", False):
            rs = torch.from_numpy(np.load(params.time_diff_stds_path)).to(torch.float32)
            self.register_buffer("residual_scale", rs, persistent=False)
        else:
            self.residual_scale = None

        self.img_shape = [params.img_shape_x, params.img_shape_y]
        self.unpredicted_inp_train = self.unpredicted_tar_train = None
        self.unpredicted_inp_eval = self.unpredicted_tar_eval = None

        sx = g("img_local_offset_x", 0)
        ex = min(sx + g("img_local_shape_x", params.img_shape_x), params.img_shape_x)
        sy = g("img_local_offset_y", 0)
        ey = min(sy + g("img_local_shape_y", params.img_shape_y), params.img_shape_y)

        feats = []
        if g("add_grid", False):
            if g("lat") is not None and g("lon") is not None:
                lat = torch.tensor(params.lat, dtype=torch.float32)
                lon = torch.tensor(params.lon, dtype=torch.float32)
                gconv = GridConverter(g("data_grid_type", "equiangular"), g("model_grid_type", "equiangular"),
                                      torch.deg2rad(lat), torch.deg2rad(lon))
                tx, ty = (t.to(torch.float32) for t in gconv.get_dst_coords())
            else:
                tx = torch.linspace(0, 1, params.img_shape_x + 1, dtype=torch.float32)[:-1]
                ty = torch.linspace(0, 1, params.img_shape_y + 1, dtype=torch.float32)[:-1]
            xg, yg = torch.meshgrid(tx, ty, indexing="ij")
            grid = torch.stack([xg, yg], dim=0).unsqueeze(0)[:, :, sx:ex, sy:ey]
            if g("gridtype", "sinusoidal") == "sinusoidal":
                nfreq = int(g("grid_num_frequencies", 1))
                grid = torch.cat([torch.sin(f * grid) for f in range(1, nfreq + 1)], dim=1)
            feats.append(grid)
        if g("add_orography", False):
            from ..utils.conditioning_inputs import get_orography
            oro = torch.as_tensor(get_orography(params.orography_path), dtype=torch.float32)
            oro = oro.reshape(1, 1, *oro.shape[-2:])
            oro = (oro - oro.mean()) / (oro.std() + 1.0e-6)
            feats.append(oro[:, :, sx:ex, sy:ey])
        if g("add_landmask", False):
            from ..utils.conditioning_inputs import get_land_mask
            lsm = torch.as_tensor(get_land_mask(params.landmask_path), dtype=torch.long)
            lsm = torch.nn.functional.one_hot(lsm).permute(2, 0, 1).to(torch.float32).unsqueeze(0)
            feats.append(lsm[:, :, sx:ex, sy:ey])
        self.do_add_static_features = len(feats) > 0
        if self.do_add_static_features:
            self.register_buffer("static_features", torch.cat(feats, dim=1).contiguous(), persistent=False)

    # ---- history layout ---------------------------------------------------------------------------
    def flatten_history(self, x):
        if x.dim() == 5:
            b, t, c, h, w = x.shape
            x = x.reshape(b, t * c, h, w)
        return x

    def expand_history(self, x, nhist):
        if x.dim() == 4:
            b, ct, h, w = x.shape
            x = x.reshape(b, nhist, ct // nhist, h, w)
        return x

    def add_residual(self, x, dx):
        if not self.learn_residual:
            return dx
        if self.residual_scale is not None:
            dx = dx * self.residual_scale
        x = self.expand_history(x, nhist=self.n_history + 1)
        x = torch.cat([x[:, :-1], (x[:, -1] + dx).unsqueeze(1)], dim=1)
        return self.flatten_history(x)

    # ---- static features --------------------------------------------------------------------------
    def add_static_features(self, x):
        if self.do_add_static_features:
            st = self.static_features.to(x.dtype).expand(x.shape[0], -1, -1, -1)
            x = torch.cat([x, st], dim=1)
        return x

    def remove_static_features(self, x):
        if self.do_add_static_features:
            x = x[:, : x.shape[1] - self.static_features.shape[1]]
        return x

    # ---- autoregression ---------------------------------------------------------------------------
    def _unpredicted(self):
        if self.training:
            return self.unpredicted_inp_train, self.unpredicted_tar_train
        return self.unpredicted_inp_eval, self.unpredicted_tar_eval

    def append_history(self, x1, x2, step):
        uinp, utar_all = self._unpredicted()
        if utar_all is not None and step < utar_all.shape[1]:
            utar = utar_all[:, step: step + 1]
            if self.n_history == 0:
                uinp.copy_(utar)
            else:
                uinp.copy_(torch.cat([uinp[:, 1:], utar], dim=1))
        if self.n_history > 0:
            x1 = self.expand_history(x1, nhist=self.n_history + 1)
            x2 = self.expand_history(x2, nhist=1)
            return self.flatten_history(torch.cat([x1[:, 1:], x2], dim=1))
        return x2

    def append_channels(self, x, xc):
        xdim = x.dim()
        x = self.expand_history(x, self.n_history + 1)
        xc = self.expand_history(xc, self.n_history + 1)
        xo = torch.cat([x, xc.to(x.dtype)], dim=2)
        return self.flatten_history(xo) if xdim == 4 else xo

    # ---- per-sample history normalisation ---------------------------------------------------------
    def history_compute_stats(self, x):
        mode = self.history_normalization_mode
        npts = float(self.img_shape[0] * self.img_shape[1])
        if mode == "none":
            self.history_mean = torch.zeros((1, 1, 1, 1), dtype=torch.float32, device=x.device)
            self.history_std = torch.ones((1, 1, 1, 1), dtype=torch.float32, device=x.device)
            return
        xr = self.expand_history(x, self.n_history + 1)
        if mode == "timediff":
            d = xr[:, 1:] - xr[:, :-1]
            dm = torch.mean(torch.sum(d, dim=(3, 4)), dim=1)
            dm = reduce_from_parallel_region(dm, "spatial") / npts
            dv = torch.mean(torch.sum(torch.square(d - dm[:, None, :, None, None]), dim=(3, 4)), dim=1)
            dv = reduce_from_parallel_region(dv, "spatial") / npts
            self.history_diff_mean = copy_to_parallel_region(dm, "spatial")
            self.history_diff_var = copy_to_parallel_region(dv, "spatial")
            return
        w = self.history_normalization_weights
        m = torch.sum(xr * w, dim=(1, 3, 4), keepdim=True)
        m = reduce_from_parallel_region(m, "spatial") / npts
        s = torch.sum(torch.square(xr - m) * w, dim=(1, 3, 4), keepdim=True)
        s = torch.sqrt(reduce_from_parallel_region(s, "spatial") / npts)
        self.history_mean = copy_to_parallel_region(m.squeeze(1), "spatial")
        self.history_std = copy_to_parallel_region(s.squeeze(1), "spatial")

    def history_normalize(self, x, target=False):
        if self.history_normalization_mode in ("none", "timediff"):
            return x
        shape5 = x.shape if x.dim() == 5 else None
        x = self.flatten_history(x)
        if target:
            xn = (x - self.history_mean[:, : x.shape[1]]) / self.history_std[:, : x.shape[1]]
        else:
            hm = self.history_mean.repeat(1, self.n_history + 1, 1, 1)
            hs = self.history_std.repeat(1, self.n_history + 1, 1, 1)
            xn = (x - hm) / hs
        return xn.reshape(shape5) if shape5 is not None else xn

    def history_denormalize(self, xn, target=False):
        if self.history_normalization_mode in ("none", "timediff"):
            return xn
        shape5 = xn.shape if xn.dim() == 5 else None
        xn = self.flatten_history(xn)
        if target:
            x = xn * self.history_std[:, : xn.shape[1]] + self.history_mean[:, : xn.shape[1]]
        else:
            hm = self.history_mean.repeat(1, self.n_history + 1, 1, 1)
            hs = self.history_std.repeat(1, self.n_history + 1, 1, 1)
            x = xn * hs + hm
        return x.reshape(shape5) if shape5 is not None else x

    # ---- unpredicted (e.g. zenith angle) channels -------------------------------------------------
    def cache_unpredicted_features(self, x, y, xz=None, yz=None):
        def upd(cur, new):
            if cur is not None and new is not None and cur.shape == new.shape:
                cur.copy_(new)
                return cur
            return new.clone() if new is not None else None

        if self.training:
            self.unpredicted_inp_train = upd(self.unpredicted_inp_train, xz)
            self.unpredicted_tar_train = upd(self.unpredicted_tar_train, yz)
        else:
            self.unpredicted_inp_eval = upd(self.unpredicted_inp_eval, xz)
            self.unpredicted_tar_eval = upd(self.unpredicted_tar_eval, yz)
        return x, y

    def append_unpredicted_features(self, inp):
        uinp, _ = self._unpredicted()
        return self.append_channels(inp, uinp) if uinp is not None else inp

    def remove_unpredicted_features(self, inp):
        uinp, _ = self._unpredicted()
        if uinp is not None:
            f = self.expand_history(inp, nhist=self.n_history + 1)
            inp = self.flatten_history(f[:, :, : f.shape[2] - uinp.shape[2]])
        return inp


def get_preprocessor(params):
    return Preprocessor2D(params)
