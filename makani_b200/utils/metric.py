"""Validation metrics: loss, L1, per-variable RMSE / ACC rollout curves and ACC area-under-curve.

Contract: makani/utils/metric.py:27-306 (`initialize_buffers`, `zero_buffers`, `update(pred, targ, loss, idt)`,
`finalize(final_inference)` -> logs dict with "base" and "metrics"; curves accumulate on the device, are
all-reduced over the `data` group and copied to pinned host buffers on a side stream).  The rollout table is a
plain list of rows (and a `wandb.Table` when wandb logging is enabled and importable).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import comm
from .metrics.functions import GeometricACC, GeometricL1, GeometricRMSE, Quadrature

_DEFAULT_VARS = ["u10m", "t2m", "u500", "z500", "r500", "q500"]


class MetricsHandler:
    def __init__(self, params, mult, clim, device, rmse_var_names=_DEFAULT_VARS, acc_vars_names=_DEFAULT_VARS,
                 acc_auc_var_names=_DEFAULT_VARS):
        self.device = torch.device(device)
        g = params.get
        self.log_to_screen = g("log_to_screen", False)
        self.log_to_wandb = g("log_to_wandb", False)
        self.channel_names = list(g("channel_names", []) or [])
        self.stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.dtxdh = g("dt", 1) * g("dhours", 6)
        self.dd = max(1, 24 // self.dtxdh)
        names = self.channel_names
        self.rmse_vars = {v: names.index(v) for v in rmse_var_names if v in names}
        self.acc_vars = {v: names.index(v) for v in acc_vars_names if v in names}
        self.acc_auc_vars = {v: names.index(v) for v in acc_auc_var_names if v in names}
        self.split_data_channels = g("split_data_channels", False)
        self.mult = mult.to(self.device)
        self.valid_autoreg_steps = g("valid_autoreg_steps", 0)
        self.simpquad = Quadrature(self.valid_autoreg_steps, 1.0 / float(self.valid_autoreg_steps + 1), self.device)
        self.clim = torch.unsqueeze(clim, 0).to(self.device, dtype=torch.float32)
        self.N_out_channels = params.N_out_channels
        msize = comm.get_size("matmul")
        if self.split_data_channels and msize > 1:
            self.out_channels_local = (self.N_out_channels + msize - 1) // msize
            self.clim = torch.split(self.clim, self.out_channels_local, dim=1)[comm.get_rank("matmul")].contiguous()
        else:
            self.split_data_channels = False
            self.out_channels_local = self.N_out_channels
        img = (params.img_shape_x, params.img_shape_y)
        crop = (params.img_crop_shape_x, params.img_crop_shape_y)
        off = (params.img_crop_offset_x, params.img_crop_offset_y)
        local = dict(local_shape=None, local_offset=(0, 0))
        if comm.get_size("spatial") > 1:
            local = dict(local_shape=(params.img_local_shape_x, params.img_local_shape_y),
                         local_offset=(params.img_local_offset_x, params.img_local_offset_y))
            lx, ly = params.img_local_offset_x - off[0], params.img_local_offset_y - off[1]
            self.clim = self.clim[..., lx: lx + params.img_local_shape_x, ly: ly + params.img_local_shape_y].contiguous()
        rule = "legendre-gauss" if g("model_grid_type", "equiangular") == "legendre-gauss" else "naive"
        common = dict(img_shape=img, crop_shape=crop, crop_offset=off, normalize=True, **local)
        self.l1_handle = GeometricL1(rule, channel_reduction="mean", batch_reduction="sum", **common).to(self.device)
        self.rmse_handle = GeometricRMSE(rule, channel_reduction="none", batch_reduction="none", **common).to(self.device)
        self.acc_handle = GeometricACC(rule, channel_reduction="none", batch_reduction="sum", **common).to(self.device)

    def initialize_buffers(self):
        nsteps = self.valid_autoreg_steps + 1
        dev = self.device
        self.valid_buffer = torch.zeros(3, dtype=torch.float32, device=dev)
        self.valid_loss, self.valid_l1, self.valid_steps = (self.valid_buffer[i].view(-1) for i in range(3))
        self.acc_curve = torch.zeros((self.out_channels_local, nsteps), dtype=torch.float32, device=dev)
        self.rmse_curve = torch.zeros((self.out_channels_local, nsteps), dtype=torch.float32, device=dev)
        self.acc_counter = torch.zeros(nsteps, dtype=torch.float32, device=dev)
        pin = dev.type == "cuda"
        self.valid_buffer_cpu = torch.zeros(3, dtype=torch.float32, pin_memory=pin)
        self.acc_curve_cpu = torch.zeros((self.N_out_channels, nsteps), dtype=torch.float32, pin_memory=pin)
        self.acc_auc_cpu = torch.zeros(self.N_out_channels, dtype=torch.float32, pin_memory=pin)
        self.rmse_curve_cpu = torch.zeros((self.N_out_channels, nsteps), dtype=torch.float32, pin_memory=pin)

    def zero_buffers(self):
        with torch.no_grad():
            self.valid_buffer.zero_()
            self.acc_curve.zero_()
            self.rmse_curve.zero_()
            self.acc_counter.zero_()

    @torch.no_grad()
    def update(self, prediction, target, loss, idt):
        prediction, target = prediction.float(), target.float()
        self.acc_curve[:, idt] += self.acc_handle(prediction - self.clim, target - self.clim)
        self.rmse_curve[:, idt] += self.mult * torch.sum(self.rmse_handle(prediction, target), dim=0)
        self.acc_counter[idt] += 1
        if idt == 0:
            self.valid_steps += 1.0
            self.valid_loss += loss.float()
            self.valid_l1 += self.l1_handle(prediction, target)

    def _gather_channels(self, curve):
        msize = comm.get_size("matmul")
        pad = self.out_channels_local * msize
        bufs = [torch.zeros_like(curve) for _ in range(msize)]
        dist.all_gather(bufs, curve.contiguous(), group=comm.get_group("matmul"))
        return torch.cat(bufs, dim=0)[: self.N_out_channels] if pad >= self.N_out_channels else torch.cat(bufs, dim=0)

    @torch.no_grad()
    def finalize(self, final_inference=False):
        if dist.is_initialized():
            dist.barrier(device_ids=[self.device.index] if self.device.type == "cuda" else None)
        valid_steps_local = int(self.valid_steps.item())
        if dist.is_initialized() and comm.get_size("data") > 1:
            grp = comm.get_group("data")
            for t in (self.valid_buffer, self.acc_curve, self.rmse_curve, self.acc_counter):
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=grp)
        acc_curve, rmse_curve = self.acc_curve, self.rmse_curve
        if self.split_data_channels:
            l1 = self.valid_buffer[1:2]
            dist.all_reduce(l1, op=dist.ReduceOp.SUM, group=comm.get_group("matmul"))
            l1 /= comm.get_size("matmul")
            acc_curve, rmse_curve = self._gather_channels(acc_curve), self._gather_channels(rmse_curve)
        self.valid_buffer[0:2] = self.valid_buffer[0:2] / torch.clamp(self.valid_buffer[2], min=1.0)
        acc_curve = acc_curve / torch.clamp(self.acc_counter, min=1.0)
        rmse_curve = rmse_curve / torch.clamp(self.acc_counter, min=1.0)
        acc_auc = self.simpquad(acc_curve, dim=1)
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self.valid_buffer_cpu.copy_(self.valid_buffer, non_blocking=True)
                self.acc_curve_cpu.copy_(acc_curve, non_blocking=True)
                self.rmse_curve_cpu.copy_(rmse_curve, non_blocking=True)
                self.acc_auc_cpu.copy_(acc_auc, non_blocking=True)
            self.stream.synchronize()
        else:
            self.valid_buffer_cpu.copy_(self.valid_buffer)
            self.acc_curve_cpu.copy_(acc_curve)
            self.rmse_curve_cpu.copy_(rmse_curve)
            self.acc_auc_cpu.copy_(acc_auc)
        vb = self.valid_buffer_cpu.numpy()
        logs = {"base": {"validation steps": valid_steps_local, "validation loss": float(vb[0]), "validation L1": float(vb[1])},
                "metrics": {}}
        rm = self.rmse_curve_cpu[:, 0].numpy()
        for name, idx in self.rmse_vars.items():
            logs["metrics"]["validation " + name] = float(rm[idx])
        auc = self.acc_auc_cpu.numpy()
        for name, idx in self.acc_auc_vars.items():
            logs["metrics"]["ACC AUC " + name] = float(auc[idx])
        table = []
        acc_arr, rmse_arr = self.acc_curve_cpu.numpy(), self.rmse_curve_cpu.numpy()
        for name, idx in self.acc_vars.items():
            for d in range(self.valid_autoreg_steps + 1):
                table.append(["ACC", name, (d + 1) * self.dtxdh, float(acc_arr[idx, d])])
        for name, idx in self.rmse_vars.items():
            for d in range(self.valid_autoreg_steps + 1):
                table.append(["RMSE", name, (d + 1) * self.dtxdh, float(rmse_arr[idx, d])])
        columns = ["metric type", "variable name", "time [h]", "value"]
        rollouts = {"columns": columns, "data": table}
        if self.log_to_wandb:
            try:
                import wandb
                rollouts = wandb.Table(data=table, columns=columns)
            except Exception:
                pass
        logs["metrics"]["rollouts"] = rollouts
        self.logs = logs
        self.acc_curve_final, self.rmse_curve_final = acc_curve, rmse_curve
        if final_inference:
            return logs, acc_curve, rmse_curve
        return logs
