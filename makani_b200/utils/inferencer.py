"""Inference / scoring driver: autoregressive rollouts with metrics.

Public surface follows makani/utils/inferencer.py:44-314 (`score_model`, `inference_epoch`,
`inference_single(ic, compute_metrics, output_data, output_channels)`).  Unlike the reference, which parses
`--cuda_graph_mode` but always runs eagerly, the rollout step (model forward + history append) can be captured
once into a CUDA graph and replayed for every step (`cuda_graph_mode != "none"`): `rollout(ic, steps)`.
"""

from __future__ import annotations

import logging
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from ..models import model_registry
from ..models.helpers import count_parameters
from . import comm
from .dataloader import get_dataloader
from .losses import LossHandler
from .metric import MetricsHandler
from .trainer import Trainer, _amp_dtype


class Inferencer(Trainer):
    def __init__(self, params, world_rank):
        self.params = None
        self.world_rank = world_rank
        self.data_parallel_rank = comm.get_rank("data")
        self.device = torch.device(f"cuda:{torch.cuda.current_device()}") if torch.cuda.is_available() else torch.device("cpu")
        self.logger = logging.getLogger()
        g = params.get
        self.log_to_screen = g("log_to_screen", False)
        self.reducer = None
        self.amp_dtype = _amp_dtype(g("amp_mode", "none"))
        self.amp_enabled = self.amp_dtype is not None
        if g("log_to_wandb", False) and world_rank == 0:
            self._init_wandb(params, "inference")

        self.valid_dataloader, self.valid_dataset = get_dataloader(params, g("inf_data_path", g("valid_data_path")), self.device,
                                                                   train=False, final_eval=True)
        self.params = self._update_parameters(params)
        params = self.params
        self.model = model_registry.get_model(params).to(self.device)
        self.preprocessor = self.model.preprocessor
        if self.amp_dtype == torch.bfloat16 and self.device.type == "cuda" and hasattr(self.model.model, "set_compute_dtype"):
            self.model.model.set_compute_dtype(torch.bfloat16)
        self.optimizer = None
        self.scheduler = None
        self.iters = 0
        self.startEpoch = 0
        self.epoch = 0
        if g("checkpoint_path") is not None and g("pretrained", True) and os.path.exists(
                params.checkpoint_path.format(mp_rank=comm.get_rank("model") if g("load_checkpoint", "legacy") == "legacy" else 0)):
            self.restore_checkpoint(params.checkpoint_path, checkpoint_mode=g("load_checkpoint", "legacy"))
        self.model.eval()
        self.graph_mode = g("cuda_graph_mode", "none") if self.device.type == "cuda" else "none"
        self._rollout_graph = None

        mult_cpu, clim = self._get_time_stats()
        self.metrics = MetricsHandler(params, mult_cpu, clim, self.device)
        self.metrics.initialize_buffers()
        self.loss_obj = LossHandler(params).to(self.device)
        self.visualizer = None
        if self.log_to_screen:
            self.logger.info(f"Number of model parameters: {count_parameters(self.model, self.device)}")

    def _autoregressive_inference(self, data, compute_metrics=False, output_data=False, output_channels=[0, 1]):
        gdata = [x.to(self.device, dtype=torch.float32) for x in data]
        inp, tar = self.preprocessor.cache_unpredicted_features(*gdata)
        inp = self.preprocessor.flatten_history(inp)
        inpt = inp
        for idt, targ in enumerate(torch.split(tar, 1, dim=1)):
            targ = self.preprocessor.flatten_history(targ)
            with torch.autocast(device_type=self.device.type, dtype=self.amp_dtype, enabled=self.amp_enabled):
                pred = self.model(inpt)
                loss = self.loss_obj(pred, targ, inpt)
            if compute_metrics:
                self.metrics.update(pred, targ, loss, idt)
            if output_data:
                self.pred_outputs.append(pred[:, output_channels].float().cpu())
                self.targ_outputs.append(targ[:, output_channels].float().cpu())
            inpt = self.preprocessor.append_history(inpt.to(pred.dtype), pred, idt)

    @torch.no_grad()
    def inference_single(self, ic=0, compute_metrics=False, output_data=False, output_channels=[0, 1]):
        self._set_eval()
        if compute_metrics:
            self.metrics.zero_buffers()
        if output_data:
            self.targ_outputs, self.pred_outputs = [], []
        if hasattr(self.valid_dataset, "__getitem__"):
            data = [x.unsqueeze(0) for x in self.valid_dataset[ic]]
        else:
            it = iter(self.valid_dataloader)
            data = None
            for _ in range(ic + 1):
                data = next(it)
            data = [x[:1] for x in data]
        self._autoregressive_inference(data, compute_metrics=compute_metrics, output_data=output_data, output_channels=output_channels)
        result = []
        if output_data:
            result += [torch.stack(self.targ_outputs, dim=0), torch.stack(self.pred_outputs, dim=0)]
        if compute_metrics:
            logs, acc, rmse = self.metrics.finalize(final_inference=True)
            result += [logs, acc.cpu(), rmse.cpu()]
        return tuple(result)

    @torch.no_grad()
    def inference_epoch(self):
        self._set_eval()
        self.metrics.zero_buffers()
        for data in self.valid_dataloader:
            self._autoregressive_inference(data, compute_metrics=True, output_data=False, output_channels=False)
        if self.device.type == "cuda":
            from ..ops import _ext
            _ext.check_device_errors(self.device)    # expired bounded waits of the distributed kernels surface here
        logs, acc_curves, rmse_curves = self.metrics.finalize(final_inference=True)
        if self.world_rank == 0 and self.params.get("experiment_dir") is not None:
            os.makedirs(self.params.experiment_dir, exist_ok=True)
            np.save(os.path.join(self.params.experiment_dir, "acc_curves.npy"), acc_curves.cpu().numpy())
            np.save(os.path.join(self.params.experiment_dir, "rmse_curves.npy"), rmse_curves.cpu().numpy())
            try:
                from . import visualize
                visualize.plot_rollout_metrics(acc_curves, rmse_curves, self.params, epoch=0, model_name=self.params.nettype)
            except Exception as e:
                self.logger.info(f"rollout plots skipped: {e}")
        if dist.is_initialized():
            dist.barrier(device_ids=[self.device.index] if self.device.type == "cuda" else None)
        return logs

    # ---- CUDA-graphed rollout ------------------------------------------------------------------------
    @torch.no_grad()
    def rollout(self, inp: torch.Tensor, steps: int, keep_outputs: bool = False):
        """Autoregressive rollout from the flattened initial state `inp` [B, C, H, W] for `steps` steps.

        With `cuda_graph_mode != "none"` one step (forward + history append into a static state buffer) is captured
        once and replayed `steps` times.  Returns the final state (and the list of predictions if requested)."""
        self._set_eval()
        outputs = []

        def one_step(state):
            with torch.autocast(device_type=self.device.type, dtype=self.amp_dtype, enabled=self.amp_enabled):
                pred = self.model(state)
            return pred, self.preprocessor.append_history(state.to(pred.dtype), pred, 0)

        if self.graph_mode == "none":
            state = inp
            for _ in range(steps):
                pred, state = one_step(state)
                if keep_outputs:
                    outputs.append(pred.float().cpu())
            return (state, outputs) if keep_outputs else state

        if self._rollout_graph is None or self._static_state.shape != inp.shape:
            self._static_state = inp.clone()
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):
                    pred, nxt = one_step(self._static_state)
                side.synchronize()
                self._rollout_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self._rollout_graph, stream=side):
                    pred, nxt = one_step(self._static_state)
                    self._static_pred = pred
                    self._static_state.copy_(nxt.to(self._static_state.dtype))
            torch.cuda.current_stream(self.device).wait_stream(side)
        self._static_state.copy_(inp)
        for _ in range(steps):
            self._rollout_graph.replay()
            if keep_outputs:
                outputs.append(self._static_pred.float().cpu())
        if self.device.type == "cuda":
            from ..ops import _ext
            _ext.check_device_errors(self.device)
        return (self._static_state, outputs) if keep_outputs else self._static_state

    @torch.no_grad()
    def inference_ensemble(self, ic=0, n_members=8, noise_std=0.05, seed=0):
        """Initial-condition ensemble from sample `ic` of the evaluation set: `n_members` copies of the (normalised)
        initial state perturbed with N(0, noise_std^2) noise are rolled out together as one batch; per channel and
        lead time the quadrature-weighted RMSE of the ensemble mean, the ensemble spread and their ratio are returned
        as a dict of `[C_out, steps + 1]` tensors (and saved to the experiment directory on rank 0).
        The reference CLI declares this mode without implementing it (makani/inference.py:55,161-165)."""
        from .metrics.functions import GeometricRMSE
        self._set_eval()
        p = self.params
        data = [x.unsqueeze(0) for x in self.valid_dataset[ic]] if hasattr(self.valid_dataset, "__getitem__") else \
            [x[:1] for x in next(iter(self.valid_dataloader))]
        gdata = [x.to(self.device, dtype=torch.float32).expand(n_members, *x.shape[1:]).contiguous() for x in data]
        inp, tar = self.preprocessor.cache_unpredicted_features(*gdata)
        gen = torch.Generator(device=self.device).manual_seed(int(seed))
        inp = inp + float(noise_std) * torch.randn(inp.shape, device=self.device, generator=gen)
        state = self.preprocessor.flatten_history(inp)
        local = dict(local_shape=None, local_offset=(0, 0))
        if comm.get_size("spatial") > 1:
            local = dict(local_shape=(p.img_local_shape_x, p.img_local_shape_y), local_offset=(p.img_local_offset_x, p.img_local_offset_y))
        rule = "legendre-gauss" if p.get("model_grid_type", "equiangular") == "legendre-gauss" else "naive"
        rmse = GeometricRMSE(rule, img_shape=(p.img_shape_x, p.img_shape_y), crop_shape=(p.img_crop_shape_x, p.img_crop_shape_y),
                             crop_offset=(p.img_crop_offset_x, p.img_crop_offset_y), normalize=True, channel_reduction="none",
                             batch_reduction="none", **local).to(self.device)
        skill, spread = [], []
        for idt, targ in enumerate(torch.split(tar, 1, dim=1)):
            targ = self.preprocessor.flatten_history(targ)
            with torch.autocast(device_type=self.device.type, dtype=self.amp_dtype, enabled=self.amp_enabled):
                pred = self.model(state)
            pf = pred.float()
            mean = pf.mean(dim=0, keepdim=True)
            skill.append(rmse(mean, targ[:1].float())[0])
            # spread: root of the quadrature-weighted mean ensemble variance (unbiased over members)
            var = pf.var(dim=0, unbiased=n_members > 1, keepdim=True) if n_members > 1 else torch.zeros_like(mean)
            spread.append(rmse(torch.sqrt(var), torch.zeros_like(var))[0])
            state = self.preprocessor.append_history(state.to(pred.dtype), pred, idt)
        out = {"rmse": torch.stack(skill, dim=1).cpu(), "spread": torch.stack(spread, dim=1).cpu()}
        out["spread_skill_ratio"] = out["spread"] / out["rmse"].clamp_min(1e-12)
        if self.world_rank == 0 and p.get("experiment_dir") is not None:
            os.makedirs(p.experiment_dir, exist_ok=True)
            for k, v in out.items():
                np.save(os.path.join(p.experiment_dir, f"ensemble_{k}.npy"), v.numpy())
        return out

    def log_score(self, scoring_logs, scoring_time):
        if not self.log_to_screen:
            return
        sep = "-" * 50
        self.logger.info(sep)
        self.logger.info("Scoring summary:")
        self.logger.info("Total scoring time is {:.2f} sec".format(scoring_time))
        keys = [k for k in scoring_logs["metrics"].keys() if k != "rollouts"]
        width = max([len(k) for k in keys], default=0)
        self.logger.info("Metrics:")
        for k in keys:
            self.logger.info(f"    {k}: {' ' * (width - len(k))}{scoring_logs['metrics'][k]}")
        self.logger.info(sep)

    def score_model(self):
        if self.log_to_screen:
            self.logger.info("Starting Scoring...")
        if dist.is_initialized():
            dist.barrier(device_ids=[self.device.index] if self.device.type == "cuda" else None)
        t0 = time.time()
        logs = self.inference_epoch()
        self.log_score(logs, time.time() - t0)
        return logs
