"""Training driver.

Public surface and experiment layout follow makani/utils/trainer.py:57-1193: `Trainer(params, world_rank)`,
`.train()`, `.train_one_epoch()`, `.validate_one_epoch(epoch)`, `.save_checkpoint(...)`,
`.restore_checkpoint(...)`, `.test_autoregression_pipeline()`, `.log_weights_and_grads(...)`.

What is different by design:
  * no DistributedDataParallel wrapper: gradients live in one flat buffer (`GradReducer`) that is averaged over
    the `data` group by an in-kernel NVLink all-reduce and summed over the model-parallel groups each parameter
    is replicated on (same semantics as the reference's DDP comm hook, makani/mpu/mappings.py:104-169);
  * Adam/AdamW are the fused multi-tensor sm_100a kernel on CUDA;
  * `cuda_graph_mode` "fwdbwd" captures forward+backward (+ gradient reduction) of the static-shape step,
    "step" additionally captures the optimiser update (its hyper-parameters live in device memory);
  * checkpoints are written by `makani_b200.utils.checkpoint` in the same legacy / flexible formats.
"""

from __future__ import annotations

import gc
import logging
import os
import time
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..models import model_registry
from ..models.helpers import count_parameters
from ..ops import _ext
from ..ops.optim import FusedAdamW
from ..parallel.grad_reduce import GradReducer
from ..parallel.helpers import sync_params
from . import checkpoint as ckpt
from . import comm
from .dataloader import get_dataloader
from .features import get_auxiliary_channels
from .losses import LossHandler
from .metric import MetricsHandler


def _amp_dtype(mode: str) -> Optional[torch.dtype]:
    return {"none": None, "fp16": torch.float16, "bf16": torch.bfloat16}[mode or "none"]


class Trainer:
    # ------------------------------------------------------------------------------------------ setup
    def __init__(self, params, world_rank, job_type="train"):
        self.params = None
        self.world_rank = world_rank
        self.data_parallel_rank = comm.get_rank("data")
        self.device = torch.device(f"cuda:{torch.cuda.current_device()}") if torch.cuda.is_available() else torch.device("cpu")
        self.logger = logging.getLogger()
        g = params.get
        self.log_to_screen = g("log_to_screen", False)

        if dist.is_initialized():
            # one small all-reduce up front so that communicators exist before anything is timed or captured
            tens = torch.ones(1, device=self.device)
            dist.all_reduce(tens, group=comm.get_group("data"))

        self.amp_dtype = _amp_dtype(g("amp_mode", "none"))
        self.amp_enabled = self.amp_dtype is not None

        if g("log_to_wandb", False) and world_rank == 0:
            self._init_wandb(params, job_type)

        # data
        if self.log_to_screen:
            self.logger.info("initializing data loader")
        self.train_dataloader, self.train_dataset, self.train_sampler = get_dataloader(
            params, g("train_data_path"), self.device, train=True)
        self.valid_dataloader, self.valid_dataset = get_dataloader(params, g("valid_data_path"), self.device, train=False)

        self.params = self._update_parameters(params)
        params = self.params

        if world_rank == 0 and g("experiment_dir") is not None and not g("enable_synthetic_data", False):
            try:
                from ..models.model_package import save_model_package
                save_model_package(params)
            except Exception as e:  # missing stats files etc. must not stop a run
                self.logger.warning(f"model package not written: {e}")

        # model
        self.model = model_registry.get_model(params).to(self.device)
        self.preprocessor = self.model.preprocessor
        if self.amp_dtype == torch.bfloat16 and self.device.type == "cuda" and hasattr(self.model.model, "set_compute_dtype"):
            self.model.model.set_compute_dtype(torch.bfloat16)
        if dist.is_initialized():
            sync_params(self.model, mode="broadcast")

        mult_cpu, clim = self._get_time_stats()
        self.metrics = MetricsHandler(params, mult_cpu, clim, self.device)
        self.metrics.initialize_buffers()
        self.loss_obj = LossHandler(params).to(self.device)

        self.reducer = None
        if (dist.is_initialized() and not g("disable_ddp", False)) or self.device.type == "cuda":
            self.reducer = GradReducer(self.model)
        self.optimizer = self._make_optimizer(params)
        self.scheduler = self._make_scheduler(params)
        self.gscaler = torch.amp.GradScaler(self.device.type, enabled=(self.amp_dtype == torch.float16))

        self._set_train()
        self.graph = None
        self.graph_mode = g("cuda_graph_mode", "none") if self.device.type == "cuda" else "none"
        if self.graph_mode == "step" and self.amp_dtype == torch.float16:
            # the captured optimiser launch cannot honour the loss scaler's inf/NaN check; keep the scaler on the host
            if self.log_to_screen:
                self.logger.info("amp_mode fp16: cuda_graph_mode 'step' falls back to 'fwdbwd' (the GradScaler steps on the host)")
            self.graph_mode = "fwdbwd"

        self.visualizer = None
        if g("log_video", 0) and g("log_video", 0) > 0:
            try:
                from . import visualize
                out_bias, out_scale = self.train_dataloader.get_output_normalization()
                lat, lon = self.valid_dataset.grid_converter.get_dst_coords()
                self.visualizer = visualize.VisualizationWrapper(
                    g("log_to_wandb", False), path=g("experiment_dir"), prefix="viz", plot_list=[],
                    lat=lat.cpu().numpy(), lon=lon.cpu().numpy() - np.pi, scale=out_scale[0], bias=out_bias[0],
                    num_workers=g("num_visualization_workers", 1))
            except Exception as e:
                self.logger.warning(f"visualisation disabled: {e}")

        self.iters = 0
        self.startEpoch = 0
        if g("finetune", False) and not g("resuming", False):
            assert g("pretrained_checkpoint_path") is not None, "Error, please specify a valid pretrained checkpoint path"
            self.restore_checkpoint(params.pretrained_checkpoint_path, checkpoint_mode=params.load_checkpoint,
                                    load_optimizer=params.load_optimizer, load_scheduler=params.load_scheduler,
                                    load_counters=params.load_counters)
        if g("resuming", False):
            self.restore_checkpoint(params.checkpoint_path, checkpoint_mode=params.load_checkpoint,
                                    load_optimizer=params.load_optimizer, load_scheduler=params.load_scheduler,
                                    load_counters=params.load_counters)
        self.epoch = self.startEpoch

        pcount = count_parameters(self.model, self.device)
        if self.log_to_screen:
            self.logger.info(f"Number of trainable model parameters: {pcount}")

    def _init_wandb(self, params, job_type):
        try:
            import wandb
        except ImportError:
            params.log_to_wandb = False
            return
        g = params.get
        mode = os.environ.get("WANDB_MODE", "offline")
        wandb.init(dir=g("wandb_dir", g("experiment_dir")), config=params.to_dict(), name=g("wandb_name"),
                   group=g("wandb_group"), project=g("wandb_project"), entity=g("wandb_entity"), job_type=job_type,
                   resume="allow", mode=mode,
                   tags=[f"ngpu{comm.get_world_size()}", f"mp{comm.get_size('model')}", f"sp{comm.get_size('spatial')}"])

    def _update_parameters(self, params):
        """The single place where dataset-derived and defaulted parameters are filled in."""
        ds = self.valid_dataset
        params.N_in_channels = len(ds.in_channels)
        params.N_out_channels = len(ds.out_channels)
        for k in ("img_shape_x", "img_shape_y", "img_crop_shape_x", "img_crop_shape_y", "img_crop_offset_x", "img_crop_offset_y",
                  "img_local_shape_x", "img_local_shape_y", "img_local_offset_x", "img_local_offset_y"):
            params[k] = getattr(ds, k)
        params["N_in_predicted_channels"] = params.N_in_channels
        defaults = dict(add_zenith=False, add_grid=False, add_orography=False, add_landmask=False, n_history=0, n_future=0,
                        history_normalization_mode="none", num_visualization_workers=1, log_video=0, log_weights_and_grads=0,
                        skip_validation=False, load_checkpoint="legacy", save_checkpoint="legacy", load_optimizer=True,
                        load_scheduler=True, load_counters=True, target="default", normalize_residual=False,
                        valid_autoreg_steps=0, optimizer_type="AdamW", optimizer_beta1=0.9, optimizer_beta2=0.999,
                        weight_decay=0.0, lr=1e-3, scheduler="None", lr_warmup_steps=0, lr_start=1e-3, max_epochs=1,
                        checkpointing=0, split_data_channels=False, print_timings_frequency=-1, log_to_screen=False,
                        log_to_wandb=False, gridtype="sinusoidal", loss="l2", channel_weights="auto")
        for k, v in defaults.items():
            if params.get(k) is None and k not in params:
                params[k] = v
        if params.add_zenith:
            params.N_in_channels += 1
        if params.n_history >= 1:
            params.N_in_channels = (params.n_history + 1) * params.N_in_channels
            params.N_in_predicted_channels *= params.n_history + 1
        if params.add_grid:
            n_grid = 2
            if params.gridtype == "sinusoidal" and params.get("grid_num_frequencies") is not None:
                n_grid *= params.grid_num_frequencies
            params.N_in_channels += n_grid
        if params.add_orography:
            params.N_in_channels += 1
        if params.add_landmask:
            params.N_in_channels += 2
        params["aux_channel_names"] = get_auxiliary_channels(**params.to_dict())
        params.N_target_channels = (params.n_future + 1) * params.N_out_channels
        if params.get("channel_names") is None:
            params["channel_names"] = [f"ch{i}" for i in range(params.N_out_channels)]
        return params

    def _get_time_stats(self):
        """Output scale for de-normalised RMSE and the climatology (normalised time mean) for ACC."""
        p = self.params
        _, out_scale = self.valid_dataloader.get_output_normalization()
        mult_cpu = torch.from_numpy(np.asarray(out_scale))[0, :, 0, 0].float()
        shape = (p.N_out_channels, p.img_crop_shape_x, p.img_crop_shape_y)
        if p.get("enable_synthetic_data", False) or p.get("time_means_path") is None:
            clim = torch.zeros(shape, dtype=torch.float32)
        else:
            in_bias, in_scale = self.valid_dataloader.get_input_normalization()
            sx, sy = p.img_crop_offset_x, p.img_crop_offset_y
            tm = np.load(p.time_means_path)[0, p.out_channels, sx: sx + p.img_crop_shape_x, sy: sy + p.img_crop_shape_y]
            clim = torch.as_tensor((tm - in_bias[0]) / in_scale[0], dtype=torch.float32)
        return mult_cpu, clim

    def _make_optimizer(self, p):
        betas = (p.optimizer_beta1, p.optimizer_beta2)
        params = [q for q in self.model.parameters() if q.requires_grad]
        ot = p.optimizer_type
        if ot in ("Adam", "AdamW", "FusedAdam"):
            if self.device.type == "cuda":
                return FusedAdamW(params, lr=p.lr, betas=betas, weight_decay=p.weight_decay, adamw=(ot != "Adam"),
                                  complex_mode=p.get("optimizer_complex_mode", "split"))
            cls = torch.optim.Adam if ot == "Adam" else torch.optim.AdamW
            return cls(params, betas=betas, lr=p.lr, weight_decay=p.weight_decay)
        if ot == "SGD":
            return torch.optim.SGD(params, lr=p.lr, weight_decay=p.weight_decay, momentum=p.get("momentum", 0.0))
        if ot in ("FusedLAMB", "LAMB"):
            from ..ops.optim import LAMB
            return LAMB(params, lr=p.lr, betas=betas, weight_decay=p.weight_decay, max_grad_norm=p.get("optimizer_max_grad_norm", 1.0))
        raise ValueError(f"Unknown optimizer type {ot}")

    def _make_scheduler(self, p):
        sched = None
        name = p.get("scheduler", "None")
        if name == "ReduceLROnPlateau":
            if p.skip_validation:
                raise ValueError("Error, you cannot skip validation when using ReduceLROnPlateau scheduler.")
            sched = torch.optim.lr_scheduler.ReduceLROnPlateau(self.optimizer, factor=p.scheduler_factor,
                                                               patience=p.scheduler_patience, mode=p.get("scheduler_mode", "min"))
        elif name == "StepLR":
            sched = torch.optim.lr_scheduler.StepLR(self.optimizer, step_size=p.scheduler_step_size, gamma=p.scheduler_gamma)
        elif name == "CosineAnnealingLR":
            sched = torch.optim.lr_scheduler.CosineAnnealingLR(self.optimizer, T_max=p.scheduler_T_max, eta_min=p.get("scheduler_min_lr", 0.0))
        elif name == "OneCycleLR":
            sched = torch.optim.lr_scheduler.OneCycleLR(self.optimizer, max_lr=p.lr, total_steps=p.scheduler_T_max, steps_per_epoch=1)
        if p.get("lr_warmup_steps", 0) > 0:
            if name == "ReduceLROnPlateau":
                raise NotImplementedError("Error, warmup scheduler not implemented for ReduceLROnPlateau scheduler")
            warm = torch.optim.lr_scheduler.LinearLR(self.optimizer, start_factor=p.lr_start, end_factor=1.0, total_iters=p.lr_warmup_steps)
            if sched is None:
                sched = warm
            else:
                sched = torch.optim.lr_scheduler.SequentialLR(self.optimizer, [warm, sched], milestones=[p.lr_warmup_steps])
        return sched

    # ------------------------------------------------------------------------------------------ modes
    def _set_train(self):
        self.model.train()
        self.loss_obj.train()
        self.preprocessor.train()

    def _set_eval(self):
        self.model.eval()
        self.loss_obj.eval()
        self.preprocessor.eval()

    def __del__(self):
        try:
            if getattr(self, "reducer", None) is not None:
                self.reducer.close()
        except Exception:
            pass

    # ------------------------------------------------------------------------------------------ one step
    def _forward_backward(self, inp, tar):
        if self.reducer is not None:
            self.reducer.zero_grad()
        else:
            self.optimizer.zero_grad(set_to_none=True)
        with torch.autocast(device_type=self.device.type, dtype=self.amp_dtype, enabled=self.amp_enabled):
            pred = self.model(inp)
            loss = self.loss_obj(pred, tar, inp)
        self.gscaler.scale(loss).backward()
        if self.reducer is not None:
            self.reducer.reduce()
        return loss.detach()

    def _capture(self, inp, tar, num_warmup_steps=3):
        """Capture forward + backward (+ optimiser) of the static-shape step into a CUDA graph."""
        self.static_inp = inp.clone()
        self.static_tar = tar.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(num_warmup_steps):
                self._forward_backward(self.static_inp, self.static_tar)
            if self.graph_mode == "step" and hasattr(self.optimizer, "prepare_tables"):
                self.optimizer.prepare_tables()      # pointer tables are uploaded before the capture starts
            side.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            n0 = _ext.launch_count()
            with torch.cuda.graph(self.graph, stream=side):
                self.static_loss = self._forward_backward(self.static_inp, self.static_tar)
                if self.graph_mode == "step":
                    # only the kernels go into the graph; step counters and hyper-parameters are uploaded per replay
                    if hasattr(self.optimizer, "launch_step"):
                        self.optimizer.launch_step()
                    else:
                        self.optimizer.step()
            # kernels of the extension inside the graph: counted per replay, not at capture time
            self._launches_per_replay = _ext.launch_count() - n0
            _ext.add_launches(-self._launches_per_replay)
        torch.cuda.current_stream(self.device).wait_stream(side)

    def _train_step(self, inp, tar):
        if self.graph_mode != "none":
            if self.graph is None:
                self._capture(inp, tar)
            self.static_inp.copy_(inp)
            self.static_tar.copy_(tar)
            if self.graph_mode == "step" and hasattr(self.optimizer, "prepare_step"):
                self.optimizer.prepare_step()
            self.graph.replay()
            _ext.add_launches(getattr(self, "_launches_per_replay", 0))
            loss = self.static_loss
            if self.graph_mode != "step":
                self.gscaler.step(self.optimizer)
                self.gscaler.update()
        else:
            loss = self._forward_backward(inp, tar)
            self.gscaler.step(self.optimizer)
            self.gscaler.update()
        return loss

    def _prepare_batch(self, data):
        gdata = [x.to(self.device, dtype=torch.float32, non_blocking=True) for x in data]
        inp, tar = self.preprocessor.cache_unpredicted_features(*gdata)
        return self.preprocessor.flatten_history(inp), self.preprocessor.flatten_history(tar)

    # ------------------------------------------------------------------------------------------ epochs
    def train(self):
        p = self.params
        if self.log_to_screen:
            self.logger.info("Starting Training Loop...")
        best_valid_loss = 1.0e6
        training_start = time.time()
        for epoch in range(self.startEpoch, p.max_epochs):
            if self.train_sampler is not None:
                self.train_sampler.set_epoch(epoch)
            if hasattr(self.train_dataloader, "set_epoch"):
                self.train_dataloader.set_epoch(epoch)
            self.epoch = epoch + 1          # epochs started so far: a checkpoint written below resumes at the next one
            t0 = time.time()
            train_time, train_data_gb, train_logs = self.train_one_epoch()
            valid_logs = {"base": {}, "metrics": {}}
            valid_time = 0.0
            viz_time = 0.0
            if not p.skip_validation:
                valid_time, viz_time, valid_logs = self.validate_one_epoch(epoch)
            if self.scheduler is not None:
                if isinstance(self.scheduler, torch.optim.lr_scheduler.ReduceLROnPlateau):
                    self.scheduler.step(valid_logs["base"]["validation loss"])
                else:
                    self.scheduler.step()
            if p.get("log_to_wandb", False) and self.world_rank == 0:
                self._log_wandb(train_logs, valid_logs)
            if p.save_checkpoint != "none" and p.get("checkpoint_path") is not None:
                save_needed = (self.data_parallel_rank == 0) or p.save_checkpoint == "flexible"
                if save_needed:
                    self.save_checkpoint(p.checkpoint_path, checkpoint_mode=p.save_checkpoint)
                    vl = valid_logs["base"].get("validation loss")
                    if vl is not None and vl <= best_valid_loss and p.get("best_checkpoint_path") is not None:
                        self.save_checkpoint(p.best_checkpoint_path, checkpoint_mode=p.save_checkpoint)
                        best_valid_loss = vl
            if dist.is_initialized():
                dist.barrier(device_ids=[self.device.index] if self.device.type == "cuda" else None)
            epoch_time = time.time() - t0
            self.log_epoch(train_logs, valid_logs, {"epoch time [s]": epoch_time, "training time [s]": train_time,
                                                    "validation time [s]": valid_time, "visualization time [s]": viz_time,
                                                    "training step time [ms]": train_logs["train_steps"] and (train_time / train_logs["train_steps"]) * 1e3,
                                                    "minimal IO rate [GB/s]": train_data_gb / max(train_time, 1e-9)})
        if self.log_to_screen:
            self.logger.info("Total training time is {:.2f} sec".format(time.time() - training_start))

    def train_one_epoch(self):
        self._set_train()
        p = self.params
        t0 = time.perf_counter()
        data_gb = 0.0
        steps = 0
        loss = torch.zeros((), device=self.device)
        accumulated = torch.zeros((2,), dtype=torch.float32, device=self.device)
        tstep = time.perf_counter_ns()
        wd = self._watchdog()
        for data in self.train_dataloader:
            self.iters += 1
            if wd is not None:
                # host-side liveness check before this step's collectives: a lost peer ends the epoch with an exception
                # (after an emergency checkpoint from the surviving ranks) instead of a hang inside NCCL
                wd.begin_step(self.iters)
                try:
                    wd.check()
                except Exception:
                    self._emergency_checkpoint()
                    raise
            inp, tar = self._prepare_batch(data)
            data_gb += (inp.numel() + tar.numel()) * 4 / 1e9
            loss = self._train_step(inp, tar)
            accumulated[0] += loss.float() * inp.shape[0]
            accumulated[1] += inp.shape[0]
            steps += 1
            freq = p.print_timings_frequency
            if freq > 0 and self.iters % freq == 0 and self.log_to_screen:
                if self.device.type == "cuda":
                    torch.cuda.synchronize()
                now = time.perf_counter_ns()
                self.logger.info(f"Iteration {self.iters}: average step time {(now - tstep) / freq * 1e-6:.2f} ms, loss {float(loss):.5f}")
                tstep = now
            if p.get("log_weights_and_grads", 0) > 0 and self.iters % p.log_weights_and_grads == 0:
                self.log_weights_and_grads(os.path.join(p.experiment_dir, "weights_and_grads"))
                if dist.is_initialized() and comm.get_size("data") > 1:
                    # only data rank 0 wrote files: re-align the ranks on the host so that the next step's in-kernel
                    # handshakes do not have to absorb the skew
                    dist.barrier(group=comm.get_group("data"))
            # the device error word (expired bounded waits) is read every `check_device_errors_every` steps; the fused
            # optimiser already skips its update while the word is set, so a late read loses no consistency
            every = int(p.get("check_device_errors_every", 50))
            if self.device.type == "cuda" and every > 0 and self.iters % every == 0:
                _ext.check_device_errors(self.device)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
            _ext.check_device_errors(self.device)
        if dist.is_initialized() and comm.get_size("data") > 1:
            dist.all_reduce(accumulated, group=comm.get_group("data"))
        acc = accumulated.cpu().numpy()
        train_time = time.perf_counter() - t0
        logs = {"loss": float(loss), "loss accumulated": float(acc[0] / max(acc[1], 1.0)), "train_steps": steps}
        return train_time, data_gb, logs

    def _watchdog(self):
        """Heartbeat watchdog (params: enable_watchdog, watchdog_timeout_s, step_deadline_s); None when disabled."""
        if not self.params.get("enable_watchdog", False):
            return None
        if getattr(self, "_wd", None) is None:
            from .watchdog import from_process_group
            self._wd = from_process_group(interval=1.0, timeout=float(self.params.get("watchdog_timeout_s", 120.0)),
                                          step_deadline=self.params.get("step_deadline_s", None))
        return self._wd

    def _emergency_checkpoint(self):
        """Local, collective-free save of this rank's state (legacy per-rank format) when a peer is lost."""
        try:
            path = os.path.join(self.params.experiment_dir, f"emergency_rank{comm.get_world_rank()}.tar")
            torch.save({"model_state": {k: v.detach().cpu() for k, v in self.model.state_dict().items()},
                        "iters": self.iters, "epoch": self.epoch}, path)
            if self.log_to_screen:
                self.logger.info(f"peer lost: emergency checkpoint written to {path}")
        except Exception as e:  # the job is going down anyway; do not mask the original failure
            self.logger.info(f"emergency checkpoint failed: {e}")

    @torch.no_grad()
    def validate_one_epoch(self, epoch):
        self._set_eval()
        p = self.params
        self.metrics.zero_buffers()
        t0 = time.time()
        viz_time = 0.0
        for eval_steps, data in enumerate(self.valid_dataloader):
            gdata = [x.to(self.device, dtype=torch.float32) for x in data]
            inp, tar = self.preprocessor.cache_unpredicted_features(*gdata)
            inp = self.preprocessor.flatten_history(inp)
            inpt = inp
            for idt, targ in enumerate(torch.split(tar, 1, dim=1)):
                targ = self.preprocessor.flatten_history(targ)
                with torch.autocast(device_type=self.device.type, dtype=self.amp_dtype, enabled=self.amp_enabled):
                    pred = self.model(inpt)
                    loss = self.loss_obj(pred, targ, inpt)
                self.metrics.update(pred, targ, loss, idt)
                if self.visualizer is not None and eval_steps == 0 and self.world_rank == 0 and comm.get_size("spatial") == 1:
                    tv = time.time()
                    self.visualizer.add(f"{epoch}_{idt}", pred[0].float().cpu().numpy(), targ[0].float().cpu().numpy())
                    viz_time += time.time() - tv
                inpt = self.preprocessor.append_history(inpt.to(pred.dtype), pred, idt)
        if self.device.type == "cuda":
            _ext.check_device_errors(self.device)    # validation uses the same bounded handshakes as training
        logs = self.metrics.finalize()
        if self.visualizer is not None and self.world_rank == 0:
            tv = time.time()
            self.visualizer.finalize()
            viz_time += time.time() - tv
        return time.time() - t0, viz_time, logs

    # ------------------------------------------------------------------------------------------ logging
    def log_epoch(self, train_logs, valid_logs, timing_logs):
        if not self.log_to_screen:
            return
        lr = self.optimizer.param_groups[0]["lr"]
        self.logger.info(f"Epoch {self.epoch} summary:")
        self.logger.info(f"Performance Parameters:")
        if self.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.device)
            self.logger.info(f"   gpu memory footprint [GB]: {(total - free) / 1024 ** 3:.2f}")
        for k, v in timing_logs.items():
            self.logger.info(f"   {k}: {v:.2f}" if isinstance(v, float) else f"   {k}: {v}")
        self.logger.info("Metrics:")
        self.logger.info(f"   learning rate: {lr}")
        for k, v in train_logs.items():
            self.logger.info(f"   training {k}: {v}")
        for k, v in valid_logs.get("base", {}).items():
            self.logger.info(f"   {k}: {v}")
        for k, v in valid_logs.get("metrics", {}).items():
            if k != "rollouts":
                self.logger.info(f"   {k}: {v}")

    def _log_wandb(self, train_logs, valid_logs):
        try:
            import wandb
            wandb.log({"learning rate": self.optimizer.param_groups[0]["lr"], **train_logs, **valid_logs.get("base", {}),
                       **{k: v for k, v in valid_logs.get("metrics", {}).items()}}, step=self.epoch)
        except Exception:
            pass

    def log_weights_and_grads(self, weights_and_grads_path, model=None, iters=None, epoch=None):
        """Dump every parameter and its gradient of this model rank to
        `<path>/weights_and_grads_epoch{epoch}_step{iters}_mp{rank}.tar` (file name of makani/utils/trainer.py:1175-1181);
        `model`, `iters`, `epoch` default to the trainer's own."""
        if self.data_parallel_rank != 0:
            return
        model = self.model if model is None else model
        iters = self.iters if iters is None else iters
        epoch = self.epoch if epoch is None else epoch
        os.makedirs(weights_and_grads_path, exist_ok=True)
        weights = {k: v.detach().cpu() for k, v in model.named_parameters()}
        grads = {k: v.grad.detach().cpu() for k, v in model.named_parameters() if v.grad is not None}
        fname = os.path.join(weights_and_grads_path, f"weights_and_grads_epoch{epoch}_step{iters}_mp{comm.get_rank('model')}.tar")
        torch.save({"step": iters, "epoch": epoch, "weights": weights, "grads": grads}, fname)

    # ------------------------------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, checkpoint_path, model=None, checkpoint_mode="flexible"):
        if self.log_to_screen:
            self.logger.info(f"Writing checkpoint to {checkpoint_path} ({checkpoint_mode} format)")
        ckpt.save_checkpoint(checkpoint_path, model or self.model, self.optimizer, self.scheduler, self.params, self.iters,
                             self.epoch, mode=checkpoint_mode, world_rank=self.world_rank, device=self.device)

    def restore_checkpoint(self, checkpoint_path, checkpoint_mode="flexible", load_optimizer=False, load_scheduler=False,
                           load_counters=False):
        if self.log_to_screen:
            self.logger.info(f"Loading checkpoint {checkpoint_path} in {checkpoint_mode} mode")
        iters, epoch = ckpt.restore_checkpoint(checkpoint_path, self.model, getattr(self, "optimizer", None),
                                               getattr(self, "scheduler", None), mode=checkpoint_mode,
                                               load_optimizer=load_optimizer, load_scheduler=load_scheduler,
                                               load_counters=load_counters, logger=self.logger)
        if load_counters and iters is not None:
            self.iters, self.startEpoch = iters, epoch

    # ------------------------------------------------------------------------------------------ self test
    @torch.no_grad()
    def test_autoregression_pipeline(self):
        """With the identity-like DebugNet: the rolled-out prediction must reproduce the input history, shifted."""
        self._set_eval()
        ok = True
        for data in self.valid_dataloader:
            gdata = [x.to(self.device, dtype=torch.float32) for x in data]
            inp, tar = self.preprocessor.cache_unpredicted_features(*gdata)
            inp = self.preprocessor.flatten_history(inp)
            inpt = inp
            for idt, targ in enumerate(torch.split(tar, 1, dim=1)):
                targ = self.preprocessor.flatten_history(targ)
                pred = self.model(inpt)
                nch = targ.shape[1]
                # DebugNet returns factor * input: the newest history slot of the input must come back
                expect = self.preprocessor.append_unpredicted_features(inpt)
                expect = self.preprocessor.add_static_features(expect)
                if not torch.allclose(pred, self.model.model.factor * expect, rtol=1e-5, atol=1e-6):
                    ok = False
                newest = pred[:, :nch] if self.params.n_history == 0 else pred[:, -expect.shape[1] // (self.params.n_history + 1):][:, :nch]
                inpt = self.preprocessor.append_history(inpt, targ, idt)
                # after appending, the newest slot must equal the value that was fed in
                tail = self.preprocessor.expand_history(inpt, self.params.n_history + 1)[:, -1]
                if not torch.allclose(tail, targ, rtol=1e-5, atol=1e-6):
                    ok = False
            break
        if self.log_to_screen:
            self.logger.info(f"autoregression pipeline test {'passed' if ok else 'FAILED'}")
        return ok
