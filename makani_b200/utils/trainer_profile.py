"""Trainer with a profiler capture window: NVTX ranges around epochs and steps, and `cudaProfilerStart/Stop`
(through `torch.cuda.profiler`) around a chosen range of training or validation steps on chosen ranks, each
toggle bracketed by a barrier so the windows of all ranks line up.

Flag semantics: makani/train_profile.py (`--capture_mode`, `--capture_range_start/stop`, `--capture_ranks`) and
makani/utils/trainer_profile.py:54-72,301-305,659-710.  Unlike the reference, which keeps a second copy of the
whole trainer, this class only overrides the step wrappers.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import comm
from .trainer import Trainer


class _Window:
    def __init__(self, enabled, start, stop, ranks, world_rank, device):
        self.enabled = enabled and (not ranks or world_rank in ranks)
        self.start, self.stop, self.device = start, stop, device
        self.active = False

    def _sync(self):
        if dist.is_initialized():
            dist.barrier(device_ids=[self.device.index] if self.device.type == "cuda" else None)
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def before(self, step):
        if step == self.start:
            self._sync()
            if self.enabled and self.device.type == "cuda":
                torch.cuda.profiler.start()
                self.active = True

    def after(self, step):
        if step == self.stop:
            self._sync()
            if self.active:
                torch.cuda.profiler.stop()
                self.active = False


def _nvtx_push(name, device):
    if device.type == "cuda":
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop(device):
    if device.type == "cuda":
        torch.cuda.nvtx.range_pop()


class ProfilingTrainer(Trainer):
    def __init__(self, params, world_rank, job_type="train"):
        super().__init__(params, world_rank, job_type)
        g = params.get
        mode = g("capture_mode", [])
        mode = mode if isinstance(mode, (list, tuple)) else [mode]
        ranks = g("capture_ranks", []) or []
        self._train_window = _Window("training" in mode, g("capture_range_start", 0), g("capture_range_stop", 50), ranks,
                                     world_rank, self.device)
        self._valid_window = _Window("validation" in mode, g("capture_range_start", 0), g("capture_range_stop", 50), ranks,
                                     world_rank, self.device)
        self._train_steps = 0

    def _train_step(self, inp, tar):
        step = self._train_steps
        self._train_window.before(step)
        _nvtx_push(f"train step {step}", self.device)
        loss = super()._train_step(inp, tar)
        _nvtx_pop(self.device)
        self._train_window.after(step)
        self._train_steps += 1
        return loss

    def train_one_epoch(self):
        _nvtx_push("training", self.device)
        out = super().train_one_epoch()
        _nvtx_pop(self.device)
        return out

    def validate_one_epoch(self, epoch):
        self._valid_window.before(self._valid_window.start)
        _nvtx_push("validation", self.device)
        out = super().validate_one_epoch(epoch)
        _nvtx_pop(self.device)
        self._valid_window.after(self._valid_window.stop)
        return out


Trainer = ProfilingTrainer
