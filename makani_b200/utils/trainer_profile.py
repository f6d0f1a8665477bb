"""Trainer with a profiler capture window: NVTX ranges around epochs and steps, and `cudaProfilerStart/Stop`
(through `torch.cuda.profiler`) around a chosen range of training or validation steps on chosen ranks, each
toggle bracketed by a barrier so the windows of all ranks line up.

Flag semantics: makani/train_profile.py (`--capture_mode`, `--capture_range_start/stop`, `--capture_ranks`) and
makani/utils/trainer_profile.py:54-72,301-305,659-710.  Unlike the reference, which keeps a second copy of the
whole trainer, this class wraps the step, the two data loaders (NVTX range per fetch; the validation window counts
validation steps) and the visualiser.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import comm
from .trainer import Trainer


def cudaProfilerStart(device=None, enabled=True):
    """Names and calling convention of makani/utils/trainer_profile.py:59-74 (there through ctypes): a barrier so that
    the windows of all ranks line up, then the profiler toggle on the ranks where `enabled`."""
    if dist.is_initialized():
        dist.barrier(device_ids=[device.index] if device is not None and device.type == "cuda" else None)
    if enabled and torch.cuda.is_available():
        torch.cuda.profiler.start()


def cudaProfilerStop(device=None, enabled=True):
    if enabled and torch.cuda.is_available():
        torch.cuda.profiler.stop()
    if dist.is_initialized():
        dist.barrier(device_ids=[device.index] if device is not None and device.type == "cuda" else None)


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


class _InstrumentedLoader:
    """Iterates a data loader with an NVTX range around every fetch ("data loading") and, when a capture window is
    given, opens / closes the window around the loop body of the chosen steps: `before(i)` runs right before batch i is
    handed out, `after(i)` when the body of step i has finished (i.e. when the next batch is asked for)."""

    def __init__(self, loader, device, window=None, label="data loading"):
        self.loader, self.device, self.window, self.label = loader, device, window, label

    def __len__(self):
        return len(self.loader)

    def __getattr__(self, name):
        return getattr(self.loader, name)

    def __iter__(self):
        it = iter(self.loader)
        step = 0
        while True:
            if self.window is not None and step > 0:
                self.window.after(step - 1)
            _nvtx_push(self.label, self.device)
            try:
                batch = next(it)
            except StopIteration:
                _nvtx_pop(self.device)
                return
            _nvtx_pop(self.device)
            if self.window is not None:
                self.window.before(step)
            yield batch
            step += 1


class _InstrumentedVisualizer:
    """NVTX ranges around the visualiser calls (they run on the host between validation steps)."""

    def __init__(self, viz, device):
        self._viz, self._device = viz, device

    def __getattr__(self, name):
        attr = getattr(self._viz, name)
        if not callable(attr):
            return attr

        def wrapped(*args, **kwargs):
            _nvtx_push(f"visualization {name}", self._device)
            try:
                return attr(*args, **kwargs)
            finally:
                _nvtx_pop(self._device)

        return wrapped


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
        if self.visualizer is not None:
            self.visualizer = _InstrumentedVisualizer(self.visualizer, self.device)

    def test_model_output(self, model):
        """Checkpoint self-test (makani/utils/trainer_profile.py:842-866): the first call stores a random input and the
        model's output for it in the experiment directory; later calls (e.g. after a restore) log how far the output
        for the same input has moved."""
        import os

        import numpy as np

        p = self.params
        hl = p.get("img_local_shape_x", p.img_shape_x)
        wl = p.get("img_local_shape_y", p.img_shape_y)
        cin = p.N_in_channels
        if p.get("split_data_channels", False):
            cin = (cin + comm.get_size("matmul") - 1) // comm.get_size("matmul")
        mrank = comm.get_rank("model")
        f_in = os.path.join(p.experiment_dir, f"random_tensor{mrank}.npy")
        f_out = os.path.join(p.experiment_dir, f"random_output{mrank}.npy")
        if not os.path.exists(f_in):
            np.save(f_in, torch.rand(p.batch_size, cin, hl, wl).numpy())
        x = torch.from_numpy(np.load(f_in)).float().to(self.device)
        with torch.no_grad():
            out = model(x).detach().float().cpu().numpy()
        if os.path.exists(f_out):
            diff = (out - np.load(f_out)).ravel()
            self.logger.info(f"Diff metrics: norm = {np.linalg.norm(diff)}, max = {diff.max()}, min = {diff.min()}")
        np.save(f_out, out)

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
        loader = self.train_dataloader
        self.train_dataloader = _InstrumentedLoader(loader, self.device)
        try:
            out = super().train_one_epoch()
        finally:
            self.train_dataloader = loader
            _nvtx_pop(self.device)
        return out

    def validate_one_epoch(self, epoch):
        # the capture window counts validation steps (batches of the validation loader), as for training
        _nvtx_push("validation", self.device)
        loader = self.valid_dataloader
        self.valid_dataloader = _InstrumentedLoader(loader, self.device, window=self._valid_window)
        try:
            out = super().validate_one_epoch(epoch)
        finally:
            self.valid_dataloader = loader
            if self._valid_window.active:       # the loader ended inside the window
                self._valid_window.after(self._valid_window.stop)
            _nvtx_pop(self.device)
        return out


Trainer = ProfilingTrainer
