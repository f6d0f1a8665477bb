"""Assembly of the flagship benchmark workload (SFNO-73ch, 721x1440) from the framework's public pieces."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.networks.sfnonet import SphericalFourierNeuralOperatorNet
from ..ops import _ext
from ..ops.optim import FusedAdamW
from ..parallel.grad_reduce import GradReducer
from ..parallel.helpers import sync_params
from ..utils import comm
from .losses import LossHandler
from .train_step import GraphedTrainStep, TrainStep
from .YParams import ParamsBase


@dataclass
class FlagshipConfig:
    small: bool = False
    name: str = "sfno_linear_73chq_sc3_layers8_edim384"
    nlat: int = 721
    nlon: int = 1440
    in_chans: int = 74      # 73 prognostic + 1 static cos(latitude)
    out_chans: int = 73
    embed_dim: int = 384
    num_layers: int = 8
    scale_factor: int = 3
    batch_per_gpu: int = 1
    loss: str = "absolute squared geometric l2"
    lr: float = 1e-3
    h: int = 1              # latitude-parallel ranks
    w: int = 1              # longitude-parallel ranks
    graph: bool = True      # replay the whole step from one CUDA graph after an eager warm-up
    native: bool = True     # False: the reference's op sequence on stock PyTorch (cuDNN / cuFFT / cuBLAS / ATen / NCCL)
    model: str = "sfno"     # "sfno" (headline) or "afno" (FourCastNet v1: 720x1440x20, patch 8, embed 768, 12 layers, 8 blocks)

    def __post_init__(self):
        if self.model == "afno":
            self.name = "afno_20ch_p8_e768_l12_b8"
            self.nlat, self.nlon, self.in_chans, self.out_chans = 720, 1440, 20, 20
            self.loss = "l2"
        if self.small:
            self.name += "_small"
            self.nlat, self.nlon = 361, 720


class FlagshipRunner:
    def __init__(self, cfg: FlagshipConfig, device: torch.device):
        self.cfg, self.device = cfg, device
        from ..parallel.helpers import compute_split_shapes
        lat_shapes = compute_split_shapes(cfg.nlat, comm.get_size("h"))
        lon_shapes = compute_split_shapes(cfg.nlon, comm.get_size("w"))
        rh, rw = comm.get_rank("h"), comm.get_rank("w")
        self.lat0, self.lon0 = sum(lat_shapes[:rh]), sum(lon_shapes[:rw])
        self.hl, self.wl = lat_shapes[rh], lon_shapes[rw]
        torch.manual_seed(0)
        if cfg.model == "afno":
            from ..models.networks.afnonet import AdaptiveFourierNeuralOperatorNet
            self.model = AdaptiveFourierNeuralOperatorNet(
                inp_shape=(cfg.nlat, cfg.nlon), patch_size=(8, 8), inp_chans=cfg.in_chans, out_chans=cfg.out_chans, embed_dim=768,
                num_layers=12, mlp_ratio=4.0, num_blocks=8, sparsity_threshold=0.01, hard_thresholding_fraction=1.0).to(device)
        else:
            self.model = self._build_sfno(cfg, device)
        self._finish_init(cfg, device)

    @staticmethod
    def _build_sfno(cfg, device):
        return SphericalFourierNeuralOperatorNet(
            spectral_transform="sht", model_grid_type="equiangular", sht_grid_type="legendre-gauss", filter_type="linear",
            operator_type="dhconv", inp_shape=(cfg.nlat, cfg.nlon), out_shape=(cfg.nlat, cfg.nlon),
            scale_factor=cfg.scale_factor, inp_chans=cfg.in_chans, out_chans=cfg.out_chans, embed_dim=cfg.embed_dim,
            num_layers=cfg.num_layers, use_mlp=True, mlp_ratio=2.0, activation_function="gelu", encoder_layers=1,
            pos_embed="none", normalization_layer="instance_norm", hard_thresholding_fraction=1.0, big_skip=True).to(device)

    def _finish_init(self, cfg, device):
        if cfg.native:
            self.model.set_compute_dtype(torch.bfloat16)
        sync_params(self.model)
        p = ParamsBase()
        p.update_params(dict(loss=cfg.loss, n_future=0, img_shape_x=cfg.nlat, img_shape_y=cfg.nlon,
                             img_crop_shape_x=cfg.nlat, img_crop_shape_y=cfg.nlon, img_crop_offset_x=0, img_crop_offset_y=0,
                             N_out_channels=cfg.out_chans, channel_weights="auto", model_grid_type="equiangular",
                             img_local_shape_x=self.hl, img_local_shape_y=self.wl, img_local_offset_x=self.lat0,
                             img_local_offset_y=self.lon0))
        self.loss_fn = LossHandler(p).to(device)
        if cfg.native:
            self.reducer = GradReducer(self.model)
            self.optimizer = FusedAdamW(self.model.parameters(), lr=cfg.lr, weight_decay=0.0)
            step_cls = GraphedTrainStep if cfg.graph else TrainStep
            self.train_step = step_cls(self.model, self.loss_fn, self.optimizer, self.reducer)
        else:
            # what the reference runs: fp32 parameters and transforms, bf16 autocast for the convolutions, foreach
            # AdamW, NCCL all-reduce of the gradients (makani/utils/trainer.py:429-433,683-754)
            self.reducer = GradReducer(self.model, use_peer=False, overlap=False)
            self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=cfg.lr, weight_decay=0.0, foreach=True)
            self.train_step = TrainStep(self.model, self.loss_fn, self.optimizer, self.reducer, amp_dtype=torch.bfloat16)
        self.io_dtype = torch.bfloat16 if cfg.native else torch.float32
        lat = torch.linspace(math.pi / 2, -math.pi / 2, cfg.nlat, device=device)[self.lat0: self.lat0 + self.hl]
        self.coslat = torch.cos(lat).view(1, 1, -1, 1).expand(cfg.batch_per_gpu, 1, self.hl, self.wl)

    def synthetic_batch(self, seed: int):
        cfg = self.cfg
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        x = torch.randn(cfg.batch_per_gpu, cfg.out_chans, self.hl, self.wl, device=self.device, generator=g)
        if cfg.in_chans == cfg.out_chans:
            inp = x.to(self.io_dtype).contiguous()
        else:
            inp = torch.cat([x, self.coslat], dim=1).to(self.io_dtype).contiguous()
        tgt = torch.randn(cfg.batch_per_gpu, cfg.out_chans, self.hl, self.wl, device=self.device, generator=g).to(self.io_dtype)
        return inp, tgt

    def step(self, inp, tgt):
        return self.train_step(inp, tgt)

    def end_to_end(self, steps: int, warmup: int, world: int, local_rank: int):
        """Same step, but every step's input/target come from pinned host memory (double-buffered H2D copy on a
        side stream) and every step's loss is read back to the host."""
        cfg = self.cfg
        dev = self.device
        nb = 2
        host = []
        for i in range(nb):
            gi = torch.Generator().manual_seed(100 + i + 17 * local_rank)
            hi = torch.randn(cfg.batch_per_gpu, cfg.in_chans, self.hl, self.wl, generator=gi).to(self.io_dtype).pin_memory()
            ht = torch.randn(cfg.batch_per_gpu, cfg.out_chans, self.hl, self.wl, generator=gi).to(self.io_dtype).pin_memory()
            host.append((hi, ht))
        dbuf = [(torch.empty_like(h[0], device=dev), torch.empty_like(h[1], device=dev)) for h in host]
        copy_stream = torch.cuda.Stream(device=dev)
        ready = [torch.cuda.Event() for _ in range(nb)]
        consumed = [torch.cuda.Event() for _ in range(nb)]
        h2d = host[0][0].numel() * host[0][0].element_size() + host[0][1].numel() * host[0][1].element_size()
        loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

        def issue(i):
            b = i % nb
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[b])
                dbuf[b][0].copy_(host[b][0], non_blocking=True)
                dbuf[b][1].copy_(host[b][1], non_blocking=True)
                ready[b].record(copy_stream)

        def run(n, timed):
            cur = torch.cuda.current_stream(dev)
            for b in range(nb):
                consumed[b].record(cur)
            issue(0)
            for i in range(n):
                b = i % nb
                if i + 1 < n:
                    issue(i + 1)
                cur.wait_event(ready[b])
                loss = self.train_step(dbuf[b][0], dbuf[b][1])
                consumed[b].record(cur)
                loss_host.copy_(loss.reshape(1).float(), non_blocking=False)  # D2H read of the step result
            return float(loss_host.item())

        run(warmup, False)
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run(steps, True)
        e1.record()
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item() / steps
        dp = max(1, world // comm.get_size("model"))
        return {"value": cfg.batch_per_gpu * dp / (ms / 1e3), "unit": "samples/s", "ms_per_step": ms,
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4}


    @torch.no_grad()
    def rollout(self, steps: int, warmup: int, world: int, local_rank: int, graph: bool = True):
        """Autoregressive inference: state <- [model(state), static channel]; one step is captured in a CUDA graph (as
        `Inferencer.rollout` does) and replayed.  Returns milliseconds per step (device-timed, max over ranks)."""
        self.model.eval()
        dev = self.device
        state, _ = self.synthetic_batch(seed=99)
        static = state.clone()

        def one_step():
            pred = self.model(static)
            static[:, : pred.shape[1]].copy_(pred)        # prognostic channels advance; the static channel stays

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        g = None
        with torch.cuda.stream(side):
            for _ in range(max(2, warmup)):
                one_step()
            side.synchronize()
            if graph:
                g = torch.cuda.CUDAGraph()
                n0 = _ext.launch_count()
                with torch.cuda.graph(g, stream=side):
                    one_step()
                per_replay = _ext.launch_count() - n0
                _ext.add_launches(-per_replay)
        torch.cuda.current_stream(dev).wait_stream(side)
        static.copy_(state)
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()
        l0 = _ext.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            if g is not None:
                g.replay()
                _ext.add_launches(per_replay)
            else:
                one_step()
        e1.record()
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        self._rollout_graph = g
        finite = bool(torch.isfinite(static.float()).all())
        return t.item() / steps, _ext.launch_count() - l0, finite


def build_flagship(cfg: FlagshipConfig, device: torch.device) -> FlagshipRunner:
    return FlagshipRunner(cfg, device)
