"""Data-loader factory (contract: makani/utils/dataloader.py:27-151).

`get_dataloader(params, files_pattern, device, train, final_eval)` returns `(loader, dataset, sampler)` for
training and `(loader, dataset)` otherwise.  `dataset` exposes the channel lists, the grid converter and the
global / cropped / local image geometry; the loader exposes `get_input_normalization()` and
`get_output_normalization()`.  Sources: the seeded synthetic generator (`enable_synthetic_data`) or yearly
`[T, C, H, W]` files (`multifiles`, the default for real data here; the reference's DALI pipeline is not
reproduced — the synthetic generator and a pinned-memory prefetcher take its place).
"""

from __future__ import annotations

import math
import types

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from . import comm


def init_distributed_io(params):
    if dist.is_initialized():
        params.data_num_shards = comm.get_size("data")
        params.data_shard_id = comm.get_rank("data")
        params.io_grid = [1, comm.get_size("h"), comm.get_size("w")]
        params.io_rank = [0, comm.get_rank("h"), comm.get_rank("w")]
    else:
        params.data_num_shards = 1
        params.data_shard_id = 0
        if params.get("io_grid") is None:
            params.io_grid = [1, 1, 1]
        if params.get("io_rank") is None:
            params.io_rank = [0, 0, 0]


def _geometry(obj):
    names = ["in_channels", "out_channels", "grid_converter", "img_shape_x", "img_shape_y", "img_crop_shape_x",
             "img_crop_shape_y", "img_crop_offset_x", "img_crop_offset_y", "img_local_shape_x", "img_local_shape_y",
             "img_local_offset_x", "img_local_offset_y"]
    return types.SimpleNamespace(**{n: getattr(obj, n) for n in names})


class PrefetchLoader:
    """Wraps a host-side loader: batches are staged in pinned memory and copied to the device on a side stream
    one batch ahead of the consumer (the role DALI's GPU prefetch queue plays in the reference)."""

    def __init__(self, loader, device):
        self.loader, self.device = loader, torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None

    def __len__(self):
        return len(self.loader)

    def __getattr__(self, name):
        return getattr(self.loader, name)

    def _stage(self, batch):
        if self.stream is None:
            return tuple(t.to(self.device) for t in batch)
        with torch.cuda.stream(self.stream):
            out = tuple((t if t.is_pinned() else t.pin_memory()).to(self.device, non_blocking=True) for t in batch)
        return out

    def __iter__(self):
        it = iter(self.loader)
        try:
            nxt = self._stage(next(it))
        except StopIteration:
            return
        for batch in it:
            cur = nxt
            if self.stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.stream)
            nxt = self._stage(batch)
            yield cur
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        yield nxt


def get_dataloader(params, files_pattern, device, train=True, final_eval=False):
    init_distributed_io(params)
    sampler = None
    if params.get("enable_synthetic_data", False):
        from .dataloaders.data_loader_synthetic import SyntheticLoader
        dataloader = SyntheticLoader(params, files_pattern, train, device)
        dataset = _geometry(dataloader)
    else:
        from torch.utils.data.distributed import DistributedSampler

        from .dataloaders.data_loader_multifiles import MultifilesDataset
        dataset = MultifilesDataset(params, files_pattern, train)
        if params.data_num_shards > 1:
            sampler = DistributedSampler(dataset, shuffle=train, num_replicas=params.data_num_shards, rank=params.data_shard_id)
        loader = DataLoader(dataset, batch_size=int(params.batch_size), num_workers=params.get("num_data_workers", 0),
                            shuffle=(sampler is None) and train, sampler=sampler, drop_last=True,
                            pin_memory=torch.cuda.is_available())
        dataloader = PrefetchLoader(loader, device) if torch.device(device).type == "cuda" else loader
        dataloader.get_output_normalization = dataset.get_output_normalization
        dataloader.get_input_normalization = dataset.get_input_normalization
    if train:
        return dataloader, dataset, sampler
    return dataloader, dataset
