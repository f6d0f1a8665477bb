"""Gradient reduction for data parallelism and for parameters replicated across model-parallel groups.

Semantics (reference: makani/mpu/mappings.py:30-174): gradients are averaged over the `data` group and then
summed over every group named in `param.is_shared_mp` (default ["model"]).  Complex gradients are reduced
through their real view.

Mechanism here: all gradients live as views into one flat fp32 buffer.  On a single NVSwitch node with NCCL
the buffer is symmetric peer memory and the data-parallel average is the in-kernel P2P all-reduce of
`csrc/peer.cu`, which fuses the 1/N scaling; otherwise (CPU/gloo, or more ranks than one node) it is an
all_reduce of the flat buffer.  Keeping `.grad` as persistent views also lets the fused AdamW run from a
fixed pointer table.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils import comm


class GradReducer:
    def __init__(self, model: torch.nn.Module, use_peer: Optional[bool] = None, align: int = 64,
                 bucket_mb: Optional[float] = None, overlap: bool = True):
        if bucket_mb is None:
            bucket_mb = float(os.environ.get("MAKANI_B200_BUCKET_MB", "256"))
        self.params = [p for p in model.parameters() if p.requires_grad]
        dev = self.params[0].device
        self.device = dev
        sizes = []
        total = 0
        for p in self.params:
            n = p.numel() * (2 if p.is_complex() else 1)
            sizes.append((total, n))
            total += (n + align - 1) // align * align
        self.total = total
        self.data_size = comm.get_size("data")
        # groups (other than `data`) over which some parameter's gradient has to be summed
        shared_names: List[str] = []
        for p in self.params:
            for g in getattr(p, "is_shared_mp", ["model"]):
                if comm.get_size(g) > 1 and g not in shared_names:
                    shared_names.append(g)
        self._shared_names = shared_names
        if use_peer is None:
            use_peer = (dev.type == "cuda" and dist.is_initialized() and dist.get_world_size() <= 8
                        and (self.data_size > 1 or len(shared_names) > 0) and dist.get_backend() == "nccl")
        # diagnosis only: MAKANI_B200_DP_DIAG=noreduce leaves the data-parallel average out (replicas diverge), to tell
        # the cost of the reduction apart from what running N ranks side by side costs by itself
        self.diag_noreduce = "noreduce" in os.environ.get("MAKANI_B200_DP_DIAG", "").split(",")
        # MAKANI_B200_DP_DIAG=timeline (eager steps only): CUDA events around every bucket's reduction and around the final
        # join; `timeline_report()` returns when each bucket became ready, how long its reduction took and how long the
        # compute stream waited at the end of backward
        self.diag_timeline = "timeline" in os.environ.get("MAKANI_B200_DP_DIAG", "").split(",")
        # MAKANI_B200_DP_DIAG=noar: everything as in a real run (symmetric buffer, buckets, side stream) except that the
        # all-reduce kernels are not launched
        self.diag_noar = "noar" in os.environ.get("MAKANI_B200_DP_DIAG", "").split(",")
        self._timeline = []
        self._t_zero = None
        self._t_join = None
        if self.diag_noreduce:
            use_peer = False
        self.sym = None
        if use_peer:
            from .peer import SymmetricBuffer
            # one buffer mapped by every rank of the node; the data-parallel average and each model-parallel sum run over
            # their own sub-group of it with their own set of barrier flags
            self.sym = SymmetricBuffer(total * 4, group=None, device=dev, flag_sets=1 + len(shared_names))
            self._data_members = comm.get_group_ranks("data")
            self._shared_members = {g: comm.get_group_ranks(g) for g in shared_names}
            self.flat = self.sym.view(torch.float32, total)
            self.flat.zero_()
        else:
            self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        for p, (off, n) in zip(self.params, sizes):
            if p.is_complex():
                g = torch.view_as_complex(self.flat[off: off + n].view(*p.shape, 2))
            else:
                g = self.flat[off: off + n].view(p.shape)
            p.grad = g
        # ---- buckets for overlapping the data-parallel reduction with the backward pass ----------------------
        # Parameters are bucketed in reverse registration order (the order in which backward produces gradients);
        # a bucket is a contiguous range of the flat buffer.  When the last gradient of a bucket has been
        # accumulated, its all-reduce is queued on a side stream behind an event of the compute stream.
        self.overlap = bool(overlap and self.sym is not None and self.data_size > 1)
        self.buckets: List[List[int]] = []        # [start, end) element ranges of the flat buffer
        self._bucket_of: Dict[int, int] = {}
        self._pending: List[int] = []
        if self.overlap:
            limit = int(bucket_mb * 1024 * 1024 / 4)
            end = total
            cur_start = total
            members: List[int] = []
            for idx in range(len(self.params) - 1, -1, -1):
                off, n = sizes[idx]
                cur_start = off
                members.append(idx)
                if end - cur_start >= limit or idx == 0:
                    b = len(self.buckets)
                    self.buckets.append([cur_start, end])
                    for m in members:
                        self._bucket_of[m] = b
                    members = []
                    end = cur_start
            self._pending = [0] * len(self.buckets)
            self._counts = [0] * len(self.buckets)
            for idx in range(len(self.params)):
                self._counts[self._bucket_of[idx]] += 1
            self._side = torch.cuda.Stream(device=dev)
            self._launched = [False] * len(self.buckets)
            for idx, p in enumerate(self.params):
                p.register_post_accumulate_grad_hook(self._make_hook(idx))
            self._reset_pending()
        # parameters whose gradient must additionally be summed over model-parallel groups
        # (kept as merged [start, end) ranges of the flat buffer, reduced in place: no staging copies)
        self.shared: Dict[str, List[List[int]]] = {}
        for p, (off, n) in zip(self.params, sizes):
            for g in getattr(p, "is_shared_mp", ["model"]):
                if comm.get_size(g) > 1:
                    ranges = self.shared.setdefault(g, [])
                    end = off + (n + align - 1) // align * align
                    if ranges and ranges[-1][1] == off:
                        ranges[-1][1] = end
                    else:
                        ranges.append([off, end])

    def _reset_pending(self):
        self._pending = list(self._counts)
        self._launched = [False] * len(self.buckets)

    def _make_hook(self, idx):
        def hook(param):
            b = self._bucket_of[idx]
            self._pending[b] -= 1
            if self._pending[b] == 0 and not self._launched[b]:
                self._launch_bucket(b)
        return hook

    def _launch_bucket(self, b):
        start, end = self.buckets[b]
        self._launched[b] = True
        timeline = self.diag_timeline and not torch.cuda.is_current_stream_capturing()
        ev = torch.cuda.Event(enable_timing=timeline)
        ev.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._side):
            self._side.wait_event(ev)
            if not self.diag_noar:
                self.sym.all_reduce_(end - start, torch.float32, scale=1.0 / self.data_size, byte_offset=start * 4,
                                     members=self._data_members, flag_set=0)
            if timeline:
                done = torch.cuda.Event(enable_timing=True)
                done.record(self._side)
                self._timeline.append((b, (end - start) * 4, ev, done))

    def zero_grad(self):
        if self.overlap:
            # the previous step's side-stream work must be finished before the buffer is cleared (`reduce` has joined
            # it already; under stream capture a wait on the not yet captured side stream is not allowed)
            if not torch.cuda.is_current_stream_capturing():
                torch.cuda.current_stream(self.device).wait_stream(self._side)
            self._reset_pending()
        if self.diag_timeline and not torch.cuda.is_current_stream_capturing():
            self._timeline = []
            self._t_zero = torch.cuda.Event(enable_timing=True)
            self._t_zero.record(torch.cuda.current_stream(self.device))
        self.flat.zero_()

    def reduce(self):
        """Average over `data`, then sum over the model-parallel groups each parameter is shared on."""
        if self.data_size > 1 and not self.diag_noreduce:
            if self.overlap:
                for b in range(len(self.buckets)):     # buckets whose hooks did not all fire (unused parameters)
                    if not self._launched[b]:
                        self._launch_bucket(b)
                timeline = self.diag_timeline and not torch.cuda.is_current_stream_capturing()
                if timeline:
                    e0 = torch.cuda.Event(enable_timing=True)
                    e0.record(torch.cuda.current_stream(self.device))
                torch.cuda.current_stream(self.device).wait_stream(self._side)
                if timeline:
                    e1 = torch.cuda.Event(enable_timing=True)
                    e1.record(torch.cuda.current_stream(self.device))
                    self._t_join = (e0, e1)
            elif self.sym is not None:
                self.sym.all_reduce_(self.total, torch.float32, scale=1.0 / self.data_size, members=self._data_members, flag_set=0)
            else:
                dist.all_reduce(self.flat, group=comm.get_group("data"))
                self.flat.mul_(1.0 / self.data_size)
        for gname, ranges in self.shared.items():
            if self.sym is not None:
                # in-kernel peer sum over the ranks that share these parameters (no NCCL call on the step)
                fs = 1 + self._shared_names.index(gname)
                for start, end in ranges:
                    self.sym.all_reduce_(end - start, torch.float32, scale=1.0, byte_offset=start * 4,
                                         members=self._shared_members[gname], flag_set=fs)
            else:
                grp = comm.get_group(gname)
                for start, end in ranges:
                    dist.all_reduce(self.flat[start:end], group=grp)

    def timeline_report(self):
        """Of the last eager step (MAKANI_B200_DP_DIAG=timeline): per bucket (index, MB, ms after the start of the step at
        which it became ready, ms at which its reduction had finished) and the ms the compute stream waited at the join."""
        if not (self.diag_timeline and self._t_zero is not None and self._t_join is not None):
            return None
        torch.cuda.synchronize(self.device)
        rows = [(b, nbytes / 1e6, self._t_zero.elapsed_time(ev), self._t_zero.elapsed_time(done)) for b, nbytes, ev, done in self._timeline]
        e0, e1 = self._t_join
        return {"buckets": rows, "backward_end_ms": self._t_zero.elapsed_time(e0), "join_wait_ms": e0.elapsed_time(e1)}

    def close(self):
        if self.sym is not None:
            for p in self.params:
                p.grad = None
            self.flat = None
            self.sym.close()
            self.sym = None
