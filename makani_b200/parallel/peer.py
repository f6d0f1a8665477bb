"""Symmetric peer memory for the GPUs of one NVSwitch node.

Every rank of a process group allocates the same-sized buffer with `cudaMalloc`, exports a CUDA IPC handle,
exchanges the handles through `torch.distributed` and maps all peers' buffers.  Kernels then receive the raw
peer pointers and move data with plain loads/stores over NVLink (no NCCL call on the hot path, no TMA
multicast).  The reference has no counterpart: all its communication goes through NCCL process groups
(makani/utils/comm.py:97-133).
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext

FLAG_BYTES = 128 * 9 * 4  # PEER_MAX_BLOCKS * (PEER_MAX + 1) * sizeof(uint32), see csrc/peer.cuh


class SymmetricBuffer:
    """`nbytes` of device memory on every rank of `group`, mapped into every other rank."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        assert dist.is_initialized(), "SymmetricBuffer needs an initialised process group"
        self.ext = _ext.require()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= 8, "peer collectives support up to 8 ranks (one NVSwitch node)"
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        with torch.cuda.device(self.device):
            out: list = []
            handle = self.ext.peer_alloc(self.nbytes + FLAG_BYTES, out)
            self.local_ptr = out[0]
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            self.ptrs = []
            for r, h in enumerate(handles):
                self.ptrs.append(self.local_ptr if r == self.rank else self.ext.peer_open(h))
        self.flag_ptrs = [p + self.nbytes for p in self.ptrs]
        self.local = self.ext.tensor_from_ptr(self.local_ptr, self.nbytes, self.device.index)
        dist.barrier(group=group)
        self._closed = False

    def view(self, dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        return self.local[byte_offset: byte_offset + numel * esz].view(dtype)

    def all_reduce_(self, numel: int, dtype=torch.float32, scale: float = 1.0, byte_offset: int = 0) -> None:
        """In-place sum (times `scale`) over the group of `numel` elements starting at `byte_offset`."""
        assert dtype in (torch.float32, torch.bfloat16)
        ptrs = [p + byte_offset for p in self.ptrs]
        self.ext.peer_allreduce(ptrs, self.flag_ptrs, self.rank, int(numel), 1 if dtype == torch.bfloat16 else 0,
                                float(scale), 0, self.device.index)

    def close(self):
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        try:
            dist.barrier(group=self.group)
        except Exception:
            pass
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.ext.peer_close(p)
        self.ext.peer_free(self.local_ptr)
