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


# ---------------------------------------------------------------------------------------------- handshake slots
#
# A slot is a symmetric buffer that one kernel on every rank of a group writes (its own copy) and a later kernel
# on every rank reads (all copies, through peer pointers), again and again.  Ordering between ranks is kept by
# monotonic counters in device memory, so no host synchronisation and no NCCL call is involved and the whole
# sequence can be captured in a CUDA graph:
#
#   ready[p]  (on every rank)  incremented by rank p when its copy of generation g is complete
#   free[p]   (on every rank)  incremented by rank p when it has finished reading generation g everywhere
#   n_prod, n_read (local)     generations produced / consumed so far by this rank
#
# A producer waits for free[p] >= n_prod for all p, a consumer for ready[p] >= n_read + 1; both waits are bounded
# in the kernels (a device error code is raised instead of a hang).

CTRL_BYTES = 256
_READY, _FREE, _NPROD, _NREAD, _DONE = 0, 32, 64, 68, 72   # byte offsets inside the control block


class PeerSlot:
    """Symmetric buffer plus handshake counters over one named communicator group (CUDA, one node)."""

    is_peer = True

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.buf = SymmetricBuffer(CTRL_BYTES + nbytes, group=group, device=device)
        self.world, self.rank, self.device = self.buf.world, self.buf.rank, self.buf.device
        self.capacity = self.buf.nbytes - CTRL_BYTES
        self._hold = None

    # data ------------------------------------------------------------------------------------------
    def tensor(self, dtype, shape) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        return self.buf.view(dtype, n, CTRL_BYTES).view(*shape)

    def sources(self):
        """Device addresses of every rank's copy (to be read by this rank's kernels only, never by library code)."""
        return [p + CTRL_BYTES for p in self.buf.ptrs]

    # handshake pieces ------------------------------------------------------------------------------
    def consume_lists(self):
        me, b = self.rank, self.buf
        wait = (b.local_ptr + _READY, b.local_ptr + _NREAD, 1, b.local_ptr + _NREAD, self.world)
        sig = (self.world, [p + _FREE + 4 * me for p in b.ptrs])
        return wait, sig

    def produce_lists(self):
        me, b = self.rank, self.buf
        wait = (b.local_ptr + _FREE, b.local_ptr + _NPROD, 0, b.local_ptr + _NPROD, self.world)
        sig = (self.world, [p + _READY + 4 * me for p in b.ptrs])
        return wait, sig

    @property
    def done_ptr(self) -> int:
        return self.buf.local_ptr + _DONE

    def close(self):
        self.buf.close()


def sync_descriptor(consume: Optional[PeerSlot] = None, produce: Optional[PeerSlot] = None) -> Optional[List[int]]:
    """Flat handshake descriptor for a kernel that reads `consume` from all peers and/or writes its copy of `produce`.

    Layout: [nwait, nsig, done_ctr, {wait, expected, offset, bump, peers} x 2, {peers, signal[8]} x 2]."""
    lists = []
    if consume is not None and getattr(consume, "is_peer", False):
        lists.append(consume.consume_lists())
    if produce is not None and getattr(produce, "is_peer", False):
        lists.append(produce.produce_lists())
    if not lists:
        return None
    first = consume if (consume is not None and getattr(consume, "is_peer", False)) else produce
    out = [len(lists), len(lists), first.done_ptr]
    for i in range(2):
        if i < len(lists):
            w = lists[i][0]
            out += [w[0], w[1], w[2], w[3], w[4]]
        else:
            out += [0, 0, 0, 0, 0]
    for i in range(2):
        if i < len(lists):
            n, ptrs = lists[i][1]
            out += [n] + list(ptrs) + [0] * (8 - len(ptrs))
        else:
            out += [0] * 9
    assert len(out) == 31
    return out


def begin_produce(slot) -> None:
    """Before a non-GEMM kernel overwrites this rank's copy of `slot`: wait until every peer has read the last one."""
    if getattr(slot, "is_peer", False):
        d = sync_descriptor(produce=slot)
        _ext.require().peer_sync(d, 0, slot.device.index)


def end_produce(slot) -> None:
    if getattr(slot, "is_peer", False):
        d = sync_descriptor(produce=slot)
        _ext.require().peer_sync(d, 1, slot.device.index)


class GatherSlot:
    """Same interface on top of an all-gather, for CPU runs (gloo) and for ranks that cannot map each other's
    memory: `sources()` returns every rank's copy as ordinary tensors."""

    is_peer = False

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cpu")
        self.capacity = int(nbytes)
        self.store = torch.zeros(self.capacity, dtype=torch.uint8, device=self.device)
        self._last = None

    def tensor(self, dtype, shape) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        esz = torch.empty((), dtype=dtype).element_size()
        self._last = self.store[: n * esz].view(dtype).view(*shape)
        return self._last

    def sources(self):
        t = self._last.contiguous()
        raw = t.view(-1).view(torch.uint8)
        outs = [torch.empty_like(raw) for _ in range(self.world)]
        dist.all_gather(outs, raw, group=self.group)
        return [o.view(t.dtype).view(t.shape) for o in outs]

    def close(self):
        pass


_SLOTS = {}


def get_slot(name: str, group_name: str, nbytes: int, device: torch.device):
    """Process-wide slot `name` over communicator group `group_name`, grown (collectively) to at least `nbytes`.
    Every rank of the group must request the same sizes in the same order."""
    from ..utils import comm

    key = (name, group_name, str(device))
    slot = _SLOTS.get(key)
    if slot is not None and slot.capacity >= nbytes:
        return slot
    if slot is not None:
        slot.close()
    group = comm.get_group(group_name)
    use_peer = device.type == "cuda" and dist.get_backend(group) == "nccl"
    cls = PeerSlot if use_peer else GatherSlot
    slot = cls(int(nbytes * 1.0), group=group, device=device)
    _SLOTS[key] = slot
    return slot


def release_slots() -> None:
    for slot in _SLOTS.values():
        slot.close()
    _SLOTS.clear()
