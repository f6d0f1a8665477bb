"""Symmetric peer memory for the GPUs of one NVSwitch node.

Every rank of a process group allocates the same-sized buffer with `cudaMalloc`, exports a CUDA IPC handle,
exchanges the handles through `torch.distributed` and maps all peers' buffers.  Kernels then receive the raw
peer pointers and move data with plain loads/stores over NVLink (no NCCL call on the hot path, no TMA
multicast).  The reference has no counterpart: all its communication goes through NCCL process groups
(makani/utils/comm.py:97-133).
"""

from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext

FLAG_BYTES = 128 * 9 * 4  # PEER_MAX_BLOCKS * (PEER_MAX + 1) * sizeof(uint32), see csrc/peer.cuh

# How far apart the ranks of a data-parallel group may reach the gradient all-reduce (rank-0-only logging, a slow
# first batch, a checkpoint write).  Lost ranks are detected on the host (utils/watchdog.py), so this is generous.
PEER_SKEW_SECONDS = float(os.environ.get("MAKANI_B200_PEER_SKEW_SECONDS", "120"))


_DIAG_SELF = "selfar" in os.environ.get("MAKANI_B200_DP_DIAG", "").split(",")


class SymmetricBuffer:
    """`nbytes` of device memory on every rank of `group`, mapped into every other rank."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None, flag_sets: int = 1):
        """`flag_sets` > 1 reserves that many independent barrier-flag areas, so that collectives over different
        sub-groups of `group` (see `all_reduce_`'s `members`) never share epoch counters."""
        assert dist.is_initialized(), "SymmetricBuffer needs an initialised process group"
        self.ext = _ext.require()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= 8, "peer collectives support up to 8 ranks (one NVSwitch node)"
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.flag_sets = max(1, int(flag_sets))
        with torch.cuda.device(self.device):
            out: list = []
            handle = self.ext.peer_alloc(self.nbytes + self.flag_sets * FLAG_BYTES, out)
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

    def all_reduce_(self, numel: int, dtype=torch.float32, scale: float = 1.0, byte_offset: int = 0,
                    wait_seconds: Optional[float] = None, members: Optional[List[int]] = None, flag_set: int = 0) -> None:
        """In-place sum (times `scale`) over the group of `numel` elements starting at `byte_offset`.

        `members` (ranks of this buffer's group, in the order of the sub-group, this rank among them) restricts the
        reduction to a sub-group, e.g. the ranks that share a parameter under model parallelism; every sub-group
        family must use its own `flag_set`, and all its members must issue the same sequence of calls on it.

        `wait_seconds` bounds how long a rank waits for its peers inside the kernel (default: `PEER_SKEW_SECONDS`).
        It is the tolerated skew between ranks, not a liveness check: when it runs out the kernel leaves with
        error code 16 and the fused optimiser skips its update."""
        assert dtype in (torch.float32, torch.bfloat16)
        assert 0 <= flag_set < self.flag_sets
        if members is None:
            members, my = list(range(self.world)), self.rank
        else:
            members = [int(m) for m in members]
            my = members.index(self.rank)
        if len(members) == 1:
            if scale != 1.0:
                self.view(dtype, numel, byte_offset).mul_(scale)
            return
        ptrs = [self.ptrs[m] + byte_offset for m in members]
        if _DIAG_SELF:
            # diagnosis only (results are wrong): every "peer" is this rank's own buffer, so the kernel does the same
            # work and handshakes without any NVLink traffic; tells link contention from SM / L2 / HBM contention
            ptrs = [self.ptrs[self.rank] + byte_offset] * len(members)
        flags = [self.flag_ptrs[m] + flag_set * FLAG_BYTES for m in members]
        self.ext.peer_allreduce(ptrs, flags, my, int(numel), 1 if dtype == torch.bfloat16 else 0,
                                float(scale), float(PEER_SKEW_SECONDS if wait_seconds is None else wait_seconds),
                                self.device.index)

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
# A slot is a symmetric buffer holding one segment per rank of a group.  A producing kernel on rank r writes
# segment r of EVERY rank's copy (plain stores over NVLink from its epilogue: an all-gather done by the
# producer, tile by tile, while it computes); a later kernel on every rank reads all segments from its own,
# local copy.  Data therefore crosses NVLink exactly once per destination and is re-read from local HBM / L2.
# Ordering between ranks is kept by monotonic counters in device memory, so no host synchronisation and no NCCL
# call is involved and the whole sequence can be captured in a CUDA graph:
#
#   ready[p]  (on every rank)  incremented by rank p when its segment of generation g has been written everywhere
#   free[p]   (on every rank)  incremented by rank p when it has finished reading generation g
#   n_prod, n_read (local)     generations produced / consumed so far by this rank
#
# A producer waits for free[p] >= n_prod for all p, a consumer for ready[p] >= n_read + 1; both waits are bounded
# in the kernels (a device error code is raised instead of a hang).

CTRL_BYTES = 256
_READY, _FREE, _NPROD, _NREAD, _DONE = 0, 32, 64, 68, 72   # byte offsets inside the control block


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class PeerSlot:
    """Symmetric buffer of `world` segments plus handshake counters over one communicator group (CUDA, one node)."""

    is_peer = True

    def __init__(self, seg_bytes: int, group=None, device: Optional[torch.device] = None):
        world = dist.get_world_size(group)
        self.seg_capacity = (int(seg_bytes) + 255) // 256 * 256
        self.buf = SymmetricBuffer(CTRL_BYTES + world * self.seg_capacity, group=group, device=device)
        self.world, self.rank, self.device = self.buf.world, self.buf.rank, self.buf.device
        self.seg_stride = self.seg_capacity

    def set_layout(self, seg_bytes: int) -> None:
        """Segment stride for the next produce/consume pair (identical on every rank)."""
        self.seg_stride = (int(seg_bytes) + 255) // 256 * 256
        assert self.seg_stride <= self.seg_capacity

    # data ------------------------------------------------------------------------------------------
    def tensor(self, dtype, shape) -> torch.Tensor:
        """This rank's segment inside its own copy."""
        return self.buf.view(dtype, _numel(shape), CTRL_BYTES + self.rank * self.seg_stride).view(*shape)

    def dests(self, include_self: bool = False):
        """Addresses of this rank's segment inside every peer's copy (written by this rank's kernels only)."""
        off = CTRL_BYTES + self.rank * self.seg_stride
        return [p + off for r, p in enumerate(self.buf.ptrs) if include_self or r != self.rank]

    def sources(self):
        """Addresses of all segments inside this rank's own copy."""
        return [self.buf.local_ptr + CTRL_BYTES + q * self.seg_stride for q in range(self.world)]

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

    def publish(self, src: torch.Tensor, rows: int, row_elems: int, src_stride: int, dst_stride: int) -> None:
        """Strided copy of `rows` x `row_elems` elements of `src` into this rank's segment of every copy, with the
        producer handshake done by the same kernel."""
        esz = src.element_size()
        _ext.require().peer_publish(src, int(rows), int(row_elems) * esz, int(src_stride) * esz, int(dst_stride) * esz,
                                    self.dests(include_self=True), sync_descriptor(produce=self))

    def reduce_into(self, out: torch.Tensor, bias: Optional[torch.Tensor] = None, channels: int = 0) -> None:
        """out = sum over all ranks' segments (+ bias over the innermost `channels`), consumer handshake included.
        `out` must be bf16 and dense in memory in the order of the segments' contents."""
        _ext.require().peer_sum(out, self.sources(), bias, int(channels), sync_descriptor(consume=self))

    def close(self):
        self.buf.close()


def sync_descriptor(consume: Optional[PeerSlot] = None, produce: Optional[PeerSlot] = None) -> Optional[List[int]]:
    """Flat handshake descriptor for a kernel that reads all segments of `consume` and/or writes its segment of
    `produce` on every rank.

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


class GatherSlot:
    """Same interface on top of an all-gather, for CPU runs (gloo) and for ranks that cannot map each other's
    memory: the producer keeps its segment locally and `sources()` gathers every rank's segment."""

    is_peer = False

    def __init__(self, seg_bytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cpu")
        self.seg_capacity = int(seg_bytes)
        self.store = torch.zeros(self.seg_capacity, dtype=torch.uint8, device=self.device)
        self._last = None

    def set_layout(self, seg_bytes: int) -> None:
        assert seg_bytes <= self.seg_capacity

    def tensor(self, dtype, shape) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        self._last = self.store[: _numel(shape) * esz].view(dtype).view(*shape)
        return self._last

    def dests(self, include_self: bool = False):
        return None

    def publish(self, src, rows, row_elems, src_stride, dst_stride) -> None:
        flat_src = src.reshape(-1) if src.is_contiguous() else src.as_strided((src.untyped_storage().nbytes() // src.element_size() - src.storage_offset(),), (1,))
        s = flat_src.as_strided((rows, row_elems), (src_stride, 1))
        self._last.view(-1).as_strided((rows, row_elems), (dst_stride, 1)).copy_(s)

    def reduce_into(self, out, bias=None, channels=0) -> None:
        parts = self.sources()
        acc = parts[0].float()
        for p in parts[1:]:
            acc = acc + p.float()
        acc = acc.reshape(-1)
        if bias is not None:
            acc = (acc.view(-1, channels) + bias.float().view(1, channels)).reshape(-1)
        flat = out.permute(0, 2, 3, 1).reshape(-1) if (out.dim() == 4 and not out.is_contiguous()) else out.reshape(-1)
        flat.copy_(acc.to(out.dtype))

    def sources(self):
        t = self._last.contiguous()
        raw = t.view(-1).view(torch.uint8)
        outs = [torch.empty_like(raw) for _ in range(self.world)]
        dist.all_gather(outs, raw, group=self.group)
        return [o.view(t.dtype).view(t.shape) for o in outs]

    def close(self):
        pass


_SLOTS = {}


def get_slot(name: str, group_name: str, seg_bytes: int, device: torch.device):
    """Process-wide slot `name` over communicator group `group_name` with room for `seg_bytes` per rank, grown
    collectively when a larger request comes.  Every rank of the group must request the same sizes in the same
    order (sizes are therefore computed from group-wide maximum extents)."""
    from ..utils import comm

    key = (name, group_name, str(device))
    slot = _SLOTS.get(key)
    if slot is None or slot.seg_capacity < seg_bytes:
        if slot is not None:
            slot.close()
        group = comm.get_group(group_name)
        use_peer = device.type == "cuda" and dist.get_backend(group) == "nccl"
        slot = (PeerSlot if use_peer else GatherSlot)(int(seg_bytes), group=group, device=device)
        _SLOTS[key] = slot
    slot.set_layout(seg_bytes)
    return slot


def release_slots() -> None:
    for slot in _SLOTS.values():
        slot.close()
    _SLOTS.clear()
