"""Isolated timing of the peer-memory all-reduce (`csrc/peer.cu`) against NCCL on the GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m makani_b200.utils.peer_bench [--mb 64 256 1024] [--iters 10]

Per size and dtype: CUDA events around each call (after warm-up; the ranks are aligned by a barrier before every
call), median over iterations, maximum over ranks.  Reported: algorithm bandwidth (bytes of the buffer / time), bus
bandwidth (x 2(N-1)/N, the figure NCCL's tests quote) and the fraction of the kernel's NVLink roofline.  Every rank
reduces one slice: it pulls that slice from its N-1 peers and pushes the result to them.  Both the data a rank pulls and
the results its peers push to it arrive on its ingress links, (N-1)/N of the buffer each, so the floor is
2(N-1)/N x bytes / 770 GB/s (measured peer-copy rate per direction): the fraction is bus bandwidth / 770 GB/s.  These
kernels handshake across GPUs, so they are
timed with events and never put under a profiler's kernel replay.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import _ext
from ..parallel.peer import SymmetricBuffer

NVLINK_BPS = 770e9


def _time(fn, iters, dev):
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", nargs="+", type=int, default=[64, 256, 1024])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    _ext.require()
    nbytes = max(args.mb) * 1024 * 1024
    buf = SymmetricBuffer(nbytes, device=dev)
    plain = torch.empty(nbytes // 4, dtype=torch.float32, device=dev)
    rows = []
    for mb in args.mb:
        for dtype in (torch.float32, torch.bfloat16):
            esz = 4 if dtype == torch.float32 else 2
            n = mb * 1024 * 1024 // esz
            v = buf.view(dtype, n)
            v.normal_()
            w = plain.view(dtype)[:n] if dtype == torch.float32 else plain.view(torch.bfloat16)[:n]
            w.normal_()
            for _ in range(3):
                buf.all_reduce_(n, dtype, scale=1.0 / world)
                dist.all_reduce(w)
            t_peer = _time(lambda: buf.all_reduce_(n, dtype, scale=1.0 / world), args.iters, dev)
            t_nccl = _time(lambda: dist.all_reduce(w), args.iters, dev)
            _ext.check_device_errors(dev)
            b = mb * 1024 * 1024
            floor = 2 * (world - 1) / world * b / NVLINK_BPS * 1e3
            rows.append(dict(mb=mb, dtype=str(dtype).replace("torch.", ""), peer_ms=t_peer, nccl_ms=t_nccl,
                             peer_algbw_gbs=b / t_peer / 1e6, peer_busbw_gbs=b / t_peer / 1e6 * 2 * (world - 1) / world,
                             nccl_busbw_gbs=b / t_nccl / 1e6 * 2 * (world - 1) / world, roofline_ms=floor,
                             fraction=floor / t_peer))
    if rank == 0:
        print(json.dumps(dict(world=world, results=rows)))
        for r in rows:
            print(f"{r['mb']:5d} MB {r['dtype']:9s} peer {r['peer_ms']:7.3f} ms (bus {r['peer_busbw_gbs']:6.1f} GB/s, "
                  f"{100 * r['fraction']:.0f}% of the 770 GB/s ingress floor)   NCCL {r['nccl_ms']:7.3f} ms (bus {r['nccl_busbw_gbs']:6.1f} GB/s)")
    buf.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
