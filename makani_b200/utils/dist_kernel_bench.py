"""Micro-benchmark of the fused transform+communication GEMM stages on a (h x w) process grid of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m makani_b200.utils.dist_kernel_bench --h H --w W [--hw 721 1440] [--chans 384] [--iters 10]

One analysis + synthesis chain is launched per iteration with CUDA events recorded between the stages (after
warm-up; an all-reduce before each iteration keeps the ranks aligned and a 256 MB write flushes L2).  Per stage
the median over iterations, then the maximum over ranks, is reported with the roofline target: the slowest of
FLOPs / measured bf16 peak, bytes this rank stores into its peers' memory / 770 GB/s (measured peer-copy
bandwidth per direction) and local bytes / measured HBM bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops import spectral_dist as sd
from ..parallel import peer
from . import comm
from .kernel_bench import _peaks

NVLINK_BPS = 770e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--h", type=int, default=1)
    ap.add_argument("--w", type=int, default=1)
    ap.add_argument("--hw", nargs=2, type=int, default=[721, 1440])
    ap.add_argument("--modes", nargs=2, type=int, default=None, help="lmax mmax (default: nlat // 3 each)")
    ap.add_argument("--chans", type=int, default=384)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    comm.init(model_parallel_sizes=[args.h, args.w, 1, 1])
    _ext.require()
    hbm, flops_peak, src = _peaks()
    H, W = args.hw
    L, M = args.modes or (H // 3, H // 3)
    B, C = args.batch, args.chans
    ph, pw, rh, rw = comm.get_size("h"), comm.get_size("w"), comm.get_rank("h"), comm.get_rank("w")
    plan = sd.DistSHTPlan.get(H, W, L, M, "equiangular", ph, pw, rh, rw, dev)
    bf = torch.bfloat16
    x = torch.randn(B, C, plan.hl, plan.wl, device=dev).to(bf).contiguous(memory_format=torch.channels_last)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    sync_t = torch.zeros(1, device=dev)
    rows = B * plan.hl
    k2 = 2 * plan.ml
    n2 = 2 * C
    esz = 2

    # (l, m) pairs with l >= m: local l against local m (analysis rows), all l against local m (synthesis k range)
    m_glob = torch.arange(plan.m0, plan.m0 + plan.ml)
    pairs_an = int(((torch.arange(plan.l0, plan.l0 + plan.ll)[:, None] >= m_glob[None, :]).sum()))
    pairs_syn = int(((torch.arange(L)[:, None] >= m_glob[None, :]).sum()))
    # per stage: (flops, bytes this rank stores into its peers' memory over NVLink, local bytes read + written)
    t1_seg = rows * k2 * C * esz                  # this rank's T1 / T4 block
    coef_seg = B * plan.ll * plan.ml * n2 * esz   # this rank's coefficient block
    model = {
        "publish grid block": (0.0, (pw - 1) * rows * plan.wl * C * esz, 2 * rows * plan.wl * C * esz),
        "S1 dft analysis": (2.0 * k2 * W * C * rows, (ph - 1) * t1_seg, rows * W * C * esz + t1_seg),
        "S2 legendre analysis": (2.0 * pairs_an * H * n2 * B, 0, B * H * k2 * C * esz + coef_seg),
        "publish coefficient block": (0.0, (ph - 1) * coef_seg, 2 * coef_seg),
        "S4 legendre synthesis": (2.0 * pairs_syn * plan.hl * n2 * B, (pw - 1) * t1_seg, B * L * plan.ml * n2 * esz + t1_seg),
        "S5 dft synthesis": (2.0 * plan.wl * 2 * M * C * rows, 0, rows * 2 * M * C * esz + rows * plan.wl * C * esz),
    }
    holder = {}

    def chain(ev):
        def mark():
            if ev is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                ev.append(e)
        mark()
        s, v = sd.stage_grid_to_slot(x, plan)
        mark()
        t1slot, t1, hs = sd.stage_dft_analysis(s, v, plan.f_an, plan, B, C)
        mark()
        t2 = sd.stage_legendre_analysis(t1slot, t1, hs, plan.pw_an, plan, B, C)
        mark()
        slot, t3v, ls = sd.stage_lm_to_slot(t2, plan)
        mark()
        t4slot, t4, js = sd.stage_legendre_synthesis(slot, t3v, ls, True, plan.p_syn, plan, B, C)
        mark()
        holder["y"] = sd.stage_dft_synthesis(t4slot, t4, js, plan.g_syn, plan, B, C)
        mark()

    for _ in range(3):
        chain(None)
    names = list(model.keys())
    samples = [[] for _ in names]
    for _ in range(args.iters):
        flush.zero_()
        dist.all_reduce(sync_t)
        ev = []
        chain(ev)
        torch.cuda.synchronize()
        for i in range(len(names)):
            samples[i].append(ev[i].elapsed_time(ev[i + 1]))
    results = []
    for i, name in enumerate(names):
        samples[i].sort()
        t = torch.tensor([samples[i][len(samples[i]) // 2]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = max(t.item() * 1e-3, 1e-9)
        flops, link_b, local_b = model[name]
        roof = max(flops / flops_peak, link_b / NVLINK_BPS, local_b / hbm)
        results.append(dict(stage=name, ms=sec * 1e3, tflops=flops / sec / 1e12, nvlink_gbs=link_b / sec / 1e9,
                            local_gbs=local_b / sec / 1e9, roofline_ms=roof * 1e3, fraction=roof / sec))
    _ext.check_device_errors(dev)
    if comm.get_world_rank() == 0:
        print(json.dumps(dict(h=ph, w=pw, hw=[H, W], chans=C, peaks=src, results=results)))
        for r in results:
            print(f"{r['stage']:28s} {r['ms']:8.3f} ms  {r['tflops']:7.1f} TFLOP/s  NVLink out {r['nvlink_gbs']:6.1f} GB/s  "
                  f"local {r['local_gbs']:7.1f} GB/s  roofline {r['roofline_ms']:.3f} ms ({100 * r['fraction']:.0f}% of {src})")
    peer.release_slots()
    dist.barrier()
    comm.cleanup()


if __name__ == "__main__":
    main()
