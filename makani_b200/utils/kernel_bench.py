"""Micro-benchmarks of the individual sm_100a kernels with roofline fractions.

    python -m makani_b200.utils.kernel_bench [--case NAME ...] [--hw H W] [--iters N] [--json]

Each case times one kernel launch configuration with CUDA events (after warm-up, L2 flushed between
iterations by writing a 256 MB buffer) and reports achieved bytes/s and FLOP/s against the measured peaks in
`MEASURED_PEAKS.json` at the repository root (fallback 6.65 TB/s, 1.59 PFLOP/s when the file is absent).
Cases mirror the launches of the SFNO-73ch training step so that a profiler can be pointed at exactly one
of them (`--case conv_fc1 --iters 1`).
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import _ext
from ..ops.conv import _conv_dgrad, _conv_fwd, _conv_wgrad, prep_weight
from ..ops.gemm import ACT_DGELU, ACT_GELU, ACT_MULAUX, ACT_NONE, Operand, Output, gemm


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def _time(fn, iters, flush):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2] * 1e-3


def cases(H, W, dev, B=1, layout="cl"):
    hw = H * W * B
    bf = torch.bfloat16
    C, C2 = 384, 768
    out = {}
    lay = (lambda t: t.contiguous(memory_format=torch.channels_last)) if layout == "cl" else (lambda t: t)

    def conv_case(ci, co, act, preact, resid, deriv=False):
        x = lay(torch.randn(B, ci, H, W, device=dev).to(bf))
        w = prep_weight(torch.randn(co, ci, device=dev) * 0.05)
        b = torch.zeros(co, device=dev)
        r = lay(torch.randn(B, co, H, W, device=dev).to(bf)) if resid else None
        nbytes = (ci + co * (2 if preact else 1) + (co if resid else 0)) * hw * 2
        flops = 2.0 * ci * co * hw
        return (lambda: _conv_fwd(x, w, ci, b, act, r, preact, deriv=deriv)), nbytes, flops

    out["conv_fc1"] = lambda: conv_case(C, C2, ACT_GELU, True, False, deriv=True)   # MLP fc1: bias + GELU + saved GELU'
    out["conv_fc1_pre"] = lambda: conv_case(C, C2, ACT_GELU, True, False)      # same with the pre-activation saved instead
    out["conv_fc2"] = lambda: conv_case(C2, C, ACT_NONE, False, False)         # MLP fc2
    out["conv_skip"] = lambda: conv_case(C, C, ACT_NONE, False, True)          # outer skip with fused residual add
    out["conv_plain"] = lambda: conv_case(C, C, ACT_NONE, False, False)

    def dgrad_gelu(act):
        dy = lay(torch.randn(1, C, H, W, device=dev).to(bf))
        w = prep_weight(torch.randn(C, C2, device=dev) * 0.05)
        pre = lay(torch.randn(1, C2, H, W, device=dev).to(bf))
        nbytes = (C + 2 * C2) * hw * 2
        return (lambda: _conv_dgrad(dy, w, C2, act=act, aux=pre)), nbytes, 2.0 * C * C2 * hw

    out["conv_dgrad_gelu"] = lambda: dgrad_gelu(ACT_MULAUX)      # what the MLP runs: times the saved GELU'
    out["conv_dgrad_gelu_eval"] = lambda: dgrad_gelu(ACT_DGELU)  # GELU' evaluated from a saved pre-activation

    def wgrad():
        dy = lay(torch.randn(1, C, H, W, device=dev).to(bf))
        x = lay(torch.randn(1, C2, H, W, device=dev).to(bf))
        return (lambda: _conv_wgrad(dy, x)), (C + C2) * hw * 2, 2.0 * C * C2 * hw

    out["conv_wgrad"] = wgrad

    def dft_fwd():
        from ..ops.spectral import SHTPlan, dft_analysis
        plan = SHTPlan.get(H, W, H // 3, W // 6 + 1, "equiangular", dev)
        x = torch.randn(1, C, H, W, device=dev).to(bf).contiguous(memory_format=torch.channels_last)
        nbytes = C * hw * 2 + plan.k2 * C * H * 2
        return (lambda: dft_analysis(x, plan.f, False, plan.nlon, plan.k2)), nbytes, 2.0 * plan.k2 * W * C * H

    out["dft_analysis"] = dft_fwd

    def inorm():
        from ..ops.norm import instance_norm
        x = lay(torch.randn(1, C, H, W, device=dev).to(bf))
        w, b = torch.ones(C, device=dev), torch.zeros(C, device=dev)
        return (lambda: instance_norm(x, w, b, 1e-6, "gelu")), 3 * C * hw * 2, 0.0

    out["inorm_gelu"] = inorm

    # ---- the spectral stages of one SFNO block on the internal grid (H/3 x W/3 Gauss grid, lmax = H/3, mmax = lmax + 1)
    def _plan():
        from ..ops.spectral import SHTPlan
        hi, wi = H // 3, W // 3
        return SHTPlan.get(hi, wi, hi, hi + 1, "legendre-gauss", dev), hi, wi

    def leg_analysis():
        from ..ops.spectral import legendre_analysis
        plan, hi, wi = _plan()
        t1 = torch.randn(1, hi, plan.k2, C, device=dev).to(bf)
        pairs = sum(max(0, plan.lmax - m) for m in range(plan.mmax))
        nbytes = t1.numel() * 2 + plan.lmax * plan.mmax * 2 * C * 2 + plan.pw.numel() * 2
        return (lambda: legendre_analysis(t1, plan.pw)), nbytes, 2.0 * pairs * hi * 2 * C

    out["legendre_analysis"] = leg_analysis

    def leg_synthesis():
        from ..ops.spectral import legendre_synthesis
        plan, hi, wi = _plan()
        t3 = torch.randn(1, plan.mmax, plan.lmax, 2 * C, device=dev).to(bf)
        pairs = sum(max(0, plan.lmax - m) for m in range(plan.mmax))
        nbytes = t3.numel() * 2 + hi * plan.k2 * C * 2 + plan.p.numel() * 2
        return (lambda: legendre_synthesis(t3, False, plan.p, hi)), nbytes, 2.0 * pairs * hi * 2 * C

    out["legendre_synthesis"] = leg_synthesis

    def contraction():
        from ..ops.spectral import contract
        plan, hi, wi = _plan()
        t2 = torch.randn(1, plan.lmax, plan.mmax, 2 * C, device=dev).to(bf)
        wx = (torch.randn(plan.lmax, 2 * C, 2 * C, device=dev) * 0.05).to(bf)
        pairs = sum(min(l + 1, plan.mmax) for l in range(plan.lmax))
        nbytes = 2 * t2.numel() * 2 + wx.numel() * 2
        return (lambda: contract(t2, wx, False)), nbytes, 2.0 * pairs * (2 * C) * (2 * C)

    out["contract"] = contraction

    def adamw():
        from ..ops.optim import FusedAdamW
        n = 64 * 1024 * 1024                        # 64 Mi parameters: 28 bytes of traffic each (p, g, m, v read; p, m, v written)
        prm = torch.nn.Parameter(torch.randn(n, device=dev))
        prm.grad = torch.randn(n, device=dev)
        opt = FusedAdamW([prm], lr=1e-3)
        return (lambda: opt.step()), 28.0 * n, 0.0

    out["adamw"] = adamw

    def lp():
        from ..ops.loss import weighted_lp_norms
        pr = torch.randn(1, 73, H, W, device=dev).to(bf)
        tg = torch.randn(1, 73, H, W, device=dev).to(bf)
        q = torch.full((H,), 1.0 / (H * W), device=dev)
        return (lambda: weighted_lp_norms(pr, tg, q, 2)), 2.0 * 73 * H * W * 2, 0.0

    out["lp_norms"] = lp

    def afno():
        from ..ops import afno as afno_ops
        hh, ww, cc, nb = H // 8, W // 8, 768, 8           # FourCastNet token grid for a 720 x 1440 field: 90 x 180
        bs = cc // nb
        x = torch.randn(1, hh, ww, cc, device=dev).to(bf)
        ps = [torch.randn(nb, bs, bs, device=dev) * 0.05 for _ in range(2)] + [torch.zeros(nb, bs, device=dev) for _ in range(2)]
        ps = ps + [torch.randn(nb, bs, bs, device=dev) * 0.05 for _ in range(2)] + [torch.zeros(nb, bs, device=dev) for _ in range(2)]
        kx, ncols = afno_ops.mode_window_v1(hh, ww, 1.0)
        nkx = len(kx)
        flops = 2.0 * cc * (2 * ncols * ww * hh + 2 * nkx * 2 * hh * ncols) * 2 + 2.0 * 2 * ncols * nkx * nb * (2 * bs) * (2 * bs)
        nbytes = 3.0 * x.numel() * 2                       # read x (twice: input and skip), write y; intermediates stay in L2
        return (lambda: afno_ops.afno_filter(x, *ps, kx, ncols, 0.01, skip=x)), nbytes, flops

    out["afno_filter"] = afno
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", nargs="*", default=None)
    ap.add_argument("--hw", nargs=2, type=int, default=[721, 1440])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1, help="images per launch for the conv cases")
    ap.add_argument("--layout", default="cl", choices=["cl", "nchw"], help="activation layout of the conv / norm cases")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    _ext.require()
    dev = torch.device("cuda", 0)
    hbm, flops_peak, src = _peaks()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    all_cases = cases(args.hw[0], args.hw[1], dev, args.batch, args.layout)
    names = args.case or list(all_cases.keys())
    results = []
    for name in names:
        fn, nbytes, flops = all_cases[name]()
        t = _time(fn, args.iters, flush)
        _ext.check_device_errors(dev)
        roof = max(nbytes / hbm, flops / flops_peak)
        res = dict(case=name, hw=args.hw, seconds=t, gbytes_per_s=nbytes / t / 1e9, tflops=flops / t / 1e12,
                   roofline_seconds=roof, fraction_of_roofline=roof / t, peaks=src)
        results.append(res)
        if not args.json:
            print(f"{name:18s} {t * 1e3:8.3f} ms  {res['gbytes_per_s']:8.1f} GB/s  {res['tflops']:7.1f} TFLOP/s  "
                  f"{100 * res['fraction_of_roofline']:5.1f}% of {src} roofline")
        del fn
        torch.cuda.empty_cache()
    if args.json:
        print(json.dumps(results))


if __name__ == "__main__":
    main()
