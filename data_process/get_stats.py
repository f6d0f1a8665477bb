"""Normalisation statistics of a dataset of yearly `[T, C, H, W]` files (`????.npy`, or `????.h5` with h5py).

Writes `global_means.npy`, `global_stds.npy`, `mins.npy`, `maxs.npy` ([1, C, 1, 1]), `time_means.npy`
([1, C, H, W]) and `time_diff_means.npy`, `time_diff_stds.npy` ([1, C, 1, 1], statistics of x[t+dt] - x[t]) into
`--output_path`.  Work is split over time and merged with Welford/Chan updates, across `torch.distributed`
ranks when launched with torchrun (gloo), otherwise in one process.  Latitude weighting uses the sin(theta)
quadrature so that polar rows do not dominate.  Same products as the reference's MPI tool
(data_process/get_stats.py:97-132,225-264,405-412).
"""

from __future__ import annotations

import argparse
import glob
import os

import numpy as np


def _open(path, dataset):
    if path.endswith(".npy"):
        return np.load(path, mmap_mode="r")
    import h5py
    return h5py.File(path, "r")[dataset]


def welford_combine(a, b):
    """Merge (count, mean, M2) triples (Chan et al.)."""
    na, ma, m2a = a
    nb, mb, m2b = b
    n = na + nb
    if n == 0:
        return a
    d = mb - ma
    mean = ma + d * (nb / n)
    m2 = m2a + m2b + d * d * (na * nb / n)
    return n, mean, m2


def chunk_stats(arr, quad):
    """arr: [t, C, H, W] float64; quad: [H, 1] weights summing to 1 over (H, W)."""
    t = arr.shape[0]
    wmean = (arr * quad).sum(axis=(2, 3))                       # [t, C]
    mean = wmean.mean(axis=0)
    m2 = (((arr - mean[None, :, None, None]) ** 2) * quad).sum(axis=(2, 3)).sum(axis=0)
    return float(t), mean, m2


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_path", required=True)
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--dataset", default="fields")
    ap.add_argument("--dt", default=1, type=int)
    ap.add_argument("--batch", default=16, type=int)
    args = ap.parse_args(argv)

    rank, world = 0, 1
    try:
        import torch.distributed as dist
        if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1:
            dist.init_process_group("gloo")
            rank, world = dist.get_rank(), dist.get_world_size()
    except Exception:
        dist = None

    files = sorted(glob.glob(os.path.join(args.input_path, "????.npy")) + glob.glob(os.path.join(args.input_path, "????.h5")))
    assert files, f"no yearly files in {args.input_path}"
    first = _open(files[0], args.dataset)
    C, H, W = first.shape[1:]
    lat = np.linspace(0, np.pi, H)
    quad = np.clip(np.sin(lat), 0, None)[:, None] * np.ones((1, W))
    quad = quad / quad.sum()

    acc = (0.0, np.zeros(C), np.zeros(C))
    dacc = (0.0, np.zeros(C), np.zeros(C))
    tsum = np.zeros((C, H, W))
    tcount = 0.0
    mins, maxs = np.full(C, np.inf), np.full(C, -np.inf)
    work = []
    for f in files:
        n = _open(f, args.dataset).shape[0]
        for s in range(0, n, args.batch):
            work.append((f, s, min(n, s + args.batch)))
    for i, (f, s, e) in enumerate(work):
        if i % world != rank:
            continue
        d = _open(f, args.dataset)
        arr = np.asarray(d[s:e], dtype=np.float64)
        acc = welford_combine(acc, chunk_stats(arr, quad))
        tsum += arr.sum(axis=0)
        tcount += arr.shape[0]
        mins = np.minimum(mins, arr.min(axis=(0, 2, 3)))
        maxs = np.maximum(maxs, arr.max(axis=(0, 2, 3)))
        e2 = min(d.shape[0], e + args.dt)
        if e2 - s > args.dt:
            nxt = np.asarray(d[s + args.dt:e2], dtype=np.float64)
            diff = nxt - np.asarray(d[s:s + nxt.shape[0]], dtype=np.float64)
            dacc = welford_combine(dacc, chunk_stats(diff, quad))

    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (acc, dacc, tsum, tcount, mins, maxs))
        acc = (0.0, np.zeros(C), np.zeros(C))
        dacc = (0.0, np.zeros(C), np.zeros(C))
        tsum, tcount = np.zeros((C, H, W)), 0.0
        mins, maxs = np.full(C, np.inf), np.full(C, -np.inf)
        for a, da, ts, tc, mn, mx in gathered:
            acc, dacc = welford_combine(acc, a), welford_combine(dacc, da)
            tsum, tcount = tsum + ts, tcount + tc
            mins, maxs = np.minimum(mins, mn), np.maximum(maxs, mx)

    if rank == 0:
        os.makedirs(args.output_path, exist_ok=True)
        sh = (1, C, 1, 1)
        np.save(os.path.join(args.output_path, "global_means.npy"), acc[1].reshape(sh).astype(np.float32))
        np.save(os.path.join(args.output_path, "global_stds.npy"), np.sqrt(acc[2] / max(acc[0], 1.0)).reshape(sh).astype(np.float32))
        np.save(os.path.join(args.output_path, "mins.npy"), mins.reshape(sh).astype(np.float32))
        np.save(os.path.join(args.output_path, "maxs.npy"), maxs.reshape(sh).astype(np.float32))
        np.save(os.path.join(args.output_path, "time_means.npy"), (tsum / max(tcount, 1.0))[None].astype(np.float32))
        np.save(os.path.join(args.output_path, "time_diff_means.npy"), dacc[1].reshape(sh).astype(np.float32))
        np.save(os.path.join(args.output_path, "time_diff_stds.npy"), np.sqrt(dacc[2] / max(dacc[0], 1.0)).reshape(sh).astype(np.float32))
        print(f"statistics of {int(acc[0])} samples written to {args.output_path}")


if __name__ == "__main__":
    main()
