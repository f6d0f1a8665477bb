"""Rewrite yearly HDF5 files (dataset `fields`, [T, C, H, W]) as plain `.npy` files that the loaders memory-map
(the role of the reference's h5_convert.py / h5_align.py re-layout tools for its O_DIRECT reader).  Needs h5py."""

from __future__ import annotations

import argparse
import glob
import os

import numpy as np


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_path", required=True)
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--dataset", default="fields")
    ap.add_argument("--batch", default=32, type=int)
    args = ap.parse_args(argv)
    import h5py
    os.makedirs(args.output_path, exist_ok=True)
    for f in sorted(glob.glob(os.path.join(args.input_path, "????.h5"))):
        with h5py.File(f, "r") as h:
            d = h[args.dataset]
            out = np.lib.format.open_memmap(os.path.join(args.output_path, os.path.basename(f).replace(".h5", ".npy")),
                                            mode="w+", dtype=np.float32, shape=d.shape)
            for s in range(0, d.shape[0], args.batch):
                out[s:s + args.batch] = d[s:s + args.batch]
            out.flush()
        print("converted", f)


if __name__ == "__main__":
    main()
