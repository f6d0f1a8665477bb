"""Convert yearly `.h5` / `.npy` files into one zarr store per year.

    python data_process/zarr_convert.py --input_dir IN --output_dir OUT [--overwrite]

Counterpart of data_process/zarr_convert.py in the reference.  Needs `xarray` + `zarr` (not part of the base image): the
labelled array from `datasets.era5.open_year` is written with `Dataset.to_zarr`.
"""

import argparse
import glob
import os
import shutil
import sys

sys.path.append(os.path.dirname(os.path.dirname(os.path.realpath(__file__))))


def output_name(ifname: str, output_dir: str) -> str:
    base = os.path.basename(ifname)
    return os.path.join(output_dir, os.path.splitext(base)[0] + ".zarr")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    import datasets.era5 as era5
    files = sorted(glob.glob(os.path.join(args.input_dir, "*.h5")) + glob.glob(os.path.join(args.input_dir, "*.npy")))
    os.makedirs(args.output_dir, exist_ok=True)
    for ifname in files:
        ofname = output_name(ifname, args.output_dir)
        if os.path.exists(ofname):
            if not args.overwrite:
                print(f"{ofname} exists, skipping", flush=True)
                continue
            shutil.rmtree(ofname)
        arr = era5.open_year(ifname)
        if not hasattr(arr, "to_dataset"):
            raise SystemExit("zarr_convert needs xarray and zarr to be installed")
        print(f"{ifname} -> {ofname}", flush=True)
        arr.to_dataset().to_zarr(ofname)


if __name__ == "__main__":
    main()
