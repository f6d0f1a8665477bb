"""Re-chunk (and optionally transpose to channels-last) the `fields` dataset of every yearly HDF5 file in a directory.

    python data_process/h5_convert.py --input_dir IN --output_dir OUT [--chunksize auto|none|<N>MB] [--transpose] [--overwrite]

Counterpart of data_process/h5_convert.py in the reference.  Differences: data is streamed one time step at a time
instead of being read whole into memory (a 721x1440x73 year is ~0.4 TB), and an existing output *file* is removed
with `os.remove` (the reference calls `shutil.rmtree` on it).  Needs h5py.
"""

import argparse
import glob
import os


def parse_chunks(spec, shape, itemsize):
    if spec == "auto":
        return True
    if spec == "none":
        return None
    if spec.endswith("MB"):
        limit = int(spec[:-2]) * 1024 * 1024
        per_step = itemsize
        for s in shape[1:]:
            per_step *= s
        steps = max(1, min(shape[0], limit // max(per_step, 1)))
        return (steps,) + tuple(shape[1:])
    raise ValueError(f"chunksize {spec!r} not supported")


def convert(ifname, ofname, chunksize, transpose):
    import h5py
    with h5py.File(ifname, "r") as fin:
        src = fin["fields"]
        shape = (src.shape[0], src.shape[2], src.shape[3], src.shape[1]) if transpose else src.shape
        with h5py.File(ofname, "w") as fout:
            dst = fout.create_dataset("fields", shape, dtype=src.dtype, chunks=parse_chunks(chunksize, shape, src.dtype.itemsize))
            for t in range(src.shape[0]):
                step = src[t]
                dst[t] = step.transpose(1, 2, 0) if transpose else step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--chunksize", default="auto")
    ap.add_argument("--transpose", action="store_true")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args()
    os.makedirs(args.output_dir, exist_ok=True)
    for ifname in sorted(glob.glob(os.path.join(args.input_dir, "*.h5"))):
        ofname = os.path.join(args.output_dir, os.path.basename(ifname))
        if os.path.exists(ofname):
            if not args.overwrite:
                print(f"{ofname} exists, skipping", flush=True)
                continue
            os.remove(ofname)
        print(f"{ifname} -> {ofname}", flush=True)
        convert(ifname, ofname, args.chunksize, args.transpose)


if __name__ == "__main__":
    main()
