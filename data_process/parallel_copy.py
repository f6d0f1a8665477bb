"""Copy a directory of yearly data files with several worker processes, verifying sizes.

    python data_process/parallel_copy.py --input_dir IN --output_dir OUT [--workers 8] [--pattern '*.h5'] [--overwrite]

The reference's data_process/parallel_copy.py distributes the files of a directory over MPI ranks and copies each
through h5py; this version needs neither MPI nor h5py: files are split round-robin over a process pool, copied in
16 MB blocks, and a file whose size differs afterwards is reported and counted as failed.
"""

import argparse
import glob
import os
import shutil
from multiprocessing import Pool


def _copy(job):
    src, dst, overwrite = job
    if os.path.exists(dst) and not overwrite and os.path.getsize(dst) == os.path.getsize(src):
        return dst, "skipped"
    tmp = dst + ".part"
    with open(src, "rb") as fi, open(tmp, "wb") as fo:
        shutil.copyfileobj(fi, fo, length=16 * 1024 * 1024)
    if os.path.getsize(tmp) != os.path.getsize(src):
        os.remove(tmp)
        return dst, "failed"
    os.replace(tmp, dst)
    return dst, "copied"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--workers", type=int, default=8)
    ap.add_argument("--pattern", default="*.h5")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args()
    os.makedirs(args.output_dir, exist_ok=True)
    files = sorted(glob.glob(os.path.join(args.input_dir, args.pattern)))
    jobs = [(f, os.path.join(args.output_dir, os.path.basename(f)), args.overwrite) for f in files]
    failed = 0
    with Pool(max(1, min(args.workers, len(jobs) or 1))) as pool:
        for dst, status in pool.imap_unordered(_copy, jobs):
            print(f"{status:8s} {dst}", flush=True)
            failed += status == "failed"
    raise SystemExit(1 if failed else 0)


if __name__ == "__main__":
    main()
