"""Rewrite yearly HDF5 files so that the `fields` dataset starts on an aligned file offset (for O_DIRECT / GPUDirect
style readers), optionally transposed to channels-last, or check that aligned files open with the direct driver.

    python data_process/h5_align.py --input_dir IN --output_dir OUT [--align_size_bytes 4096] [--batch_size 32]
                                    [--transpose] [--overwrite] [--verify_integrity]

Counterpart of data_process/h5_align.py in the reference (user block of `align_size_bytes`, contiguous dataset, copy in
batches of time steps).  The direct-IO access list is used when this h5py build offers it and silently skipped
otherwise; an existing output file is removed with `os.remove`.  Needs h5py.
"""

import argparse
import glob
import os


def batches(n: int, size: int):
    for start in range(0, n, size):
        yield start, min(start + size, n)


def align_file(ifname, ofname, align, block, batch, transpose):
    import h5py
    fcpl = h5py.h5p.create(h5py.h5p.FILE_CREATE)
    fcpl.set_userblock(max(512, align))
    fapl = h5py.h5p.create(h5py.h5p.FILE_ACCESS)
    if hasattr(fapl, "set_fapl_direct"):
        try:
            fapl.set_fapl_direct(align, block, 0)
        except Exception:
            pass
    with h5py.File(ifname, "r") as fin:
        src = fin["fields"]
        shape = (src.shape[0], src.shape[2], src.shape[3], src.shape[1]) if transpose else src.shape
        fid = h5py.h5f.create(ofname.encode("ascii"), flags=h5py.h5f.ACC_TRUNC, fcpl=fcpl, fapl=fapl)
        fout = h5py.Group(fid)
        dst = fout.create_dataset("fields", shape, dtype=src.dtype)
        for a, b in batches(src.shape[0], batch):
            data = src[a:b]
            dst[a:b] = data.transpose(0, 2, 3, 1) if transpose else data
        fid.close()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--batch_size", type=int, default=32)
    ap.add_argument("--align_size_bytes", type=int, default=4096)
    ap.add_argument("--block_size_bytes", type=int, default=0)
    ap.add_argument("--verify_integrity", action="store_true")
    ap.add_argument("--transpose", action="store_true")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    os.makedirs(args.output_dir, exist_ok=True)
    for ifname in sorted(glob.glob(os.path.join(args.input_dir, "*.h5"))):
        if args.verify_integrity:
            import h5py
            try:
                f = h5py.File(ifname, "r", driver="direct")
            except Exception:
                f = h5py.File(ifname, "r")
            print(f"{ifname}: shape {f['fields'].shape}", flush=True)
            f.close()
            continue
        ofname = os.path.join(args.output_dir, os.path.basename(ifname))
        if os.path.exists(ofname):
            if not args.overwrite:
                print(f"{ofname} exists, skipping", flush=True)
                continue
            os.remove(ofname)
        print(f"{ifname} -> {ofname}", flush=True)
        align_file(ifname, ofname, args.align_size_bytes, args.block_size_bytes, args.batch_size, args.transpose)


if __name__ == "__main__":
    main()
