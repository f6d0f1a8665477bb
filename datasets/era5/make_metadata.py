"""Write the dataset descriptor `data.json` (coords, channel names, time step) for a lat/lon dataset."""

import argparse
import json

import numpy as np

LEVELS = [50, 100, 150, 200, 250, 300, 400, 500, 600, 700, 850, 925, 1000]
CHANNELS = ["u10m", "v10m", "u100m", "v100m", "t2m", "sp", "msl", "tcwv"] + [f"{v}{l}" for v in "uvztq" for l in LEVELS]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--output", required=True)
    ap.add_argument("--nlat", default=721, type=int)
    ap.add_argument("--nlon", default=1440, type=int)
    ap.add_argument("--dhours", default=6, type=int)
    args = ap.parse_args(argv)
    meta = dict(dataset_name="era5_73ch", h5_path="fields", dhours=args.dhours,
                attrs=dict(description="ERA5 reanalysis subset, 73 variables"),
                coords=dict(grid_type="equiangular", lat=np.linspace(90, -90, args.nlat).tolist(),
                            lon=(np.arange(args.nlon) * 360.0 / args.nlon).tolist(), channel=CHANNELS))
    with open(args.output, "w") as f:
        json.dump(meta, f)


if __name__ == "__main__":
    main()
