"""Download ERA5 pressure-level and surface fields from the Copernicus Climate Data Store, one NetCDF file per month
(and per pressure level).

    python datasets/copernicus/get_data.py --output_dir OUT --years 2018 2019 [--hourly_subsample 6] [--resolution 0.25]

Counterpart of datasets/copernicus/get_data.py in the reference: same product (`reanalysis-era5-complete`), parameters
(u, v, w, z, t, q on levels; 10u, 10v, 100u, 100v, 2t, sp, msl, tcwv at the surface) and file naming
(`raw/pl_<level>_<yyyy>-<mm>.nc`, `raw/sfc_<yyyy>-<mm>.nc`).  The request dictionaries are built by pure functions so they
can be inspected without network access; `cdsapi` is imported only when downloading.  `--pressure_level` is honoured
(the reference ignores it and always walks 50..1000 hPa).
"""

import argparse
import calendar
import os
from typing import Dict, List

PL_PARAMS = "131/132/135.128/129.128/130.128/133.128"
SFC_PARAMS = "165.128/166.128/246.228/247.228/167.128/134.128/151.128/137.128"


def timestamps(hourly_subsample: int) -> List[str]:
    return [f"{t:02d}:00" for t in range(0, 24, hourly_subsample)]


def _common(year: int, month: int, resolution: float, hourly_subsample: int) -> Dict:
    last = calendar.monthrange(year, month)[1]
    return {"class": "ea", "expver": "1", "stream": "oper", "type": "an", "grid": [resolution, resolution],
            "format": "netcdf", "date": f"{year}-{month:02d}-01/to/{year}-{month:02d}-{last:02d}",
            "time": timestamps(hourly_subsample)}


def pressure_level_request(year, month, level, resolution=0.25, hourly_subsample=1) -> Dict:
    return dict(_common(year, month, resolution, hourly_subsample), levtype="pl", levelist=str(level), param=PL_PARAMS)


def surface_request(year, month, resolution=0.25, hourly_subsample=1) -> Dict:
    return dict(_common(year, month, resolution, hourly_subsample), levtype="sfc", param=SFC_PARAMS)


def plan(output_dir, years, levels, resolution, hourly_subsample):
    """(file name, request) pairs in download order."""
    base = os.path.join(output_dir, "raw")
    out = []
    for y in years:
        for m in range(1, 13):
            for pl in levels:
                out.append((os.path.join(base, f"pl_{pl}_{y}-{m:02d}.nc"), pressure_level_request(y, m, pl, resolution, hourly_subsample)))
            out.append((os.path.join(base, f"sfc_{y}-{m:02d}.nc"), surface_request(y, m, resolution, hourly_subsample)))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--years", type=int, nargs="+", required=True)
    ap.add_argument("--pressure_level", type=int, nargs="+", default=list(range(50, 1050, 50)))
    ap.add_argument("--hourly_subsample", type=int, default=1)
    ap.add_argument("--resolution", type=float, default=0.25)
    ap.add_argument("--overwrite", action="store_true")
    ap.add_argument("--dry_run", action="store_true", help="print the planned files and exit")
    args = ap.parse_args(argv)
    jobs = plan(args.output_dir, args.years, args.pressure_level, args.resolution, args.hourly_subsample)
    if args.dry_run:
        for fname, _ in jobs:
            print(fname)
        return
    import cdsapi
    os.makedirs(os.path.join(args.output_dir, "raw"), exist_ok=True)
    client = cdsapi.Client()
    for fname, req in jobs:
        if os.path.isfile(fname):
            if not args.overwrite:
                print(f"{fname} exists, skipping")
                continue
            os.remove(fname)
        print(f"downloading {fname}")
        client.retrieve("reanalysis-era5-complete", req, fname)
    print("done")


if __name__ == "__main__":
    main()
