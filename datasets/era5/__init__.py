"""Labelled view of one ERA5 year file (`<year>.h5` with dataset `fields[time, channel, lat, lon]`, or `<year>.npy`).

`open_year(path)` returns an `xarray.DataArray` when xarray is installed (dask-chunked for .h5 when dask is there, as
datasets/era5/__init__.py:31-70 of the reference does) and otherwise a light `LabelledArray` carrying the same
dims / coords / attrs, so that the tools in `data_process/` work with or without the scientific stack.
"""

import datetime
import json
import pathlib
from dataclasses import dataclass, field
from typing import Any, Dict, Sequence, Tuple

import numpy as np

from . import time as era5_time

__all__ = ["open_year", "open_34_vars", "LabelledArray", "METADATA"]

METADATA = pathlib.Path(__file__).parent / "data.json"


@dataclass
class LabelledArray:
    data: Any
    dims: Tuple[str, ...]
    coords: Dict[str, Any]
    attrs: Dict[str, Any] = field(default_factory=dict)
    name: str = "fields"

    @property
    def shape(self):
        return tuple(self.data.shape)

    def __getitem__(self, idx):
        return np.asarray(self.data[idx])


def _open_array(path: str, h5_path: str):
    if path.endswith(".npy"):
        return np.load(path, mmap_mode="r")
    import h5py
    return h5py.File(path, "r")[h5_path]


def open_year(path: str, chunks: Sequence[int] = (1, 1, -1, -1), metadata_path=None, time_step_hours=None):
    meta = json.loads(pathlib.Path(metadata_path or METADATA).read_text())
    h5_path = meta.get("h5_path", "fields")
    dims = tuple(meta.get("dims", ["time", "channel", "lat", "lon"]))
    arr = _open_array(path, h5_path)
    n = int(arr.shape[0])
    step = datetime.timedelta(hours=time_step_hours or meta.get("dhours", 6))
    coords = dict(meta.get("coords", {}))
    coords.pop("grid_type", None)
    nchan = int(arr.shape[1])
    if "channel" in coords and len(coords["channel"]) != nchan:
        coords["channel"] = [f"channel_{i}" for i in range(nchan)]
    coords["time"] = era5_time.datetime_range(era5_time.filename_to_year(path), step, n)
    attrs = dict(meta.get("attrs", {}), path=path)
    try:
        import xarray
    except ImportError:
        return LabelledArray(arr, dims, coords, attrs, h5_path)
    data = arr
    try:
        import dask.array as da
        data = da.from_array(arr, chunks=tuple(chunks))
    except ImportError:
        pass
    times = np.array([t.replace(tzinfo=None) for t in coords["time"]], dtype="datetime64[ns]")
    out = xarray.DataArray(data, name=h5_path, dims=dims)
    return out.assign_coords(time=times, **{k: v for k, v in coords.items() if k != "time"}).assign_attrs(attrs)


open_34_vars = open_year   # name used by the reference's tools
