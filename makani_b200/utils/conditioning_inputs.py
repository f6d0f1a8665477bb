"""Readers for static conditioning fields (orography `Z`, land-sea mask `LSM`).

The reference reads netCDF files (makani/utils/conditioning_inputs.py:25-42).  Here `.npy` files are read
directly and netCDF / HDF5 files through whichever of netCDF4 / h5py / scipy.io is importable.
"""

from __future__ import annotations

import numpy as np


def _read_var(path: str, var: str) -> np.ndarray:
    if path.endswith(".npy"):
        return np.load(path)
    try:
        import netCDF4 as nc  # type: ignore
        with nc.Dataset(path, "r") as f:
            return np.asarray(f.variables[var][:])
    except ImportError:
        pass
    try:
        import h5py  # type: ignore
        with h5py.File(path, "r") as f:
            return np.asarray(f[var][...])
    except ImportError:
        pass
    from scipy.io import netcdf_file
    with netcdf_file(path, "r", mmap=False) as f:
        return np.array(f.variables[var][:])


def get_orography(orography_path: str) -> np.ndarray:
    """Surface geopotential / orography as [H, W] float32."""
    oro = np.asarray(_read_var(orography_path, "Z"), dtype=np.float32)
    return oro.reshape(oro.shape[-2], oro.shape[-1])


def get_land_mask(land_mask_path: str) -> np.ndarray:
    """Binary land-sea mask as [H, W] integers (fractions are rounded)."""
    lsm = np.asarray(_read_var(land_mask_path, "LSM"), dtype=np.float32)
    lsm = lsm.reshape(lsm.shape[-2], lsm.shape[-1])
    return np.rint(lsm).astype(np.int64)
