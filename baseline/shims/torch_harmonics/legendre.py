"""Orthonormal associated Legendre functions P̄_l^m(cos θ) by the standard three-term recurrence (float64, host)."""

import numpy as np


def precompute_legpoly(mmax, lmax, theta, norm="ortho", inverse=False, csphase=True):
    """Returns the table `[mmax, lmax, len(theta)]` (zero for l < m)."""
    nmax = max(mmax, lmax)
    x = np.cos(theta)
    s = np.sin(theta)
    vdm = np.zeros((nmax, nmax, len(theta)), dtype=np.float64)
    norm_factor = 1.0 if norm == "ortho" else np.sqrt(4 * np.pi)
    norm_factor = 1.0 / norm_factor if inverse else norm_factor
    vdm[0, 0, :] = norm_factor / np.sqrt(4 * np.pi)
    for l in range(1, nmax):
        vdm[l - 1, l, :] = np.sqrt(2 * l + 1) * x * vdm[l - 1, l - 1, :]
        vdm[l, l, :] = np.sqrt((2 * l + 1) / (2 * l)) * s * vdm[l - 1, l - 1, :]
    for l in range(2, nmax):
        for m in range(0, l - 1):
            vdm[m, l, :] = (x * np.sqrt((2 * l - 1) / (l - m) * (2 * l + 1) / (l + m)) * vdm[m, l - 1, :]
                            - np.sqrt((l + m - 1) / (l - m) * (2 * l + 1) / (2 * l - 3) * (l - m - 1) / (l + m)) * vdm[m, l - 2, :])
    if norm == "schmidt":
        for l in range(0, nmax):
            f = np.sqrt(2 * l + 1)
            vdm[:, l, :] = vdm[:, l, :] * f if inverse else vdm[:, l, :] / f
    vdm = vdm[:mmax, :lmax]
    if csphase:
        vdm[1::2] *= -1.0
    return vdm
