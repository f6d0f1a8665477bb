"""Orthonormal associated Legendre functions for the spherical harmonic transforms.

`legendre_table(mmax, lmax, theta)` returns P[m, l, k] = Pbar_l^m(cos theta_k) with the
"ortho" normalisation (sum over the sphere of |Y_l^m|^2 = 1) and the Condon-Shortley phase,
zero for l < m.  This is the table that torch-harmonics' `RealSHT` holds as its `weights`
buffer (call sites: makani/models/networks/sfnonet.py:523-539).  Computed in float64 with the
standard three-term recurrence in degree l, vectorised over (m, k).
"""

from __future__ import annotations

import numpy as np


def legendre_table(mmax: int, lmax: int, theta: np.ndarray, csphase: bool = True) -> np.ndarray:
    theta = np.asarray(theta, dtype=np.float64)
    nlat = theta.shape[0]
    x = np.cos(theta)
    s = np.sin(theta)
    nmax = max(mmax, lmax)

    # diagonal terms P_m^m, shape [nmax, nlat]
    pmm = np.zeros((nmax, nlat), dtype=np.float64)
    pmm[0] = 1.0 / np.sqrt(4.0 * np.pi)
    for m in range(1, nmax):
        pmm[m] = np.sqrt((2.0 * m + 1.0) / (2.0 * m)) * s * pmm[m - 1]

    out = np.zeros((mmax, lmax, nlat), dtype=np.float64)
    mm = np.arange(mmax, dtype=np.float64)[:, None]  # [mmax,1]
    prev1 = np.zeros((mmax, nlat))  # P[m, l-1]
    prev2 = np.zeros((mmax, nlat))  # P[m, l-2]
    for l in range(lmax):
        cur = np.zeros((mmax, nlat))
        # m == l
        if l < mmax:
            cur[l] = pmm[l]
        # m == l-1
        if l >= 1 and (l - 1) < mmax:
            cur[l - 1] = np.sqrt(2.0 * l + 1.0) * x * prev1[l - 1]
        # m <= l-2
        hi = min(l - 1, mmax)  # rows [0, hi)
        if hi > 0:
            m_ = mm[:hi]
            a = np.sqrt((2.0 * l - 1.0) * (2.0 * l + 1.0) / ((l - m_) * (l + m_)))
            b = np.sqrt((l + m_ - 1.0) * (l - m_ - 1.0) * (2.0 * l + 1.0) / ((l - m_) * (l + m_) * (2.0 * l - 3.0)))
            cur[:hi] = a * x[None, :] * prev1[:hi] - b * prev2[:hi]
        out[:, l, :] = cur
        prev2 = prev1
        prev1 = cur

    if csphase:
        out[1::2] *= -1.0
    return out
