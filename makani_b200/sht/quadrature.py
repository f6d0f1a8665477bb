"""Quadrature rules on the interval [-1, 1] used for latitude integration on the sphere.

The reference imports these from torch-harmonics
(`torch_harmonics.quadrature.{legendre_gauss_weights, clenshaw_curtiss_weights}`, used at
makani/utils/grids.py:19,32,77,83 and makani/utils/losses.py:31).  Here they are computed
from first principles in float64 numpy.

All functions return `(nodes, weights)` with nodes ascending in x = cos(theta) on [a, b].
"""

from __future__ import annotations

import numpy as np


def _rescale(x: np.ndarray, w: np.ndarray, a: float, b: float):
    x = (b - a) * 0.5 * x + (b + a) * 0.5
    w = w * (b - a) * 0.5
    return x, w


def legendre_gauss_weights(n: int, a: float = -1.0, b: float = 1.0):
    """Gauss-Legendre nodes and weights (roots of P_n), exact for polynomials of degree 2n-1."""
    x, w = np.polynomial.legendre.leggauss(n)
    return _rescale(np.asarray(x, dtype=np.float64), np.asarray(w, dtype=np.float64), a, b)


def lobatto_weights(n: int, a: float = -1.0, b: float = 1.0, tol: float = 1e-16, maxiter: int = 100):
    """Gauss-Lobatto nodes and weights (end points included), Newton iteration on P'_{n-1}."""
    x = np.cos(np.pi * np.arange(n) / (n - 1))  # Chebyshev-Gauss-Lobatto start, descending
    p = np.zeros((n, n), dtype=np.float64)
    for _ in range(maxiter):
        xold = x.copy()
        p[:, 0] = 1.0
        p[:, 1] = x
        for k in range(2, n):
            p[:, k] = ((2 * k - 1) * x * p[:, k - 1] - (k - 1) * p[:, k - 2]) / k
        x = xold - (x * p[:, n - 1] - p[:, n - 2]) / (n * p[:, n - 1])
        if np.max(np.abs(x - xold)) < tol:
            break
    w = 2.0 / ((n - 1) * n * p[:, n - 1] ** 2)
    x, w = x[::-1].copy(), w[::-1].copy()
    return _rescale(x, w, a, b)


def clenshaw_curtiss_weights(n: int, a: float = -1.0, b: float = 1.0):
    """Clenshaw-Curtis (Fejer type-2 with end points) nodes x_j = cos(j pi/(n-1)) and weights.

    w_j = c_j/(n-1) * [1 - sum_{k=1}^{floor((n-1)/2)} b_k/(4k^2-1) cos(2 k theta_j)]
    with c_j = 1 at the poles else 2, and b_k = 1 when 2k == n-1 else 2.  Sum of weights = 2.
    """
    assert n > 1
    theta = np.pi * np.arange(n, dtype=np.float64) / (n - 1)
    x = np.cos(theta)
    N = n - 1
    w = np.zeros(n, dtype=np.float64)
    kmax = N // 2
    k = np.arange(1, kmax + 1, dtype=np.float64)
    bk = np.where(2 * k == N, 1.0, 2.0)
    # [n, kmax]
    s = (bk / (4.0 * k * k - 1.0))[None, :] * np.cos(2.0 * k[None, :] * theta[:, None])
    w = 1.0 - s.sum(axis=1)
    c = np.full(n, 2.0)
    c[0] = 1.0
    c[-1] = 1.0
    w = c * w / N
    # ascending in x
    x, w = x[::-1].copy(), w[::-1].copy()
    return _rescale(x, w, a, b)


def trapezoidal_weights(n: int, a: float = -1.0, b: float = 1.0):
    x = np.linspace(a, b, n)
    w = np.full(n, (b - a) / (n - 1))
    w[0] *= 0.5
    w[-1] *= 0.5
    return x, w


def precompute_latitudes(nlat: int, grid: str = "equiangular"):
    """Colatitudes theta (ascending 0..pi, i.e. north pole first) and quadrature weights on cos(theta).

    Mirrors the grids accepted by the reference SHT objects ("equiangular", "legendre-gauss",
    "lobatto"; makani/models/networks/sfnonet.py:536-539).
    """
    if grid == "legendre-gauss":
        x, w = legendre_gauss_weights(nlat)
    elif grid == "equiangular":
        x, w = clenshaw_curtiss_weights(nlat)
    elif grid == "lobatto":
        x, w = lobatto_weights(nlat)
    else:
        raise ValueError(f"unknown grid type {grid}")
    # flip so that theta ascends (x = cos theta descends): north -> south
    theta = np.flip(np.arccos(np.clip(x, -1.0, 1.0))).copy()
    w = np.flip(w).copy()
    return theta, w
