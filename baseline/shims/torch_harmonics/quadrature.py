"""Quadrature rules on cos(colatitude): each returns (nodes ascending in x, weights) as float64 numpy arrays."""

import numpy as np


def legendre_gauss_weights(n, a=-1.0, b=1.0):
    xlg, wlg = np.polynomial.legendre.leggauss(n)
    xlg = (b - a) * 0.5 * xlg + (b + a) * 0.5
    wlg = wlg * (b - a) * 0.5
    return xlg, wlg


def lobatto_weights(n, a=-1.0, b=1.0, tol=1e-16, maxiter=100):
    wlg = np.zeros((n,))
    tlg = np.zeros((n,))
    tmp = np.zeros((n,))
    vdm = np.zeros((n, n))
    # Chebyshev nodes as the initial guess, Newton iterations on the derivative of P_{n-1}
    for i in range(n):
        tlg[i] = -np.cos(np.pi * i / (n - 1))
    for _ in range(maxiter):
        tmp[:] = tlg
        vdm[:, 0] = 1.0
        vdm[:, 1] = tlg
        for k in range(2, n):
            vdm[:, k] = ((2 * k - 1) * tlg * vdm[:, k - 1] - (k - 1) * vdm[:, k - 2]) / k
        tlg = tmp - (tlg * vdm[:, n - 1] - vdm[:, n - 2]) / (n * vdm[:, n - 1])
        if np.max(np.abs(tlg - tmp)) < tol:
            break
    wlg = 2.0 / ((n * (n - 1)) * (vdm[:, n - 1] ** 2))
    tlg = (b - a) * 0.5 * tlg + (b + a) * 0.5
    wlg = wlg * (b - a) * 0.5
    return tlg, wlg


def clenshaw_curtiss_weights(n, a=-1.0, b=1.0):
    assert n > 1
    tcc = np.cos(np.linspace(np.pi, 0, n))
    if n == 2:
        wcc = np.array([1.0, 1.0])
    else:
        n1 = n - 1
        N = np.arange(1, n1, 2)
        ell = len(N)
        m = n1 - ell
        v = np.concatenate([2.0 / N / (N - 2), 1.0 / N[-1:], np.zeros(m)])
        v = 0 - v[:-1] - v[-1:0:-1]
        g0 = -np.ones(n1)
        g0[ell] = g0[ell] + n1
        g0[m] = g0[m] + n1
        g = g0 / (n1 ** 2 - 1 + (n1 % 2))
        wcc = np.fft.ifft(v + g).real
        wcc = np.concatenate((wcc, wcc[:1]))
    tcc = (b - a) * 0.5 * tcc + (b + a) * 0.5
    wcc = wcc * (b - a) * 0.5
    return tcc, wcc
