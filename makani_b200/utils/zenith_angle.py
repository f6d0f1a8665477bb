"""Cosine of the solar zenith angle from UTC time, longitude and latitude (vectorised numpy).

The reference vendors climt's implementation behind numba (makani/third_party/climt/zenith_angle.py:45-226).
This is an independent restatement of the same astronomical approximation (Julian centuries since J2000,
mean obliquity, solar mean longitude / anomaly, equation of centre, right ascension and declination, Greenwich
mean sidereal time -> local hour angle).
"""

from __future__ import annotations

import datetime

import numpy as np

RAD_PER_DEG = np.pi / 180.0
_J2000 = datetime.datetime(2000, 1, 1, 12, 0, 0, tzinfo=datetime.timezone.utc)


def _days_from_2000(times) -> np.ndarray:
    out = []
    for t in np.atleast_1d(times):
        if isinstance(t, np.datetime64):
            t = t.astype("datetime64[s]").astype(datetime.datetime)
        if t.tzinfo is None:
            t = t.replace(tzinfo=datetime.timezone.utc)
        out.append((t - _J2000).total_seconds() / 86400.0)
    return np.asarray(out, dtype=np.float64)


def _poly(x, coeffs):
    res = 0.0
    for c in reversed(coeffs):
        res = res * x + c
    return res


def _greenwich_mean_sidereal_time(jd):
    """GMST in radians."""
    theta = 67310.54841 + jd * (876600 * 3600 + 8640184.812866 + jd * (0.093104 - jd * 6.2e-5))
    return np.mod(theta * RAD_PER_DEG / 240.0, 2 * np.pi)


def _sun_ecliptic_longitude(jc):
    mean_anom = RAD_PER_DEG * _poly(jc, [357.52910, 35999.05030, -0.0001559, -0.00000048])
    mean_lon = RAD_PER_DEG * _poly(jc, [280.46645, 36000.76983, 0.0003032])
    d_l = RAD_PER_DEG * ((1.914600 - 0.004817 * jc - 0.000014 * jc * jc) * np.sin(mean_anom)
                         + (0.019993 - 0.000101 * jc) * np.sin(2 * mean_anom) + 0.000290 * np.sin(3 * mean_anom))
    return mean_lon + d_l


def _obliquity(jc):
    return RAD_PER_DEG * _poly(jc, [23.0 + 26.0 / 60 + 21.406 / 3600, -46.836769 / 3600, -0.0001831 / 3600,
                                     0.00200340 / 3600, -0.576e-6 / 3600, -4.34e-8 / 3600])


def cos_zenith_angle(time, lon, lat) -> np.ndarray:
    """time: datetime or array of datetimes [T]; lon/lat in degrees (arrays [H, W]) -> [T, H, W] (or [H, W])."""
    scalar = not isinstance(time, (list, tuple, np.ndarray))
    days = _days_from_2000(time)
    jc = days / 36525.0
    lon_r = np.asarray(lon, dtype=np.float64) * RAD_PER_DEG
    lat_r = np.asarray(lat, dtype=np.float64) * RAD_PER_DEG
    eps = _obliquity(jc)
    lam = _sun_ecliptic_longitude(jc)
    ra = np.arctan2(np.cos(eps) * np.sin(lam), np.cos(lam))
    dec = np.arcsin(np.sin(eps) * np.sin(lam))
    gmst = _greenwich_mean_sidereal_time(jc)
    shp = (-1,) + (1,) * lon_r.ndim
    hour_angle = gmst.reshape(shp) + lon_r[None] - ra.reshape(shp)
    cz = np.sin(lat_r)[None] * np.sin(dec).reshape(shp) + np.cos(lat_r)[None] * np.cos(dec).reshape(shp) * np.cos(hour_angle)
    return cz[0] if scalar else cz
