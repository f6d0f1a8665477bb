"""Import-time stand-in for `pytz` (absent from this image): `utc` and `timezone("UTC")` only."""

import datetime as _dt

utc = _dt.timezone.utc
UTC = utc


def timezone(name):
    if name.upper() != "UTC":
        raise ValueError("only UTC is available in this stand-in")
    return utc


__version__ = "2024.1"      # pandas asks for the version of every optional dependency it finds
