"""Time axis of yearly ERA5 files: the year is the first four characters of the file name and samples are equally
spaced from 1 January 00:00 UTC (counterpart of datasets/era5/time.py in the reference; timezone from the standard
library instead of pytz)."""

import datetime
import os
from typing import List


def filename_to_year(path: str) -> int:
    return int(os.path.basename(path)[:4])


def datetime_range(year: int, time_step: datetime.timedelta, n: int) -> List[datetime.datetime]:
    t0 = datetime.datetime(year=year, month=1, day=1, tzinfo=datetime.timezone.utc)
    return [t0 + i * time_step for i in range(n)]
