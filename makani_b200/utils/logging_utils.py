"""Logging configuration helpers (contract: makani/utils/logging_utils.py:16-64)."""

import logging
import os
import subprocess
from contextlib import contextmanager

_format = "%(asctime)s - %(name)s - %(levelname)s - %(message)s"


def config_logger(log_level=logging.INFO):
    logging.basicConfig(format=_format, level=log_level, force=True)


def log_to_file(logger_name=None, log_level=logging.INFO, log_filename="tensorflow.log"):
    d = os.path.dirname(log_filename)
    if d and not os.path.exists(d):
        os.makedirs(d, exist_ok=True)
    log = logging.getLogger(logger_name) if logger_name is not None else logging.getLogger()
    fh = logging.FileHandler(log_filename)
    fh.setLevel(log_level)
    fh.setFormatter(logging.Formatter(_format))
    log.addHandler(fh)


def log_versions():
    import torch

    try:
        h = subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).decode().strip()
    except Exception:
        h = "unknown"
    logging.info("--------------- Versions ---------------")
    logging.info("git hash: " + h)
    logging.info("Torch: " + str(torch.__version__))
    logging.info("----------------------------------------")


@contextmanager
def disable_logging(level=logging.ERROR):
    logging.disable(level=level)
    try:
        yield
    finally:
        logging.disable(level=logging.NOTSET)
