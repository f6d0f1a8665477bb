import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # keep files whose name starts with test_zz at the very end of the run
    items.sort(key=lambda it: (1 if os.path.basename(str(it.fspath)).startswith("test_zz") else 0))
