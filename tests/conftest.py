import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # the file that exercises the allocation-free entry point runs last
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)
