"""Shared pytest set-up: the `gpu` marker, import paths and the two libraries."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    import zt_oracle
    zt_oracle.lib()
    return zt_oracle


@pytest.fixture(scope="session")
def zt():
    """The package (its directory name has a hyphen, so it is imported by string)."""
    return importlib.import_module("z-transformer_b200")
