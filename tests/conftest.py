import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def orc():
    from oracle import q4_oracle
    q4_oracle.lib()
    return q4_oracle


@pytest.fixture(scope="session")
def q4b():
    """The package (its directory name is not a Python identifier)."""
    return importlib.import_module("cpu-llms-in-c_b200")
