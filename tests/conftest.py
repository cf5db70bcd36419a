import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (B200)")


@pytest.fixture(scope="session")
def lib():
    import mccl_b200
    return mccl_b200.load()
