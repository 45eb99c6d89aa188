import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(autouse=True)
def _fresh_oracle():
    """Each test starts with an empty oracle tape, gradient map and handle table."""
    from oracle import oracle as orc
    orc.reset_all()
    yield
