import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(autouse=True)
def _fresh_engine():
    """Every test starts and ends without a process-global engine."""
    import kraken_b200.pytorch as kk

    kk.stop()
    yield
    kk.stop()
