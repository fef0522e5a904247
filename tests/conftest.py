import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")
    config.addinivalue_line("markers", "slow: full-size case (about a minute of CPU oracle time)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import ref

    ref.build()
    return ref
