import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


@pytest.fixture(scope="session")
def ops():
    import llumnix_kv_b200

    return llumnix_kv_b200.load_ops()
