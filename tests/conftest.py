import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def native_libs():
    """Build (or reuse) the in-tree native libraries; no GPU needed."""
    from occamy_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def binding(native_libs):
    from occamy_b200 import replay
    return replay.Binding()
