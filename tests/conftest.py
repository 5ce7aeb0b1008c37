import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from tests import cases
    return cases.Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own amd64 operations, when a prebuilt library this CPU can run is present."""
    from tests import cases
    ref = cases.Reference.try_load()
    if ref is None:
        pytest.skip("no prebuilt reference library (oracle/_ref) on this machine")
    return ref
