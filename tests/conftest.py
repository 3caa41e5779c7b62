import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session", autouse=True)
def parity_report():
    """When QFA_PARITY_REPORT names a file, the error figures measured by the parity tests of this
    session (max-abs / output scale, the part beyond storage rounding, cosine) are written there as JSON."""
    yield
    path = os.environ.get("QFA_PARITY_REPORT")
    if path:
        import json
        from parity_util import REPORT
        with open(path, "w") as f:
            json.dump(REPORT, f, indent=1)
