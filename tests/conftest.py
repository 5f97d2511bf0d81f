import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def backend():
    """One context on cuda:0 for the whole session.  No skip: a GPU test without a
    usable GPU or without the built library must fail loudly."""
    import rustygradients_b200 as rg
    return rg.B200Backend(0)
