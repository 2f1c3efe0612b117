import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


@pytest.fixture(scope="session")
def ctx():
    """One context on GPU 0 for the whole session (the library has no CPU path: this raises without a GPU)."""
    import tachyon_b200 as tb

    c = tb.Context(0)
    yield c
    assert c.status() == 0, "a kernel reported a bounded wait that ran out"
    c.close()
