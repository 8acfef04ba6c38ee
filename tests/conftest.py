import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def built():
    """The product library and the oracle, built in-tree (no-op when up to date)."""
    import mcmc_bnn_example_b200 as m
    import oracle as O
    try:
        m.build()
    except Exception:
        if not os.path.exists(m.LIB_PATH):
            raise
    O.build()
    return m, O
