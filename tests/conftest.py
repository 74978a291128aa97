"""Shared fixtures. GPU tests carry the `gpu` marker; everything else runs on a CPU-only machine."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def built():
    """Builds the CUDA library and the CPU checkers once per session (no-op when they are up to date)."""
    import __graft_entry__ as ge

    ge.build()
    return ge


@pytest.fixture(scope="session")
def pkg(built):
    return built.load_package()


@pytest.fixture(scope="session")
def oracle(built):
    from oracle import oracle as O

    return O
