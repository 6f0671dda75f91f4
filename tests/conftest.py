import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture
def skv_switch(monkeypatch):
    """Set (or, with None, unset) one of the library's SKV_* environment switches for the current test.  The library
    reads them once, so every change is followed by skv_reload_env; the previous environment comes back afterwards."""
    from lokahi_b200 import _lib

    def set_switch(name, value):
        if value is None:
            monkeypatch.delenv(name, raising=False)
        else:
            monkeypatch.setenv(name, value)
        _lib.lib.skv_reload_env()

    yield set_switch
    monkeypatch.undo()
    _lib.lib.skv_reload_env()
