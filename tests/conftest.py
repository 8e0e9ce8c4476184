import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def _has_cuda():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


class _Options:
    """Sets library options (mg_set_option) for one test; everything goes back to the
    environment's values afterwards."""

    def __init__(self):
        import mixedgemm_b200 as mg
        self._mg = mg

    def setenv(self, name, value):  # same call shape as monkeypatch.setenv
        self._mg.set_option(name, int(value))

    set = setenv


@pytest.fixture
def mgopt():
    o = _Options()
    try:
        yield o
    finally:
        o._mg.reset_options()
        o._mg.set_wait_limit_us(0)
