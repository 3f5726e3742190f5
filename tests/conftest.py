import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "timeout: limit of a test in seconds (pytest-timeout)")


def pytest_collection_modifyitems(config, items):
    """Every device-side wait is bounded, but a launch that never returned would leave the
    whole run hanging in a call no signal interrupts: with pytest-timeout installed a GPU
    test that takes longer than five minutes ends the run with the stacks printed (method
    "thread"), instead of holding the GPU until somebody kills the process."""
    if not config.pluginmanager.hasplugin("timeout"):
        return
    for item in items:
        if item.get_closest_marker("gpu") is not None and item.get_closest_marker("timeout") is None:
            item.add_marker(pytest.mark.timeout(300, method="thread"))


@pytest.fixture(scope="session")
def native_lib():
    """Build (if stale) and load libypk.so; CPU-only machines can still dlopen it."""
    from yirage_b200 import build, _native
    build.build()
    return _native.load()
