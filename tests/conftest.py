import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 and the built libh3q8.so")


@pytest.fixture(scope="session")
def oracle():
    import oracle as module
    module.lib()
    return module


@pytest.fixture(scope="session")
def gpu():
    import h3cli_b200
    context = h3cli_b200.Gpu()
    yield context
    context.free()
