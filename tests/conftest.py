import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from _oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from _oracle import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libcake_ref.so not built (reference tree absent)")
    return Reference()


@pytest.fixture(scope="session")
def cake():
    """The product package with its CUDA library built; never falls back to anything."""
    from cake_on_cpu_b200 import build
    build.build()
    import cake_on_cpu_b200
    cake_on_cpu_b200.lib()
    return cake_on_cpu_b200
