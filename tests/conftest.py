import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as o

    o.lib()
    return o


@pytest.fixture(autouse=True, scope="session")
def _oracle_packs_the_test_models():
    """Synthetic models of the tests are packed by the oracle's packer, not by the library under test."""
    import oracle as o
    from quintrit_b200 import synth

    synth.PACKER = o.pack_planar
    yield
    synth.PACKER = None
