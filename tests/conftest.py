import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def orc():
    from oracle import loader
    return loader.oracle()


@pytest.fixture(scope="session")
def ref():
    from oracle import loader
    if not loader.ref_available():
        pytest.skip("oracle/_ref not built (upstream sources not on this machine)")
    return loader.reference()


@pytest.fixture(scope="session")
def gpu_lib():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import adaptq_b200
    return adaptq_b200.load()
