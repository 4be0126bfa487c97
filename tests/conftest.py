import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)  # helper modules of the tests (gpu_util, parity_util)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_port():
    from oracle import backend
    backend.build()
    return backend.OracleBackend()


@pytest.fixture(scope="session")
def oracle_ref():
    from oracle import backend
    backend.build()
    if not backend.have_ref():
        pytest.skip("oracle/_ref/libqagg_ref.so not present (reference checkout absent and no prebuilt copy)")
    return backend.RefBackend()
