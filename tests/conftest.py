import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session", autouse=True)
def _kernel_variant_from_env():
    """PS_TEST_TUNE="bulk=2,unroll=1" runs the GPU tests on another kernel variant
    (keys and values as ps_tune takes them: bulk 0 / 2 / 3 / 4, unroll 1 / 2 / 4, ...)."""
    spec = os.environ.get("PS_TEST_TUNE", "")
    if spec:
        from patrickstar_b200 import _lib
        for kv in spec.split(","):
            k, v = kv.split("=")
            _lib.tune(k.strip(), int(v))
    yield


@pytest.fixture(scope="session")
def oracle_port():
    from oracle import port
    port.lib()
    return port


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
