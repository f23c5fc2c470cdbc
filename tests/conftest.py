import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as o

    o.lib()
    return o


@pytest.fixture(scope="session")
def zkb():
    import zk_inference_prover_b200 as z
    from zk_inference_prover_b200 import build

    build.build()
    return z


@pytest.fixture(scope="session")
def ctx(zkb):
    c = zkb.Context(device=0, max_log_size=22)
    yield c
    c.close()
