import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def C():
    import splitrpc_b200

    return splitrpc_b200._C


@pytest.fixture()
def mtu8k(C):
    old = C.rpc_mtu()
    C.set_rpc_mtu(8192)
    yield 8192
    C.set_rpc_mtu(old)


@pytest.fixture()
def mtu1k(C):
    old = C.rpc_mtu()
    C.set_rpc_mtu(1024)
    yield 1024
    C.set_rpc_mtu(old)


def lenet5_weights(seed=0):
    import numpy as np

    rng = np.random.default_rng(seed)
    shapes = [(6, 1, 5, 5), (6,), (16, 6, 5, 5), (16,), (120, 400), (120,), (84, 120), (84,), (10, 84), (10,)]
    return [(rng.standard_normal(s) * 0.1).astype(np.float32) for s in shapes]
