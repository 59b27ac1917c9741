"""pytest configuration: the `gpu` marker and helpers to run multi-rank cases as child processes."""
import os
import socket
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture
def port():
    return free_port()


@pytest.fixture
def persist_mode():
    """Setter for the many-token GEMM selection (0 never, 2 / 3 forced tile shapes); the
    environment's choice is restored afterwards."""
    from libtbvcoll_b200 import ops
    yield ops.gemm_persist_mode
    ops.gemm_persist_mode(None)
