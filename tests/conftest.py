import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ops():
    """The product's host API, initialised on cuda:0.  Fails loudly without a GPU or the library."""
    from orin_llm_b200 import build, ops as _ops
    build.build()
    _ops.init(0)
    return _ops


@pytest.fixture(scope="session")
def refcuda(ops):
    """The reference's own CUDA kernels recompiled for sm_100a (oracle/_ref/libref_cuda.so), when they were built."""
    from oracle.oracle import RefCuda
    if not RefCuda.available():
        pytest.skip("oracle/_ref/libref_cuda.so is not built (needs the reference tree and nvcc at build time)")
    return RefCuda()
