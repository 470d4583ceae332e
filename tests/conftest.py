import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def dev():
    """One Device (vtlb_ctx) on GPU 0 for the whole session.  The library must be
    built; a missing library is an error, a missing GPU skips."""
    from vtl_b200 import capi
    capi.load()
    if capi.device_count() == 0:
        pytest.skip("no CUDA device")
    d = capi.Device(0)
    yield d
    d.sync()
    assert d.check_status() == 0
    d.close()


@pytest.fixture(params=["tensor_cores_only", "small_products_on_cuda_cores"])
def gemm_path(request, dev):
    """Runs a test twice: with every f32 product forced onto the tcgen05 path, and with the
    library's default routing of small products to the CUDA-core kernel."""
    dev.set_small_gemm_limit(0.0 if request.param == "tensor_cores_only" else 1.4e8)
    yield request.param
    dev.set_small_gemm_limit(1.4e8)


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.build()
    return oracle
