import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_stays_zero(request):
    """After every GPU test: no kernel-side bounded wait may have run out (the kernels then return
    early and leave outputs incomplete, which a lucky comparison could miss)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if not torch.cuda.is_available():
        return
    import turbofno_b200 as t

    for h in list(t.Handle._cache.values()):
        assert h.device_status == 0, "a kernel-side wait ran out during " + request.node.name
