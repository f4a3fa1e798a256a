import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device")


@pytest.fixture(scope="session")
def ulm():
    """The product bindings; building the library first if this checkout has none."""
    import ulmblas_b200.build as b
    if not os.path.exists(b.LIB):
        b.build()
    import ulmblas_b200.api as api
    return api


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu but no CUDA device is visible")
    torch.cuda.init()
    return torch


@pytest.fixture(autouse=True)
def _library_rereads_its_environment():
    """The library reads its ULMB200_* variables once.  Tests that set one call ``ulm.reload_env()``
    themselves; this puts the library back on the unmodified environment afterwards (it is set up
    before ``monkeypatch`` and therefore torn down after it)."""
    yield
    api = sys.modules.get("ulmblas_b200.api")
    if api is not None:
        api.reload_env()
