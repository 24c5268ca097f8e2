import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__  # noqa: E402,F401  (registers the package as ``dfb_b200``)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu and needs a CUDA device")
    from dfb_b200 import native

    native.lib()  # fail loudly if the CUDA library was not built
    torch.cuda.set_device(0)
    return torch.device("cuda", 0)
