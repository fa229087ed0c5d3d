import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_addoption(parser):
    parser.addoption("--device", action="store", default="cuda")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library must exist for every test; build it if it is stale or missing."""
    from trident_b200 import build

    build.build()


@pytest.fixture
def device(request):
    dev = request.config.getoption("--device")
    if dev.startswith("cuda") and not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return dev


@pytest.fixture(params=[torch.float32, torch.float16, torch.bfloat16], ids=["fp32", "fp16", "bf16"])
def dtype(request):
    return request.param
