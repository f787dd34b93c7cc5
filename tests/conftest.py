import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def library():
    from flash_gordon_b200.build import build_library
    build_library()
    from flash_gordon_b200 import load_library
    return load_library()


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.load("port")


@pytest.fixture(scope="session")
def context(library):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test ran without a CUDA device: there is no CPU fallback to test")
    from flash_gordon_b200 import Context
    ctx = Context(0)
    yield ctx
    ctx.close()
