import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def tf_ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from turbo_fieldfare_b200.kernels import TurboContext
    ctx = TurboContext(0)
    yield ctx
    ctx.close()
