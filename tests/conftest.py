import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def ctx():
    import torch
    from diffgemma_b200.step_attn import Context
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    c = Context(0)
    yield c
    c.close()
