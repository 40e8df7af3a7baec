import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) and the built libkiln_cuda.so")


@pytest.fixture(scope="session")
def ctx():
    """One device context for the whole GPU session. Fails loudly when the extension is absent."""
    import torch
    from kiln_b200 import api
    assert torch.cuda.is_available(), "gpu-marked tests need a CUDA device"
    c = api.Context(0)
    yield c
    c.sync()
    st = c.device_status()
    assert st == 0, f"a kernel recorded a bounded-wait failure: 0x{st:x}"


def cosine(a, b):
    import torch
    a = a.float().flatten()
    b = b.float().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))
