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


def parity(label, got, want, bar=2e-2, min_cos=0.9999):
    """The floating-point bar, with the raw figures printed (and appended to the file named by KILN_PARITY_REPORT when
    that is set): max-abs <= `bar` flat wherever |want| < 4; where |want| >= 4 one bf16 spacing of the value is added,
    because two bf16 numbers of that magnitude cannot be closer than 0.03 unless they are equal. Returns True when the
    case is inside the bar and the cosine is at least `min_cos`."""
    g, w = got.float().flatten(), want.float().flatten()
    d = (g - w).abs()
    small = w.abs() < 4
    err_small = float(d[small].max()) if bool(small.any()) else 0.0
    err_all = float(d.max())
    excess_large = float((d - (bar + w.abs() * 2 ** -7))[~small].max()) if bool((~small).any()) else -1.0
    cos = cosine(got, want)
    line = (f"{label}: max-abs {err_all:.4g} (where |want| < 4: {err_small:.4g}; bar {bar:g}), cosine {cos:.7f}, "
            f"max |want| {float(w.abs().max()):.3g}, {int(g.numel())} values")
    print(line)
    path = os.environ.get("KILN_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")
    return err_small <= bar and excess_large <= 0 and cos >= min_cos
