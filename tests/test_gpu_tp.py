"""Tensor parallelism (the 70B configuration's partition) on two GPUs: skipped where fewer are visible."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.timeout(600)
def test_two_rank_forward_matches_oracle_and_ranks_agree():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "tp_check.py")],
                       capture_output=True, text=True, timeout=560, cwd=str(ROOT))
    assert r.returncode == 0 and "TP CHECK PASSED" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
