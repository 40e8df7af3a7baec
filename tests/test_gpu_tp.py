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


def test_two_devices_in_one_process():
    """Kernel attributes (dynamic shared memory opt-in) belong to a device's copy of the kernel: a second context on a
    second device in the same process must run the GEMM (both lanes) and the attention like the first."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from kiln_b200 import api
    from kiln_b200.synth import PRESETS, quantize_affine, synth_checkpoint
    outs = []
    for dev in (0, 1):
        torch.cuda.set_device(dev)
        ctx = api.Context(dev)
        g = torch.Generator().manual_seed(3)
        w = torch.empty(256, 512).normal_(0, 0.02, generator=g)
        p, s, b = quantize_affine(w, 4, 64)
        x = torch.randn(5, 512, generator=g).to(torch.bfloat16)
        qw = api.QuantizedWeight(ctx, p.cuda(dev), s.cuda(dev), b.cuda(dev), 4, 64)
        y = qw.matmul(x.cuda(dev)).cpu()
        ys = qw.matmul_stream(x.cuda(dev)).cpu()
        cfg = PRESETS["tiny-llama"]
        model = api.CudaModel(ctx, cfg, synth_checkpoint(cfg, seed=0), max_step_tokens=64, max_step_seqs=4)
        kv = api.PagedKv(ctx, model.kv_spec(16, 16))
        ids = torch.randint(0, cfg.vocab_size, (20,), generator=g).tolist()
        lg = model.forward_step(api.StepBatch(ids, [api.SeqStep(20, 0, 1, [0, 1])]), kv)
        ctx.sync()
        outs.append((y, ys, lg.cpu().clone()))
        assert ctx.device_status() == 0
        qw.close(); model.close(); kv.close(); ctx.close()
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
