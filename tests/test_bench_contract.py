"""CPU checks of bench.py's bookkeeping: every workload names a model preset that exists, and the algorithmic bytes and
flops of the headline verify step are the figures the roofline quotes (weights once, K/V once per sequence).
Nothing here touches a GPU or the oracle."""
import importlib.util
from pathlib import Path

import pytest

from kiln_b200 import synth

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_every_workload_names_a_preset(bench):
    for name, w in bench.WORKLOADS.items():
        preset, batch, k, lo, hi, gen = w[:6]
        assert preset in synth.PRESETS, name
        assert batch >= 1 and k >= 1 and 1 <= lo <= hi and gen >= 1, name
        cfg = synth.PRESETS[preset]
        assert batch * (k + 1) <= 512, f"{name}: a verify step of {batch * (k + 1)} rows exceeds the step-token limit"
        assert cfg.num_attention_heads % cfg.num_key_value_heads == 0, name
    assert bench.WORKLOADS["llama-3.1-8b-w4g64-verify-k5-bs32"][:3] == ("llama-3.1-8b", 32, 5)


def test_headline_algorithmic_bytes_and_flops(bench):
    cfg = synth.PRESETS["llama-3.1-8b"]
    a = bench.algorithmic(cfg, batch=32, k=5, mean_ctx=1400.0)
    assert a["M"] == 192
    # 4-bit weights with bf16 scale and bias per 64 inputs: 0.5 + 4/64 bytes per parameter, incl. the head
    params = cfg.num_hidden_layers * (2 * 4096 * 4096 + 2 * 1024 * 4096 + 3 * 14336 * 4096) + 128256 * 4096
    assert a["weight_bytes"] == pytest.approx(params * (0.5 + 4 / 64), rel=1e-12)
    assert 4.2e9 < a["weight_bytes"] < 4.25e9
    # K and V of every cached token once per sequence: 32 layers x 2 x 8 heads x 128 x 2 B = 128 KiB per token
    assert a["kv_read_bytes"] == pytest.approx(32 * 1400.0 * 131072)
    assert a["gemm_flops"] == pytest.approx(2 * 192 * params)
    assert a["attn_flops"] == pytest.approx(4 * 192 * 1400.0 * 32 * 128 * 32)
    assert 9.9e9 < a["bytes"] < 10.3e9


def test_tensor_parallel_workloads_shard_evenly(bench):
    for name, w in bench.WORKLOADS.items():
        opts = w[6] if len(w) > 6 else {}
        if not opts.get("tp"):
            continue
        cfg = synth.PRESETS[w[0]]
        for ranks in (2, 4, 8):
            assert cfg.num_key_value_heads % ranks == 0 and cfg.intermediate_size % (ranks * 128) == 0, (name, ranks)
