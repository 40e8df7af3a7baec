"""Generates the golden fixtures under tests/golden/ from the CPU oracle (run: python tests/golden/make_golden.py).

There is no upstream golden vector for the floating-point side of this path (the reference's fixtures need
Hugging Face checkpoints that do not exist here), so these files pin the ORACLE itself: a change to
oracle/kiln_oracle.cpp or kiln_b200/synth.py that moves a logit shows up as a fixture mismatch on CPU, and the
CUDA path is compared with the same files on the GPU. Each file: seeded prompts, the step batches, bf16 logit
bits of the sampled rows for both MLX arithmetic classes, and the greedy tokens.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from kiln_b200.api import SeqStep, StepBatch  # noqa: E402
from kiln_b200.synth import PRESETS, synth_checkpoint  # noqa: E402
from oracle import oracle as O  # noqa: E402

MODELS = ["tiny-llama", "tiny-llama-d128", "tiny-qwen2", "tiny-gemma2"]
BS, NB = 16, 32


def scenario(cfg):
    """Two steps: a ragged prefill of three prompts (last row sampled), then two verify segments + one decode."""
    g = torch.Generator().manual_seed(1234)
    lens = [37, 64, 5]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    tables = [[0, 1, 2], [3, 4, 5, 6, 7], [8]]
    step1 = StepBatch(sum(prompts, []), [SeqStep(n, 0, 1, t) for n, t in zip(lens, tables)])
    seg = [5, 5, 1]
    ids2 = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in seg]
    step2 = StepBatch(sum(ids2, []), [SeqStep(n, off, n, t) for n, off, t in zip(seg, lens, tables)])
    return [step1, step2]


def run(name):
    cfg = PRESETS[name]
    ck = synth_checkpoint(cfg, seed=0)
    model = O.OracleModel(cfg, ck)
    out = {}
    for cls in (0, 1):
        O.set_weight_class(cls)
        kv = O.OracleKv(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, NB, BS)
        for i, step in enumerate(scenario(cfg)):
            lg = model.forward_step(step, kv)
            out[f"logits_class{cls}_step{i}"] = lg.view(torch.int16).numpy().view(np.uint16)
            out[f"tokens_class{cls}_step{i}"] = O.greedy_rows(lg)
    O.set_weight_class(0)
    return out


if __name__ == "__main__":
    for name in MODELS:
        data = run(name)
        path = Path(__file__).resolve().parent / f"{name}.npz"
        np.savez_compressed(path, **data)
        print(path.name, {k: v.shape for k, v in data.items() if k.startswith("logits")}, path.stat().st_size, "bytes")
