"""Synthetic checkpoints in the mlx-lm tensor convention, for tests and benchmarks.

No real checkpoint exists where this code runs, so weights are seeded N(0, 0.02) values quantised by
this module's own min/max affine quantiser into the mlx storage format:

  weight  uint32 [out, in * bits / 32]   element j of a row in bits [bits*(j % (32/bits)), +bits) of
                                          word j // (32/bits)  (LSB first)
  scales  bf16   [out, in / group]
  biases  bf16   [out, in / group]        w ≈ q * scale + bias

Tensor names follow crates/kiln-models/src/nn.rs:1092-1115 (model.embed_tokens, model.layers.N.self_attn.
{q,k,v,o}_proj, model.layers.N.mlp.{gate,up,down}_proj, *_layernorm, model.norm, lm_head). The quantiser
is NOT mlx's (that one is third-party and not in the reference tree); it only has to be
self-consistent between the generator, the CPU oracle and the kernels. torch is used as an array
library here, on CPU or GPU.
"""
from __future__ import annotations

import hashlib
from typing import Dict

import torch

from .api import ModelConfig


def quantize_affine(w: torch.Tensor, bits: int, group: int):
    """Min/max affine quantisation of fp32 ``w [out, in]`` → (packed int32 holding the u32 bits, scales, biases)."""
    out_f, in_f = w.shape
    assert in_f % group == 0 and (32 % bits) == 0
    levels = (1 << bits) - 1
    g = w.reshape(out_f, in_f // group, group).float()
    lo = g.amin(dim=-1, keepdim=True)
    hi = g.amax(dim=-1, keepdim=True)
    scale = ((hi - lo) / levels).clamp_min(1e-8)
    # scales/biases are stored in bf16; quantise against the values the kernels will actually use
    scale = scale.to(torch.bfloat16).float()
    bias = lo.to(torch.bfloat16).float()
    q = torch.round((g - bias) / scale).clamp_(0, levels).to(torch.int64)
    per = 32 // bits
    q = q.reshape(out_f, in_f // per, per)
    shifts = (torch.arange(per, device=w.device, dtype=torch.int64) * bits)
    packed = (q << shifts).sum(dim=-1)                      # < 2**32
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed.contiguous(), scale.squeeze(-1).to(torch.bfloat16).contiguous(), bias.squeeze(-1).to(torch.bfloat16).contiguous()


def dequantize_affine(packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group: int) -> torch.Tensor:
    """fp32 ``q * scale + bias`` (no rounding) — used by tests only."""
    per = 32 // bits
    u = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(per, device=packed.device, dtype=torch.int64) * bits)
    q = ((u.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)).reshape(packed.shape[0], -1).float()
    s = scales.float().repeat_interleave(group, dim=1)
    b = biases.float().repeat_interleave(group, dim=1)
    return q * s + b


def _gen(seed: int, name: str, device) -> torch.Generator:
    h = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & 0x7FFFFFFFFFFFFFFF
    g = torch.Generator(device=device)
    g.manual_seed(h)
    return g


def synth_checkpoint(cfg: ModelConfig, seed: int = 0, device="cpu", num_layers: int | None = None,
                     std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random-init checkpoint of architecture ``cfg``; each tensor has its own seeded stream, so a
    checkpoint truncated to fewer layers (a draft model) shares the kept tensors bit for bit."""
    dev = torch.device(device)
    L = cfg.num_hidden_layers if num_layers is None else num_layers
    H, D = cfg.hidden_size, cfg.head_dim
    Hq, Hkv, F, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size, cfg.vocab_size
    out: Dict[str, torch.Tensor] = {}

    def qlinear(prefix: str, n_out: int, n_in: int, with_bias: bool = False):
        rows_per = max(1, min(n_out, (1 << 25) // n_in))   # bound the fp32 scratch
        ws, ss, bs = [], [], []
        g = _gen(seed, prefix, dev)
        for r0 in range(0, n_out, rows_per):
            r1 = min(n_out, r0 + rows_per)
            w = torch.empty(r1 - r0, n_in, dtype=torch.float32, device=dev).normal_(0.0, std, generator=g)
            p, s, b = quantize_affine(w, cfg.bits, cfg.group_size)
            ws.append(p); ss.append(s); bs.append(b)
        out[prefix + ".weight"] = torch.cat(ws) if len(ws) > 1 else ws[0]
        out[prefix + ".scales"] = torch.cat(ss) if len(ss) > 1 else ss[0]
        out[prefix + ".biases"] = torch.cat(bs) if len(bs) > 1 else bs[0]
        if with_bias:
            out[prefix + ".bias"] = torch.empty(n_out, dtype=torch.float32, device=dev).normal_(
                0.0, std, generator=_gen(seed, prefix + ".bias", dev)).to(torch.bfloat16)

    def norm(name: str):
        # plain archs: weight 1; gemma stores w and applies 1 + w, so w = 0 (nn.rs:241-257)
        val = 0.0 if cfg.model_type == "gemma2" else 1.0
        out[name] = torch.full((H,), val, dtype=torch.bfloat16, device=dev)

    qlinear("model.embed_tokens", V, H)
    for i in range(L):
        p = f"model.layers.{i}"
        qlinear(p + ".self_attn.q_proj", Hq * D, H, cfg.qkv_bias)
        qlinear(p + ".self_attn.k_proj", Hkv * D, H, cfg.qkv_bias)
        qlinear(p + ".self_attn.v_proj", Hkv * D, H, cfg.qkv_bias)
        qlinear(p + ".self_attn.o_proj", H, Hq * D)
        qlinear(p + ".mlp.gate_proj", F, H)
        qlinear(p + ".mlp.up_proj", F, H)
        qlinear(p + ".mlp.down_proj", H, F)
        norm(p + ".input_layernorm.weight")
        norm(p + ".post_attention_layernorm.weight")
        if cfg.model_type == "gemma2":
            norm(p + ".pre_feedforward_layernorm.weight")
            norm(p + ".post_feedforward_layernorm.weight")
    norm("model.norm.weight")
    if not (cfg.tie_word_embeddings or cfg.model_type == "gemma2"):
        qlinear("lm_head", V, H)
    return out


def truncated(cfg: ModelConfig, num_layers: int) -> ModelConfig:
    """The same architecture cut to its first ``num_layers`` layers (the draft of the 1B configuration)."""
    import dataclasses
    return dataclasses.replace(cfg, num_hidden_layers=num_layers)


_LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                   "original_max_position_embeddings": 8192}
_LLAMA32_SCALING = dict(_LLAMA3_SCALING, factor=32.0)

PRESETS: Dict[str, ModelConfig] = {
    # the five benchmark architectures
    "llama-3.2-1b": ModelConfig("llama", 2048, 16, 32, 8, 64, 8192, 128256, 4, 64, 1e-5, 500000.0, False,
                                _LLAMA32_SCALING, True),
    "llama-3.1-8b": ModelConfig("llama", 4096, 32, 32, 8, 128, 14336, 128256, 4, 64, 1e-5, 500000.0, False,
                                _LLAMA3_SCALING, False),
    "qwen2.5-7b": ModelConfig("qwen2", 3584, 28, 28, 4, 128, 18944, 152064, 8, 32, 1e-6, 1000000.0, False, None, False,
                              qkv_bias=True),
    "gemma-2-9b": ModelConfig("gemma2", 3584, 42, 16, 8, 256, 14336, 256000, 4, 128, 1e-6, 10000.0, False, None, True,
                              50.0, 30.0, 256.0, 4096),
    "llama-3-70b": ModelConfig("llama", 8192, 80, 64, 8, 128, 28672, 128256, 4, 64, 1e-5, 500000.0, False, None, False),
    # the 70B layer shapes with 8 of the 80 layers: a tensor-parallel parity case that loads in seconds
    "llama-3-70b-8l": ModelConfig("llama", 8192, 8, 64, 8, 128, 28672, 128256, 4, 64, 1e-5, 500000.0, False, None, False),
    # small shapes for parity tests (every code path of the big ones, seconds on one CPU core)
    "tiny-llama": ModelConfig("llama", 256, 2, 8, 2, 64, 512, 1024, 4, 64, 1e-5, 500000.0, False, _LLAMA3_SCALING, True),
    "tiny-llama-d128": ModelConfig("llama", 512, 2, 4, 1, 128, 1024, 2048, 4, 64, 1e-5, 10000.0, False, None, False),
    # hidden 2048: the row-wise kernels' register-resident path and split-K partials at a real row width
    "tiny-llama-h2048": ModelConfig("llama", 2048, 1, 16, 4, 128, 2048, 1024, 4, 64, 1e-5, 500000.0, False, None, False),
    # a wide MLP (208 gate_up tiles): the GEMM keeps two tiles per CTA and fuses the gated activation into its epilogue
    "tiny-llama-wide": ModelConfig("llama", 128, 1, 2, 1, 64, 13312, 512, 4, 64, 1e-5, 10000.0, False, None, False),
    "tiny-qwen2": ModelConfig("qwen2", 448, 2, 7, 1, 64, 1024, 1536, 8, 32, 1e-6, 1000000.0, False, None, False,
                              qkv_bias=True),
    "tiny-gemma2": ModelConfig("gemma2", 512, 2, 4, 2, 256, 1024, 2048, 4, 128, 1e-6, 10000.0, False, None, True,
                               50.0, 30.0, 256.0, 48),
}
