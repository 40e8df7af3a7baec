"""An independent torch-CPU statement of the verify path's arithmetic, written from the reference's op graph
(crates/kiln-models/src/nn.rs) and NOT from oracle/kiln_oracle.cpp, so that the two can be held against each other.

It keeps a contiguous per-sequence K/V history (the reference's gather result, crates/kiln-engine/src/paged.rs:191-225)
instead of pools, computes every fused op in fp32 with one rounding to bf16 at its output, and every composed op
(adds, multiplies, the gelu chain, the Gemma softcap attention) one bf16 rounding per op, as MLX evaluates them.
Nothing in the product imports this file.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

BF = torch.bfloat16


def r(x: torch.Tensor) -> torch.Tensor:
    """One rounding to bf16, carried on in fp32."""
    return x.to(BF).float()


def dequant(packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group: int) -> torch.Tensor:
    """q * scale + bias in float64 (exact), mlx affine layout: element j of a row in bits [bits*(j % per), +bits) of word j // per."""
    per = 32 // bits
    u = packed.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(per, dtype=torch.int64) * bits
    q = ((u.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)).reshape(packed.shape[0], -1).double()
    s = scales.double().repeat_interleave(group, dim=1)
    b = biases.double().repeat_interleave(group, dim=1)
    return q * s + b


def quantized_matmul(x: torch.Tensor, packed, scales, biases, bits: int, group: int, tile_class: bool) -> torch.Tensor:
    """Linear::forward (nn.rs:79-102): x . dequant(W)^T accumulated wide, one rounding to bf16.
    tile_class: the weights are rounded to bf16 before the product (MLX's dequantise-then-matmul kernels); otherwise they
    enter at full precision (its row-vector kernels)."""
    w = dequant(packed, scales, biases, bits, group)
    if tile_class:
        w = w.float().to(BF).double()
    return (x.double() @ w.t()).float().to(BF)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """fast::rms_norm (crates/kiln-mlx/src/fast.rs:36-41): fp32 inside, one rounding."""
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (w.float() * (xf * inv)).to(BF)


def rope_inv_freq(cfg) -> torch.Tensor:
    """Rope::new (nn.rs:1409-1477): base ** (arange(0, D, 2) / D) in fp32, llama3 / linear scaling; returns 1 / freqs."""
    D = cfg.head_dim
    expo = torch.arange(0, D, 2, dtype=torch.float32) / float(D)
    freqs = torch.pow(torch.tensor(cfg.rope_theta, dtype=torch.float32), expo)
    sc = cfg.rope_scaling or {}
    kind = sc.get("rope_type", sc.get("type"))
    if kind == "llama3":
        factor, lo, hi = float(sc["factor"]), float(sc["low_freq_factor"]), float(sc["high_freq_factor"])
        old = float(sc["original_max_position_embeddings"])
        wl = torch.tensor(2.0 * math.pi, dtype=torch.float32) * freqs
        low_wl, high_wl = torch.tensor(old / lo, dtype=torch.float32), torch.tensor(old / hi, dtype=torch.float32)
        f = torch.where(wl > low_wl, freqs * factor, freqs)
        smooth = (old / wl - lo) / (hi - lo)
        f = torch.where((wl > high_wl) & (wl < low_wl), f / ((1.0 - smooth) / factor + smooth), f)
        freqs = f
    inv = 1.0 / freqs
    if kind == "linear":
        inv = inv / float(sc["factor"])
    return inv.float()


def rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, traditional: bool) -> torch.Tensor:
    """fast::rope (fast.rs:45-104) on x [n, heads, D] bf16 at absolute positions pos [n]: fp32 inside, one rounding."""
    n, h, D = x.shape
    ang = pos.float().unsqueeze(-1) * inv_freq.unsqueeze(0)             # [n, D/2]
    cs, sn = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)   # [n, 1, D/2]
    xf = x.float()
    if traditional:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * cs - b * sn, a * sn + b * cs), dim=-1).reshape(n, h, D)
    else:
        a, b = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat((a * cs - b * sn, a * sn + b * cs), dim=-1)
    return out.to(BF)


def silu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """multiply(multiply(gate, sigmoid(gate)), up): three bf16 ops (nn.rs:284-294)."""
    gf = g.float()
    s = r(torch.sigmoid(gf))
    return r(r(gf * s) * u.float()).to(BF)


def gelu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """gelu_approx(gate) * up, op for op with weak (bf16) scalars (nn.rs:221-235)."""
    x = g.float()
    c = lambda v: float(torch.tensor(v, dtype=torch.float32).to(BF).float())
    cube = r(x * x * x)
    inner = r(x + r(c(0.044715) * cube))
    scaled = r(c(math.sqrt(2.0 / math.pi)) * inner)
    gate = r(1.0 + r(torch.tanh(scaled)))
    act = r(r(c(0.5) * x) * gate)
    return r(act * u.float()).to(BF)


def sdpa_fused(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, q_pos: torch.Tensor, window: int = 0) -> torch.Tensor:
    """fast::scaled_dot_product_attention (fast.rs:342-367) with the bottom-right causal mask of nn.rs:801-805:
    q [L, Hq, D], k/v [S, Hkv, D] (key j at absolute position j), fp32 softmax, one rounding of the output."""
    L, Hq, D = q.shape
    S, Hkv, _ = k.shape
    g = Hq // Hkv
    kk = k.float().repeat_interleave(g, dim=1)
    vv = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("lhd,shd->hls", q.float() * scale, kk)
    keys = torch.arange(S).view(1, 1, S)
    qp = q_pos.view(1, L, 1)
    keep = keys <= qp
    if window > 0:
        keep &= keys > qp - window
    s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hls,shd->lhd", p, vv).to(BF)


def sdpa_softcap(q, k, v, scale: float, cap: float, q_pos, window: int = 0) -> torch.Tensor:
    """Attention::manual_softcap_attention (nn.rs:497-580): every op rounds to bf16; softmax is precise (fp32 inside)."""
    L, Hq, D = q.shape
    S, Hkv, _ = k.shape
    g = Hq // Hkv
    sc = float(torch.tensor(scale, dtype=torch.float32).to(BF).float())
    capb = float(torch.tensor(cap, dtype=torch.float32).to(BF).float())
    qs = r(q.float() * sc)
    kk = k.float().repeat_interleave(g, dim=1)
    vv = v.float().repeat_interleave(g, dim=1)
    s = r(torch.einsum("lhd,shd->hls", qs, kk))
    s = r(r(torch.tanh(r(s / capb))) * capb)
    keys = torch.arange(S).view(1, 1, S)
    qp = q_pos.view(1, L, 1)
    keep = keys <= qp
    neg = -(2.0 - 2.0 ** -7) * 2.0 ** 127
    s = torch.where(keep, s, torch.tensor(neg))
    if window > 0:   # this repository's own definition (the reference has no window): keys at or before p - window are absent
        s = s.masked_fill(keys <= qp - window, float("-inf"))
    p = r(torch.softmax(s, dim=-1))
    return r(torch.einsum("hls,shd->lhd", p, vv)).to(BF)


def greedy_rows(logits: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """sample_from_row + greedy Sampler (engine.rs:879-901, sampler.rs:100-104): argmax of bf16(logits - bf16(logsumexp)),
    lowest index on ties; normalize = False is the draft lane's raw argmax (draft.rs:379-381)."""
    x = logits.float()
    if normalize:
        lse = torch.logsumexp(x.double(), dim=-1, keepdim=True).float().to(BF).float()
        x = (x - lse).to(BF).float()
    mx = x.max(dim=-1, keepdim=True).values
    idx = torch.arange(x.shape[-1]).expand_as(x)
    return torch.where(x == mx, idx, torch.full_like(idx, x.shape[-1])).min(dim=-1).values


class TorchRefModel:
    """CausalLm::forward_step (nn.rs:1303-1388) over per-sequence contiguous histories."""

    def __init__(self, cfg, tensors: Dict[str, torch.Tensor], tile_class: bool):
        self.cfg, self.t, self.tile = cfg, {k: v.cpu() for k, v in tensors.items()}, tile_class
        self.gemma = cfg.model_type == "gemma2"
        self.inv_freq = rope_inv_freq(cfg)
        self.scale = (1.0 / math.sqrt(cfg.query_pre_attn_scalar)) if (self.gemma and cfg.query_pre_attn_scalar > 0) \
            else float(torch.tensor(cfg.head_dim ** -0.5, dtype=torch.float64).float())
        self.hist: Dict[int, List[Optional[torch.Tensor]]] = {}

    def _lin(self, x, prefix):
        t = self.t
        y = quantized_matmul(x, t[prefix + ".weight"], t[prefix + ".scales"], t[prefix + ".biases"], self.cfg.bits,
                             self.cfg.group_size, self.tile)
        if prefix + ".bias" in t:
            y = (y.float() + t[prefix + ".bias"].float()).to(BF)
        return y

    def _norm(self, x, name):
        w = self.t[name]
        if self.gemma:
            w = (1.0 + w.float()).to(BF)
        return rms_norm(x, w, self.cfg.rms_norm_eps)

    def forward_step(self, ids: List[int], seqs, seq_keys: List[int]) -> Optional[torch.Tensor]:
        """seqs: objects with len / offset / sample_rows; seq_keys: a stable id per sequence (its history key)."""
        cfg, t = self.cfg, self.t
        H, D, Hq, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        idt = torch.tensor(ids, dtype=torch.int64)
        emb = dequant(t["model.embed_tokens.weight"][idt], t["model.embed_tokens.scales"][idt],
                      t["model.embed_tokens.biases"][idt], cfg.bits, cfg.group_size).float().to(BF)
        h = emb
        if self.gemma:
            h = (h.float() * float(torch.tensor(math.sqrt(H), dtype=torch.float32).to(BF).float())).to(BF)
        pos = torch.cat([torch.arange(s.offset, s.offset + s.len) for s in seqs])
        for l in range(cfg.num_hidden_layers):
            p = f"model.layers.{l}"
            normed = self._norm(h, p + ".input_layernorm.weight")
            q = self._lin(normed, p + ".self_attn.q_proj").view(-1, Hq, D)
            k = self._lin(normed, p + ".self_attn.k_proj").view(-1, Hkv, D)
            v = self._lin(normed, p + ".self_attn.v_proj").view(-1, Hkv, D)
            q = rope(q, pos, self.inv_freq, cfg.rope_traditional)
            k = rope(k, pos, self.inv_freq, cfg.rope_traditional)
            outs, row = [], 0
            window = cfg.sliding_window if (cfg.sliding_window > 0 and l % 2 == 0) else 0
            for s, key in zip(seqs, seq_keys):
                hist = self.hist.setdefault(key, [None] * cfg.num_hidden_layers)
                kk, vv = k[row: row + s.len], v[row: row + s.len]
                if hist[l] is None:
                    assert s.offset == 0
                    hist[l] = (kk.clone(), vv.clone())
                else:
                    hk, hv = hist[l]
                    hist[l] = (torch.cat((hk[: s.offset], kk)), torch.cat((hv[: s.offset], vv)))   # rollback = overwrite
                hk, hv = hist[l]
                qp = pos[row: row + s.len]
                if self.gemma:
                    o = sdpa_softcap(q[row: row + s.len], hk, hv, self.scale, cfg.attn_logit_softcapping, qp, window)
                else:
                    o = sdpa_fused(q[row: row + s.len], hk, hv, self.scale, qp, window)
                outs.append(o.reshape(s.len, Hq * D))
                row += s.len
            attn = self._lin(torch.cat(outs), p + ".self_attn.o_proj")
            if self.gemma:
                attn = self._norm(attn, p + ".post_attention_layernorm.weight")
                h = (h.float() + attn.float()).to(BF)
                x = self._norm(h, p + ".pre_feedforward_layernorm.weight")
            else:
                h = (h.float() + attn.float()).to(BF)
                x = self._norm(h, p + ".post_attention_layernorm.weight")
            g, u = self._lin(x, p + ".mlp.gate_proj"), self._lin(x, p + ".mlp.up_proj")
            a = gelu_mul(g, u) if self.gemma else silu_mul(g, u)
            m = self._lin(a, p + ".mlp.down_proj")
            if self.gemma:
                m = self._norm(m, p + ".post_feedforward_layernorm.weight")
            h = (h.float() + m.float()).to(BF)
        rows, row = [], 0
        for s in seqs:
            rows += list(range(row + s.len - s.sample_rows, row + s.len))
            row += s.len
        if not rows:
            return None
        hs = self._norm(h[torch.tensor(rows)], "model.norm.weight")
        head = "model.embed_tokens" if (self.gemma or cfg.tie_word_embeddings) else "lm_head"
        logits = self._lin(hs, head)
        if self.gemma and cfg.final_logit_softcapping > 0:
            cap = float(torch.tensor(cfg.final_logit_softcapping, dtype=torch.float32).to(BF).float())
            logits = r(r(torch.tanh(r(logits.float() / cap))) * cap).to(BF)
        return logits
