"""Pins the CPU oracle (oracle/kiln_oracle.cpp) against an independent torch-CPU implementation (tests/torch_ref.py)
of the same reference graph, op by op and end to end. MLX itself cannot be built or imported where these tests run, so
parity with the reference's own floating-point results stays unpinned; what this file adds is that the oracle is no
longer checked against itself only. Every case prints its raw distance. CPU only.
"""
import numpy as np
import pytest
import torch

from kiln_b200 import api
from kiln_b200.synth import PRESETS, quantize_affine, synth_checkpoint
from oracle import oracle as O
from tests import torch_ref as T

BF = torch.bfloat16


def ulp_gap(a: torch.Tensor, b: torch.Tensor) -> float:
    """Largest |a - b| in units of the bf16 spacing at the larger magnitude of the pair."""
    a, b = a.float(), b.float()
    mag = torch.maximum(a.abs(), b.abs()).clamp_min(2.0 ** -120)
    spacing = torch.exp2(torch.floor(torch.log2(mag)) - 7)
    return float(((a - b).abs() / spacing).max())


@pytest.mark.parametrize("bits,group,n,k,m", [(4, 64, 192, 512, 7), (4, 128, 96, 1024, 3), (4, 32, 130, 256, 5),
                                              (8, 32, 128, 448, 6), (8, 64, 77, 1024, 1)])
@pytest.mark.parametrize("cls", [0, 1])
def test_quantized_matmul(bits, group, n, k, m, cls):
    g = torch.Generator().manual_seed(bits * 1000 + group + n)
    w = torch.empty(n, k).normal_(0, 0.02, generator=g)
    p, s, b = quantize_affine(w, bits, group)
    x = torch.randn(m, k, generator=g).to(BF)
    O.set_weight_class(cls)
    try:
        got = O.quantized_matmul(x, p, s, b, bits, group)
    finally:
        O.set_weight_class(0)
    want = T.quantized_matmul(x, p, s, b, bits, group, tile_class=bool(cls))
    gap = ulp_gap(got, want)
    print(f"qmm w{bits}g{group} {n}x{k} m={m} class {cls}: {gap:.2f} bf16 spacings, max-abs {float((got.float() - want.float()).abs().max()):.3g}")
    # fp32 accumulation order differs from the float64 product: at most one spacing apart, and only where the exact
    # value sits next to a rounding boundary
    assert gap <= 1.0
    assert float((got.float() != want.float()).float().mean()) < 0.02


def test_rms_norm():
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(9, 448, generator=g) * 3).to(BF)
    w = (1 + 0.1 * torch.randn(448, generator=g)).to(BF)
    got, want = O.rms_norm(x, w, 1e-6), T.rms_norm(x, w, 1e-6)
    gap = ulp_gap(got, want)
    print(f"rms_norm: {gap:.2f} bf16 spacings")
    assert gap <= 1.0 and float((got.float() != want.float()).float().mean()) < 0.01


@pytest.mark.parametrize("hq,hkv,d,ctx_len,rows,softcap,window", [
    (8, 2, 64, 70, 5, 0.0, 0), (4, 1, 128, 513, 6, 0.0, 0), (4, 2, 256, 100, 4, 50.0, 0), (4, 2, 256, 100, 4, 50.0, 48),
    (7, 1, 64, 33, 1, 0.0, 0), (8, 8, 64, 40, 3, 0.0, 16)])
def test_paged_attention(hq, hkv, d, ctx_len, rows, softcap, window):
    """The oracle reads K/V through a (shuffled) block table; torch reads the same rows gathered contiguously."""
    bs, nb = 16, 48
    g = torch.Generator().manual_seed(hq * 100 + d + ctx_len)
    okv = O.OracleKv(1, hkv, d, nb, bs)
    total = ctx_len + rows
    nblk = -(-total // bs)
    blocks = torch.randperm(nb, generator=g)[:nblk].tolist()
    k = (torch.randn(total, hkv, d, generator=g) * 0.7).to(BF)
    v = (torch.randn(total, hkv, d, generator=g) * 0.7).to(BF)
    # every 97th value is an outlier, as in the reference's kernel tests (crates/kiln-engine/tests/paged_attn.rs:58-70)
    k.view(-1)[::97] *= 16
    pool = okv.array()
    kb = k.view(torch.int16).numpy().view(np.uint16)
    vb = v.view(torch.int16).numpy().view(np.uint16)
    for pos in range(total):
        pool[0, 0, blocks[pos // bs], :, pos % bs, :] = kb[pos]
        pool[0, 1, blocks[pos // bs], :, pos % bs, :] = vb[pos]
    q = torch.randn(rows, hq, d, generator=g).to(BF)
    scale = d ** -0.5
    got = O.paged_attention(okv, 0, q, [api.SeqStep(rows, ctx_len, rows, blocks)], scale, softcap, window)
    qpos = torch.arange(ctx_len, ctx_len + rows)
    if softcap > 0:
        want = T.sdpa_softcap(q, k, v, scale, softcap, qpos, window)
    else:
        want = T.sdpa_fused(q, k, v, scale, qpos, window)
    want = want.reshape(rows, hq * d)
    err = float((got.float() - want.float()).abs().max())
    cos = float(torch.nn.functional.cosine_similarity(got.float().flatten(), want.float().flatten(), dim=0))
    print(f"attention Hq{hq} Hkv{hkv} D{d} ctx{ctx_len} rows{rows} cap{softcap} win{window}: max-abs {err:.3g}, cosine {cos:.7f}, {ulp_gap(got, want):.2f} spacings")
    # the softcap path rounds to bf16 after every op: a score one spacing off moves a probability, so it is held to the
    # logits bar; the fused path rounds once and must agree to a spacing
    if softcap > 0:
        assert err <= 2e-2 and cos >= 0.9999
    else:
        assert ulp_gap(got, want) <= 1.0 and cos >= 0.99999


@pytest.mark.parametrize("vocab", [1000, 4099])
def test_greedy_rows(vocab):
    g = torch.Generator().manual_seed(vocab)
    x = (torch.randn(64, vocab, generator=g) * 4).to(BF)
    x[5, 17] = x[5].max(); x[5, 900] = x[5].max()            # an exact tie: the lower index wins
    x[6] = x[6, 0]                                           # a constant row
    for norm in (True, False):
        got = torch.from_numpy(O.greedy_rows(x, norm).astype(np.int64))
        assert torch.equal(got, T.greedy_rows(x, norm))


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-llama-d128", "tiny-qwen2", "tiny-gemma2"])
@pytest.mark.parametrize("cls", [0, 1])
def test_forward_step(name, cls):
    """Ragged prefill, a verify step of k + 1 rows with a rollback in between, then a decode row: logits of every
    sampled row from the oracle (paged pools, shuffled tables) and from torch (contiguous histories)."""
    cfg = PRESETS[name]
    ck = synth_checkpoint(cfg, seed=0)
    om = O.OracleModel(cfg, ck)
    bs, nb = 16, 40
    okv = O.OracleKv(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, nb, bs)
    tm = T.TorchRefModel(cfg, ck, tile_class=bool(cls))
    g = torch.Generator().manual_seed(11)
    lens = [61, 23]
    toks = [torch.randint(0, cfg.vocab_size, (n + 12,), generator=g).tolist() for n in lens]
    perm = torch.randperm(nb, generator=g).tolist()
    tables = [perm[:8], perm[8:16]]
    steps = [
        ([api.SeqStep(lens[0], 0, 1, tables[0]), api.SeqStep(lens[1], 0, 1, tables[1])],
         toks[0][:lens[0]] + toks[1][:lens[1]]),
        # verify: 5 rows each; afterwards sequence 0 keeps 2 of them (rollback of 3), sequence 1 keeps all 5
        ([api.SeqStep(5, lens[0], 5, tables[0]), api.SeqStep(5, lens[1], 5, tables[1])],
         toks[0][lens[0]:lens[0] + 5] + toks[1][lens[1]:lens[1] + 5]),
        ([api.SeqStep(4, lens[0] + 2, 4, tables[0]), api.SeqStep(1, lens[1] + 5, 1, tables[1])],
         toks[0][lens[0] + 7:lens[0] + 11] + toks[1][lens[1] + 5:lens[1] + 6]),
    ]
    O.set_weight_class(cls)
    try:
        for i, (seqs, ids) in enumerate(steps):
            got = om.forward_step(api.StepBatch(ids, seqs), okv)
            want = tm.forward_step(ids, seqs, [0, 1])
            err = float((got.float() - want.float()).abs().max())
            cos = float(torch.nn.functional.cosine_similarity(got.float().flatten(), want.float().flatten(), dim=0))
            same_tok = float((torch.from_numpy(O.greedy_rows(got).astype(np.int64)) == T.greedy_rows(want)).float().mean())
            print(f"{name} class {cls} step {i}: max-abs {err:.3g}, cosine {cos:.7f}, greedy tokens equal on {same_tok:.0%} of rows")
            assert err <= 2e-2 and cos >= 0.9999, f"{name} step {i}: oracle vs torch max-abs {err}, cosine {cos}"
    finally:
        O.set_weight_class(0)
