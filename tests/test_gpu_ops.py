"""Row-wise ops and sampling kernels against the CPU oracle / plain restatements."""
import numpy as np
import pytest
import torch

from kiln_b200 import api
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,dim", [(1, 256), (7, 2048), (192, 4096), (3, 3584)])
def test_rms_norm(ctx, rows, dim):
    g = torch.Generator().manual_seed(rows * 1000 + dim)
    x = torch.empty(rows, dim).normal_(0, 1.5, generator=g).to(torch.bfloat16)
    w = torch.empty(dim).normal_(1.0, 0.1, generator=g).to(torch.bfloat16)
    want = O.rms_norm(x, w, 1e-5)
    got = api.rms_norm(ctx, x.cuda(), w.cuda(), 1e-5).cpu()
    # fp32 inside, one bf16 rounding: at most one bf16 ulp apart (summation order differs)
    diff = (got.float() - want.float()).abs()
    assert float((diff / want.float().abs().clamp_min(1e-3)).max()) <= 2 ** -7


def test_greedy_rows_match_oracle_and_break_ties_low(ctx):
    g = torch.Generator().manual_seed(3)
    logits = torch.empty(9, 128256).normal_(0, 2.0, generator=g).to(torch.bfloat16)
    # an exact tie in the raw logits and a tie created only by the logprob rounding
    logits[1, 70000] = logits[1].max() + 1
    logits[1, 300] = logits[1, 70000]
    logits[2, 5] = 40.0
    logits[2, 90000] = 40.125   # bf16(40.125 - lse) can equal bf16(40 - lse)
    want_n = O.greedy_rows(logits, True)
    want_r = O.greedy_rows(logits, False)
    got_n = api.greedy_rows(ctx, logits.cuda(), True).cpu().numpy().astype(np.uint32)
    got_r = api.greedy_rows(ctx, logits.cuda(), False).cpu().numpy().astype(np.uint32)
    assert np.array_equal(got_n, want_n)
    assert np.array_equal(got_r, want_r)
    assert got_n[1] == 300 and got_r[1] == 300


def test_verify_accept_walk(ctx):
    """engine.rs:2336-2366 on four segments: full agreement (bonus), first-row mismatch, mid mismatch, plain decode."""
    rows = torch.tensor([5, 6, 7, 8,   9, 1, 1,   4, 4, 9, 9,   3], dtype=torch.int32).cuda()
    row_off = torch.tensor([0, 4, 7, 11], dtype=torch.int32).cuda()
    draft = torch.tensor([5, 6, 7,   2, 1,   4, 4, 8,  0], dtype=torch.int32).cuda()
    d_off = torch.tensor([0, 3, 5, 8], dtype=torch.int32).cuda()
    d_len = torch.tensor([3, 2, 3, 0], dtype=torch.int32).cuda()
    com, ncom, nacc = api.verify_accept(ctx, rows, row_off, draft, d_off, d_len, 4)
    assert ncom.cpu().tolist() == [4, 1, 3, 1]
    assert nacc.cpu().tolist() == [3, 0, 2, 0]
    com = com.cpu()
    assert com[0].tolist() == [5, 6, 7, 8] and com[1, 0].item() == 9 and com[2, :3].tolist() == [4, 4, 9] and com[3, 0].item() == 3


def test_rope_kv_write_and_block_io(ctx):
    """RoPE at per-sequence offsets + pool write (nn.rs:760-769, paged.rs:147-187), then the SSD payload
    order of read_block_bytes (paged.rs:280-304) and copy_block (paged.rs:230-250)."""
    hd, heads, kvh, bs = 64, 4, 2, 16
    spec = api.KvSpec(2, kvh, hd, 6, bs)
    kv = api.PagedKv(ctx, spec)
    seqs = [api.SeqStep(5, 14, 5, [4, 1]), api.SeqStep(1, 3, 1, [2])]
    n = 6
    g = torch.Generator().manual_seed(5)
    qkv = torch.empty(n, (heads + 2 * kvh) * hd).normal_(0, 1, generator=g).to(torch.bfloat16)
    inv = (10000.0 ** (-torch.arange(0, hd, 2).float() / hd))
    q = api.rope_kv_write(ctx, kv, 1, qkv.cuda(), inv.cuda(), heads, seqs).cpu()
    pos = torch.tensor([14, 15, 16, 17, 18, 3]).float()

    def rope(x):  # x [n, h, hd] fp32, split-halves pairing
        th = pos[:, None, None] * inv[None, None, :]
        c, s = th.cos(), th.sin()
        a, b = x[..., : hd // 2], x[..., hd // 2:]
        return torch.cat([a * c - b * s, a * s + b * c], -1)

    x = qkv.float().view(n, heads + 2 * kvh, hd)
    want_q = rope(x[:, :heads]).to(torch.bfloat16)
    want_k = rope(x[:, heads:heads + kvh]).to(torch.bfloat16)
    want_v = x[:, heads + kvh:].to(torch.bfloat16)
    assert float((q.float() - want_q.float()).abs().max()) <= 2 ** -6
    # token at position 15 of sequence 0 lives in block 4 row 15; position 16 in block 1 row 0
    plane = kvh * bs * hd
    blk4 = np.frombuffer(kv.read_block_bytes(4), dtype=np.int16).reshape(2, 2, kvh, bs, hd)   # [layer, K|V, head, row, d]
    blk1 = np.frombuffer(kv.read_block_bytes(1), dtype=np.int16).reshape(2, 2, kvh, bs, hd)
    k15 = torch.from_numpy(blk4[1, 0, :, 15].copy()).view(torch.bfloat16)
    v16 = torch.from_numpy(blk1[1, 1, :, 0].copy()).view(torch.bfloat16)
    assert float((k15.float() - want_k[1].float()).abs().max()) <= 2 ** -6
    assert torch.equal(v16, want_v[2])
    assert not blk4[0].any(), "layer 0 must stay untouched"
    assert plane * 2 * 2 * 2 == kv.bytes_per_block()
    kv.copy_block(4, 5)
    assert kv.read_block_bytes(5) == kv.read_block_bytes(4)
    kv.write_block_bytes(0, kv.read_block_bytes(1))
    assert kv.read_block_bytes(0) == kv.read_block_bytes(1)


def _bf16_neighbours(v: float):
    """The bf16 value at or below v and the next one above it (v > 0)."""
    assert v > 0
    bits = int(torch.tensor(v, dtype=torch.float32).to(torch.bfloat16).view(torch.int16))
    if float(torch.tensor(bits, dtype=torch.int16).view(torch.bfloat16)) > v:
        bits -= 1
    lo, hi = (float(torch.tensor(b, dtype=torch.int16).view(torch.bfloat16)) for b in (bits, bits + 1))
    assert lo <= v < hi
    return lo, hi


def _boundary_rows(vocab: int, n: int, seed: int) -> torch.Tensor:
    """Rows whose logsumexp sits within about 1e-4 of a bf16 rounding boundary (the midpoint of two neighbouring bf16
    values): one low-weight logit is stepped through its bf16 values until the row's float64 logsumexp is as close to
    the midpoint as its spacing allows. A row like this decides whether an fp32 logsumexp rounds the way a double one does."""
    g = torch.Generator().manual_seed(seed)
    rows = []
    while len(rows) < n:
        x = torch.empty(vocab).normal_(0, 2.0, generator=g).to(torch.bfloat16)
        lse = float(torch.logsumexp(x.double(), 0))
        lo, hi = _bf16_neighbours(lse)
        mid = 0.5 * (lo + hi)
        j = int(torch.randint(0, vocab, (1,), generator=g))
        rest = torch.logsumexp(torch.cat((x[:j], x[j + 1:])).double(), 0)
        # candidates for x[j]: the bf16 values in a band 3..7 below the logsumexp (weight e^-3 .. e^-7 of the sum)
        cand = torch.arange(lse - 7.0, lse - 3.0, 2 ** -6).to(torch.bfloat16).unique()
        lses = torch.logaddexp(rest, cand.double())
        best = int((lses - mid).abs().argmin())
        if abs(float(lses[best]) - mid) < 2e-4:
            x[j] = cand[best]
            rows.append(x)
    return torch.stack(rows)


@pytest.mark.parametrize("vocab", [128256, 152064, 256000])
def test_greedy_rows_by_the_thousand(ctx, vocab):
    """4096 random rows per vocabulary size of the benchmark models, plus rows built so that the logsumexp lies next
    to a bf16 rounding boundary: the device's tokens equal the oracle's (double-precision logsumexp) on every row."""
    torch.manual_seed(vocab)
    chunk, total, bad = 512, 4096, 0
    for c in range(total // chunk):
        scale = (0.5, 1.0, 2.0, 4.0)[c % 4]
        x = (torch.randn(chunk, vocab, device="cuda") * scale).to(torch.bfloat16)
        if c == 0:
            x[:, 7] = x.max(dim=1).values           # an exact tie with the row maximum in every row
        got = api.greedy_rows(ctx, x, True).cpu().numpy().astype(np.uint32)
        want = O.greedy_rows(x.cpu(), True)
        bad += int((got != want).sum())
        got_r = api.greedy_rows(ctx, x, False).cpu().numpy().astype(np.uint32)
        assert np.array_equal(got_r, O.greedy_rows(x.cpu(), False))
    assert bad == 0, f"{bad} of {total} rows picked another token than the oracle"
    edge = _boundary_rows(vocab, 24, vocab)
    got = api.greedy_rows(ctx, edge.cuda(), True).cpu().numpy().astype(np.uint32)
    assert np.array_equal(got, O.greedy_rows(edge, True)), "a row next to a logsumexp rounding boundary rounded the other way"


def test_handles_may_outlive_their_context(ctx):
    """The convention is handles first, context last; a garbage-collected host language does not promise an order, so a
    pool or a weight freed after its context must not touch the context's stream (it synchronises the device)."""
    import ctypes as C
    from kiln_b200 import _lib as L
    before = api.live_objects()
    c2 = api.Context(0)
    kv = api.PagedKv(c2, api.KvSpec(layers=1, kv_heads=2, head_dim=64, num_blocks=4, block_size=16))
    p = torch.randint(0, 2 ** 31 - 1, (128, 32), dtype=torch.int32)
    s = torch.full((128, 4), 0.01, dtype=torch.bfloat16)
    qw = api.QuantizedWeight(c2, p.cuda(), s.cuda(), s.cuda(), 4, 64)
    c2._children.discard(kv)
    c2._children.discard(qw)
    L.lib().kc_ctx_destroy(c2._h)            # the context goes first
    c2._h = C.c_void_p()
    kv.close()
    qw.close()
    assert api.live_objects() == before
    assert ctx.device_status() == 0
