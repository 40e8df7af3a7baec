"""Affine-dequant GEMM (kc_quantized_matmul) against the CPU oracle.

Mirrors the reference's use of quantized_matmul (crates/kiln-models/src/nn.rs:79-102) and its
row-stability probe (nn.rs:301-327): row r of Y(M) must carry the bits of Y(1).
Tolerance is the north-star logits bar applied per layer: max-abs <= 2e-2, cosine >= 0.9999.
"""
import pytest
import torch

from kiln_b200 import api
from kiln_b200.synth import quantize_affine
from oracle import oracle as O
from tests.conftest import cosine, parity

pytestmark = pytest.mark.gpu

MAX_ABS, MIN_COS = 2e-2, 0.9999


def make(n, k, bits, group, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.empty(n, k).normal_(0, 0.02, generator=g)
    # outlier-heavy values like the reference's kernel probes (crates/kiln-engine/tests/paged_attn.rs:58-70)
    w.view(-1)[::97] *= 8.0
    return quantize_affine(w, bits, group)


def acts(m, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.empty(m, k).normal_(0, 1.0, generator=g)
    x.view(-1)[::97] *= 16.0
    return x.to(torch.bfloat16)


CASES = [
    # (N, K, bits, group, M)
    (256, 256, 4, 64, 5),          # tiny: one k-split
    (200, 512, 4, 64, 17),         # N not a multiple of the 128-row tile
    (384, 1024, 4, 32, 33),        # two groups per k-block
    (256, 1024, 4, 128, 6),        # a group spans two k-blocks
    (256, 512, 8, 32, 48),         # 8-bit
    (256, 448, 8, 64, 7),          # K = 7 k-blocks
    (1024, 4096, 4, 64, 192),      # the 8B attention-output shape at verify width: split-K engaged
    (2048, 2048, 4, 64, 320),      # two accumulator tiles (M > 256)
    (512, 2048, 4, 64, 1),         # decode row
    (53248, 256, 8, 32, 100),      # 416 tiles of 8-bit records at 100 rows: four tiles per CTA do not fit shared memory
]


@pytest.mark.parametrize("n,k,bits,group,m", CASES)
def test_matches_oracle(ctx, n, k, bits, group, m):
    p, s, b = make(n, k, bits, group, 1)
    x = acts(m, k, 2)
    O.set_weight_class(1)      # the tensor-core kernel's arithmetic class: w = bf16(q * scale + bias) first
    want = O.quantized_matmul(x, p, s, b, bits, group)
    O.set_weight_class(0)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), bits, group)
    got = qw.matmul(x.cuda()).cpu()
    # 2e-2 flat below magnitude 4; above it one bf16 spacing of the value is added (outputs here reach 20+)
    assert parity(f"qlinear {n}x{k} w{bits}g{group} rows {m}", got, want, MAX_ABS, MIN_COS)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("n,k,bits,group", [(1024, 4096, 4, 64), (256, 512, 8, 32), (4096, 1024, 4, 128)])
def test_rows_do_not_depend_on_batch_width(ctx, n, k, bits, group):
    """probe_row_stability (nn.rs:301-327) widened: every row of Y(M) is bit-identical to its M=1 result."""
    p, s, b = make(n, k, bits, group, 3)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), bits, group)
    x = acts(320, k, 4).cuda()
    ref_rows = {r: qw.matmul(x[r:r + 1]).cpu() for r in (0, 1, 5, 31, 191, 319)}
    for m in (2, 5, 6, 32, 192, 320):
        y = qw.matmul(x[:m]).cpu()
        for r, want in ref_rows.items():
            if r < m:
                assert torch.equal(y[r:r + 1].view(torch.int16), want.view(torch.int16)), f"row {r} differs at M={m}"


STREAM_CASES = [
    # (N, K, bits, group, M): the weight-streaming lane, at most 8 rows
    (256, 256, 4, 64, 1),          # one k-split
    (200, 512, 4, 64, 5),          # N not a multiple of the 128-row tile
    (384, 1024, 4, 32, 8),         # two groups per k-block
    (256, 1024, 4, 128, 3),        # a group spans two k-blocks
    (256, 512, 8, 32, 8),          # 8-bit
    (256, 448, 8, 64, 7),          # K = 7 k-blocks: uneven k-splits
    (1024, 4096, 4, 64, 6),        # the 8B attention-output shape: several pieces per tile
    (28672, 4096, 4, 64, 8),       # the 8B gate_up shape
    (4099, 2048, 4, 64, 2),        # a ragged last tile
    (640, 14336, 4, 64, 4),        # the 8B down-projection depth: a tile's k-blocks spread over many CTAs
    (128256, 2048, 4, 64, 1),      # the 1B head: runs that cross two tile boundaries
]


@pytest.mark.parametrize("n,k,bits,group,m", STREAM_CASES)
def test_stream_lane_matches_oracle(ctx, n, k, bits, group, m):
    """kc_quantized_matmul_stream is of MLX's row-vector class (scale and bias applied per group to fp32 sums of
    x q and of x), the oracle's class 0; against the tensor-core lane (weights rounded to bf16 first) the distance is
    that of the two classes."""
    p, s, b = make(n, k, bits, group, 5)
    x = acts(m, k, 6)
    O.set_weight_class(0)
    want = O.quantized_matmul(x, p, s, b, bits, group)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), bits, group)
    got = qw.matmul_stream(x.cuda()).cpu()
    assert parity(f"stream lane {n}x{k} w{bits}g{group} rows {m}", got, want, MAX_ABS, MIN_COS)
    tensor = qw.matmul(x.cuda()).cpu()
    # two arithmetic classes apart: the distance is printed, and held to what the oracle's own two classes differ by on
    # the same inputs (plus one bf16 spacing of the largest value for the kernels' accumulation orders)
    O.set_weight_class(1)
    want_tile = O.quantized_matmul(x, p, s, b, bits, group)
    O.set_weight_class(0)
    class_gap = float((want.float() - want_tile.float()).abs().max())
    spacing = 2.0 ** (torch.floor(torch.log2(want.float().abs().max())) - 7)
    parity(f"stream lane vs tensor lane {n}x{k} w{bits}g{group} rows {m}", got, tensor, 1e9, MIN_COS)
    gap = float((got.float() - tensor.float()).abs().max())
    print(f"oracle class 0 vs class 1: max-abs {class_gap:.4g}; lanes: {gap:.4g}")
    assert gap <= class_gap + 2 * float(spacing)
    assert cosine(got, tensor) >= MIN_COS
    assert ctx.device_status() == 0


GEMV_CASES = [
    # (N, K, bits, group, M): the small-weight lane of the same arithmetic
    (256, 256, 4, 64, 1),
    (200, 512, 4, 64, 5),          # N not a multiple of the 128-row tile
    (384, 1024, 4, 32, 8),         # two groups per k-block
    (256, 1024, 4, 128, 3),        # a group spans two k-blocks
    (256, 512, 8, 32, 8),          # 8-bit
    (256, 448, 8, 64, 7),          # K = 7 k-blocks: uneven runs
    (3072, 2048, 4, 64, 1),        # the 1B qkv shape
    (2048, 2048, 4, 64, 4),        # the 1B attention-output shape
    (16384, 2048, 4, 64, 1),       # the 1B gate_up shape: two runs per tile
    (2048, 8192, 4, 64, 8),        # the 1B down-projection depth: eight runs of 16 k-blocks
    (4099, 2048, 4, 64, 2),        # a ragged last tile
]


@pytest.mark.parametrize("n,k,bits,group,m", GEMV_CASES)
def test_small_weight_lane_matches_oracle_and_the_streaming_lane(ctx, n, k, bits, group, m):
    """kc_quantized_matmul_gemv against the oracle's row-vector class, and against the streaming kernel of the same
    class (they differ only in where a tile's k-blocks are cut, i.e. in fp32 summation order)."""
    p, s, b = make(n, k, bits, group, 15)
    x = acts(m, k, 16)
    O.set_weight_class(0)
    want = O.quantized_matmul(x, p, s, b, bits, group)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), bits, group)
    got = qw.matmul_gemv(x.cuda()).cpu()
    assert parity(f"small-weight lane {n}x{k} w{bits}g{group} rows {m}", got, want, MAX_ABS, MIN_COS)
    stream = qw.matmul_stream(x.cuda()).cpu()
    spacing = 2.0 ** (torch.floor(torch.log2(want.float().abs().max())) - 7)
    assert float((got.float() - stream.float()).abs().max()) <= 2 * float(spacing)
    # a row's bits do not depend on how many rows ride the call
    if m > 1:
        one = qw.matmul_gemv(x[:1].cuda()).cpu()
        assert torch.equal(one.view(torch.int16), got[:1].view(torch.int16))
    assert ctx.device_status() == 0


def test_small_weight_lane_refuses_a_shape_it_cannot_hold(ctx):
    """224 k-blocks would need more than eight runs of what shared memory holds: the entry point says so."""
    p, s, b = make(640, 14336, 4, 64, 3)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), 4, 64)
    message = None
    try:
        qw.matmul_gemv(acts(2, 14336, 4).cuda())
    except api.KcError as err:     # only the text is kept: a stored traceback would keep the weight alive past its context
        message = str(err)
    assert message and "does not fit" in message


def test_stream_lane_rows_do_not_depend_on_row_count(ctx):
    """Within the lane a row's bits do not depend on how many rows ride the call (1..8)."""
    p, s, b = make(1024, 4096, 4, 64, 7)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), 4, 64)
    x = acts(8, 4096, 8).cuda()
    full = qw.matmul_stream(x).cpu()
    for m in (1, 2, 3, 5, 7):
        y = qw.matmul_stream(x[:m]).cpu()
        assert torch.equal(y.view(torch.int16), full[:m].view(torch.int16))
    one = qw.matmul_stream(x[5:6]).cpu()
    assert torch.equal(one.view(torch.int16), full[5:6].view(torch.int16))
    with pytest.raises(api.KcError, match="m = 9"):
        qw.matmul_stream(acts(9, 4096, 9).cuda())
