"""kc_quantized_matmul_static: the quantised matmul whose split-K workspace is a fixed device array of the library.

Collected last (file name) so that it also runs after every other GPU test has used the same context, kernels and
weights; it passes alone as well (`pytest tests/test_zz_no_alloc.py -m gpu`). Everything goes through the C ABI. The
bar is bit equality with kc_quantized_matmul, which shares the kernels and the order of the fp32 additions.
"""
import pytest
import torch

from kiln_b200 import _lib as L
from kiln_b200 import api
from tests.test_gpu_qlinear import acts, make

pytestmark = pytest.mark.gpu

LIMIT = 16 << 20


def buffers(m, k, n, seed):
    rows = (m + 15) // 16 * 16
    xp = torch.zeros(rows, k, dtype=torch.bfloat16, device="cuda")
    xp[:m] = acts(m, k, seed).cuda()
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    return xp, y


def test_limit_is_exported():
    assert L.lib().kc_static_scratch_bytes() == LIMIT


@pytest.mark.parametrize("n,k,bits,group,m", [
    (1024, 4096, 4, 64, 192),     # split along K: partials go through the static array (8 x 192 x 1024 fp32 = 6 MiB)
    (1024, 4096, 4, 64, 600),     # two launches; the first one's partials are exactly 16 MiB = the limit
    (512, 2048, 8, 32, 1),        # decode row, 8-bit
    (9600, 256, 4, 64, 40),       # enough tiles that K is not split: no scratch used
])
def test_two_calls_in_a_row_match_the_allocating_entry_point(ctx, n, k, bits, group, m):
    p, s, b = make(n, k, bits, group, 3)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), bits, group)
    xa, ya = buffers(m, k, n, 10)
    xb, yb = buffers(m, k, n, 11)
    # set-up call (first use on the device resolves the array and the kernel attributes), then measure
    qw.matmul_static(xa, m, ya)
    ctx.sync()
    ya.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    qw.matmul_static(xa, m, ya)       # two calls back to back on the context's stream: the second overwrites the
    qw.matmul_static(xb, m, yb)       # array only after the first one's reduction has read it (stream order)
    ctx.sync()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before, "the static entry point must not take device memory"
    want_a = qw.matmul(xa[:m])
    want_b = qw.matmul(xb[:m])
    assert torch.equal(ya.view(torch.int16), want_a.view(torch.int16))
    assert torch.equal(yb.view(torch.int16), want_b.view(torch.int16))
    assert not torch.equal(ya.view(torch.int16), yb.view(torch.int16))
    assert ctx.device_status() == 0
    qw.close()


def test_request_beyond_the_array_is_rejected_before_any_launch(ctx):
    n, k, m = 2048, 4096, 512                      # 8 splits x 512 rows x 2048 features x 4 B = 32 MiB
    p, s, b = make(n, k, 4, 64, 4)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), 4, 64)
    xp, y = buffers(m, k, n, 12)
    launches = ctx.launch_count()
    rc = L.lib().kc_quantized_matmul_static(ctx._h, qw._h, xp.data_ptr(), m, y.data_ptr())
    assert rc == L.KC_ERR_UNSUPPORTED
    msg = L.lib().kc_last_error().decode()
    assert "exceed the static scratch of 16777216 bytes" in msg
    assert ctx.launch_count() == launches
    ctx.sync()
    assert bool(torch.isnan(y.float()).all())      # nothing was written
    # half the rows fit exactly, and the allocating entry point takes the full request
    y2 = torch.empty(256, n, dtype=torch.bfloat16, device="cuda")
    qw.matmul_static(xp, 256, y2)
    ctx.sync()
    full = qw.matmul(xp[:m])
    assert torch.equal(y2.view(torch.int16), full[:256].view(torch.int16))
    qw.close()


def test_bad_arguments(ctx):
    p, s, b = make(256, 256, 4, 64, 5)
    qw = api.QuantizedWeight(ctx, p.cuda(), s.cuda(), b.cuda(), 4, 64)
    xp, y = buffers(4, 256, 256, 13)
    lib = L.lib()
    assert lib.kc_quantized_matmul_static(ctx._h, qw._h, None, 4, y.data_ptr()) == L.KC_ERR_INVALID
    assert lib.kc_quantized_matmul_static(ctx._h, qw._h, xp.data_ptr(), 0, y.data_ptr()) == L.KC_ERR_INVALID
    assert lib.kc_quantized_matmul_static(ctx._h, qw._h, xp.data_ptr() + 2, 4, y.data_ptr()) == L.KC_ERR_INVALID
    assert "16-byte" in lib.kc_last_error().decode()
    qw.close()
