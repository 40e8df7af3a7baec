"""Times single operators of libkiln_cuda.so through the C ABI with CUDA events on the context's stream.

    python -m kiln_b200.opbench qlinear --shape 28672x4096 --rows 192 [--bits 4 --group 64 --iters 20]
    python -m kiln_b200.opbench attention --seqs 32 --context 1400 --rows 6 [--heads 32 --kv-heads 8 --head-dim 128]

Each call warms up, then times `iters` back-to-back launches and prints one line with the mean duration and
the algorithmic throughput (weights read once / K+V read once per sequence). Inputs are synthetic. The qlinear
bench rotates over `--copies` separate copies of the weight (default: enough that they total more than twice the
126 MB L2), so that every launch streams its weights from HBM as it does inside a decode step; `--copies 1` times
the L2-resident case. `--iters 1 --warmup 1 --copies 1` gives a short run suitable for a profiler.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from . import _lib as L
from . import api
from .synth import quantize_affine


def _events(ctx):
    stream = torch.cuda.ExternalStream(ctx.stream)
    return stream, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def bench_qlinear(args) -> dict:
    n, k = (int(v) for v in args.shape.lower().split("x"))
    ctx = api.Context(0)
    base_rows = min(n, 8192)          # quantise a slab and repeat it: the kernel's work does not depend on the values
    w = torch.empty(base_rows, k, device="cuda").normal_(0, 0.02)
    p, s, b = quantize_affine(w, args.bits, args.group)
    reps = -(-n // base_rows)
    p, s, b = (t.repeat(reps, 1)[:n].contiguous() for t in (p, s, b))
    wbytes = n * k * args.bits / 8 + n * (k // args.group) * 4
    copies = args.copies if args.copies > 0 else max(1, int(2 * 126e6 // wbytes) + 1)
    qws = [api.QuantizedWeight(ctx, p, s, b, args.bits, args.group) for _ in range(copies)]
    m = args.rows
    x = torch.randn((m + 15) // 16 * 16, k, device="cuda").to(torch.bfloat16)
    y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    lib = L.lib()
    # the lane: the tensor-core kernel, or (at most 8 rows) the weight-streaming or the small-weight kernel
    entry = {"tensor": lib.kc_quantized_matmul, "stream": lib.kc_quantized_matmul_stream, "gemv": lib.kc_quantized_matmul_gemv}[args.lane]
    for i in range(max(args.warmup, copies)):
        api.check(entry(ctx._h, qws[i % copies]._h, x.data_ptr(), m, y.data_ptr()))
    ctx.sync()
    stream, e0, e1 = _events(ctx)
    e0.record(stream)
    for i in range(args.iters):
        api.check(entry(ctx._h, qws[i % copies]._h, x.data_ptr(), m, y.data_ptr()))
    e1.record(stream)
    ctx.sync()
    us = e0.elapsed_time(e1) * 1e3 / args.iters
    flops = 2.0 * m * n * k
    out = {"op": "qlinear", "lane": args.lane, "N": n, "K": k, "rows": m, "bits": args.bits, "group": args.group, "copies": copies, "us": us,
           "tflops": flops / us / 1e6, "weight_gbs": wbytes / us / 1e3}
    for qw in qws:
        qw.close()
    return out


def bench_attention(args) -> dict:
    ctx = api.Context(0)
    bs = 16
    rng = np.random.default_rng(0)
    lens = rng.integers(max(1, args.context // 2), args.context * 3 // 2 + 1, size=args.seqs) if args.ragged \
        else np.full(args.seqs, args.context)
    nblk = [-(-(int(c) + args.rows) // bs) for c in lens]
    spec = api.KvSpec(layers=1, kv_heads=args.kv_heads, head_dim=args.head_dim, num_blocks=sum(nblk) + 1, block_size=bs)
    kv = api.PagedKv(ctx, spec)
    block = torch.randn(spec.kv_heads * bs * spec.head_dim * 2, dtype=torch.float32).mul_(0.5).to(torch.bfloat16)
    payload = block.view(torch.uint8).numpy().tobytes()
    for blk in range(spec.num_blocks):   # any finite content will do
        kv.write_block_bytes(blk, payload)
    seqs, at = [], 0
    for c, nb in zip(lens, nblk):
        seqs.append(api.SeqStep(args.rows, int(c), args.rows, list(range(at, at + nb))))
        at += nb
    n = args.seqs * args.rows
    q = torch.randn(n, args.heads, args.head_dim, device="cuda").to(torch.bfloat16)
    p = api._PackedStep(api.StepBatch([0] * n, seqs))
    out = torch.empty(n, args.heads * args.head_dim, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    lib = L.lib()
    scale = args.head_dim ** -0.5

    def call():
        api.check(lib.kc_paged_attention(ctx._h, kv._h, 0, q.data_ptr(), n, args.heads, p.seq_arr, p.n_seqs, scale, 0.0, 0,
                                         out.data_ptr()))
    for _ in range(args.warmup):
        call()
    ctx.sync()
    # kc_paged_attention builds its step metadata on every call (it is a single-op convenience entry), so the kernels
    # are timed with the library's own per-launch events rather than around the call
    ctx.profile_read()
    ctx.profile_enable(True)
    for _ in range(args.iters):
        call()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    us = prof["attention"][0] * 1e3 / args.iters
    kv_bytes = float(sum(int(c) + args.rows for c in lens)) * args.kv_heads * args.head_dim * 2 * 2
    return {"op": "attention", "seqs": args.seqs, "mean_context": float(np.mean(lens)), "rows": args.rows, "heads": args.heads,
            "kv_heads": args.kv_heads, "head_dim": args.head_dim, "us": us, "kv_gbs": kv_bytes / us / 1e3,
            "kv_mb": kv_bytes / 1e6}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="op", required=True)
    a = sub.add_parser("qlinear")
    a.add_argument("--shape", required=True, help="out_features x in_features, e.g. 28672x4096")
    a.add_argument("--rows", type=int, default=192)
    a.add_argument("--bits", type=int, default=4)
    a.add_argument("--group", type=int, default=64)
    a.add_argument("--copies", type=int, default=0, help="separate weight copies to rotate over (0: more than 2 x L2 in total)")
    a.add_argument("--lane", choices=["tensor", "stream", "gemv"], default="tensor",
                   help="tensor: kc_quantized_matmul; stream / gemv: the two small-step lanes (at most 8 rows; the time includes the reduction of their partials)")
    b = sub.add_parser("attention")
    b.add_argument("--seqs", type=int, default=32)
    b.add_argument("--context", type=int, default=1400)
    b.add_argument("--rows", type=int, default=6, help="query rows per sequence (k + 1)")
    b.add_argument("--heads", type=int, default=32)
    b.add_argument("--kv-heads", type=int, default=8)
    b.add_argument("--head-dim", type=int, default=128)
    b.add_argument("--ragged", action="store_true", help="contexts uniform in [context/2, 3*context/2]")
    for s in (a, b):
        s.add_argument("--iters", type=int, default=40)
        s.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    r = bench_qlinear(args) if args.op == "qlinear" else bench_attention(args)
    print(" ".join(f"{k}={v:.1f}" if isinstance(v, float) else f"{k}={v}" for k, v in r.items()))


if __name__ == "__main__":
    main()
