"""Operator timings in the format of the reference's benchmark table
(``benchmarks/ops/benchmark_linear_attn.py``: forward and forward+backward milliseconds of
``linear_attention`` over T in {1024, 4096, 16384, 32768}, bf16, H=16, D=64), extended to the
other operators.  Timing: CUDA events around back-to-back calls of the public API, median of
``--reps`` repetitions after warm-up; inputs are larger than L2 from T=4096 up at B=8.

    python benchmarks/benchmark_ops.py [--batch 8] [--op linear_attn|layers|fp32|blhd|simple_la|decoupled_la|varlen|pisa|all]
                                       [--long] [--impl b200|reference [--ref-path DIR]]

``--long`` adds ``simple_la`` at B4 H32 T262144 D128 (8.6 GB per tensor, about 70 GB on the device).
``--impl reference`` times the reference's own Triton operators instead, imported from ``--ref-path``
(an installed copy of the reference package; default ``baseline/_ref`` at the repository root), on the
same GPU with the same inputs and timer.  Its piecewise operator has no backward: that column is nan.
"""
import argparse
import os
import statistics
import sys

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _early(flag, default):
    return sys.argv[sys.argv.index(flag) + 1] if flag in sys.argv[:-1] else default


IMPL = _early("--impl", "b200")
if IMPL == "reference":
    sys.path.insert(0, os.path.abspath(_early("--ref-path", os.path.join(os.path.dirname(_PKG), "baseline", "_ref"))))
else:
    sys.path.insert(0, _PKG)

import torch
import torch.nn.functional as F

from flash_bla.ops.linear_attn.decoupled import decoupled_la
from flash_bla.ops.linear_attn.fused import linear_attention
from flash_bla.ops.linear_attn.varlen import varlen_linear_attention
from flash_bla.ops.piecewise_attn.kernel import piecewise_sparse_attention
from flash_bla.ops.simple_la.fused import simple_la


def timed(fn, reps, inner=4):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(inner):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / inner)
    return statistics.median(out)


def graphed(fn, leaves):
    """``fn`` (a forward + backward) captured once in a CUDA graph; returns the replay callable."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    for x in leaves:
        x.grad = None
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g.replay


def row(name, shape, fwd, fwd_bwd, tokens, nbytes_fwd, nbytes_all):
    print(f"{name:14s} {shape:28s} fwd {fwd:8.4f} ms ({nbytes_fwd / fwd / 1e6:6.0f} GB/s)   fwd+bwd {fwd_bwd:8.4f} ms "
          f"({nbytes_all / fwd_bwd / 1e6:6.0f} GB/s, {tokens / fwd_bwd * 1e3:.3e} tokens/s)", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--op", default="all")
    ap.add_argument("--long", action="store_true")
    ap.add_argument("--graph", action="store_true", help="also time linear_attn fwd+bwd replayed from a CUDA graph")
    ap.add_argument("--lengths", default="1024,4096,16384,32768", help="T values of the linear_attn rows")
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--ref-path", default=None)
    args = ap.parse_args()
    B, H, D = args.batch, args.heads, args.dim
    print(f"# impl={IMPL} package={os.path.dirname(os.path.dirname(sys.modules[linear_attention.__module__].__file__))}")
    if IMPL == "reference":
        import triton
        if hasattr(triton, "set_allocator"):    # the piecewise kernel's tensor descriptors need scratch memory
            triton.set_allocator(lambda size, align, stream: torch.empty(size, dtype=torch.int8, device="cuda"))
    dev, dt = "cuda", torch.bfloat16
    pos = lambda *s: (F.elu(torch.randn(*s, device=dev)) + 1).to(dt).requires_grad_()
    gau = lambda *s: torch.randn(*s, device=dev).to(dt).requires_grad_()

    def both(make_out, leaves, do):
        def fb():
            for x in leaves:
                x.grad = None
            make_out().backward(do)
        with torch.no_grad():
            f = timed(make_out, args.reps)
        if do is None:
            return f, float("nan")
        return f, timed(fb, args.reps)

    if args.op in ("all", "linear_attn"):
        for T in [int(x) for x in args.lengths.split(",")]:
            q, k, v = pos(B, H, T, D), pos(B, H, T, D), gau(B, H, T, D)
            do = torch.randn_like(v)
            P = B * H * T * D * 2
            f, fb = both(lambda: linear_attention(q, k, v), (q, k, v), do)
            row("linear_attn", f"B{B} H{H} T{T} D{D}", f, fb, B * T, 4 * P, 11 * P)
            if args.graph:
                def once():
                    linear_attention(q, k, v).backward(do)
                replay = graphed(once, (q, k, v))
                tg = timed(replay, args.reps)
                print(f"{'':14s} {'  replayed from a CUDA graph':28s} {'':33s}   fwd+bwd {tg:8.4f} ms "
                      f"({11 * P / tg / 1e6:6.0f} GB/s, {B * T / tg * 1e3:.3e} tokens/s)", flush=True)
    if args.op in ("all", "layers"):
        # the reference layers' head dim (32), at their sizes (14 x 14 and 56 x 56 tokens) and at streaming size
        for (b, h, T, d) in ((32, 4, 196, 32), (8, 8, 3136, 32), (B, H, 32768, 32)):
            q, k, v = pos(b, h, T, d), pos(b, h, T, d), gau(b, h, T, d)
            do = torch.randn_like(v)
            P = b * h * T * d * 2
            f, fb = both(lambda: linear_attention(q, k, v), (q, k, v), do)
            row("linear_attn", f"B{b} H{h} T{T} D{d}", f, fb, b * T, 4 * P, 11 * P)
            qr, kr = gau(b, h, T, d), gau(b, h, T, d)
            f, fb = both(lambda: decoupled_la(q, k, qr, kr, v), (q, k, qr, kr, v), do)
            row("decoupled_la", f"B{b} H{h} T{T} D{d}", f, fb, b * T, 6 * P, 16 * P)
    if args.op in ("all", "fp32"):
        # fp32 inputs (the 1e-5 parity case): B2 H4 T1024 D64 as the reference's CPU-runnable configuration, and a
        # streaming-size case
        for (b, h, T, d) in ((2, 4, 1024, 64), (8, 16, 4096, 64)):
            q, k, v = (x.detach().float().requires_grad_() for x in (pos(b, h, T, d), pos(b, h, T, d), gau(b, h, T, d)))
            do = torch.randn_like(v)
            P = b * h * T * d * 4
            f, fb = both(lambda: linear_attention(q, k, v), (q, k, v), do)
            row("linear_attn", f"fp32 B{b} H{h} T{T} D{d}", f, fb, b * T, 4 * P, 11 * P)
    if args.op in ("all", "blhd") and IMPL != "reference":
        # projection-layout inputs (B, L, H, D): the op on them as they are, against the reference layers' route
        # (permute + contiguous into (B, H, L, D), the op, permute back)
        for T in (4096, 32768):
            q, k, v = pos(B, T, H, D), pos(B, T, H, D), gau(B, T, H, D)
            do = torch.randn_like(v)
            P = B * H * T * D * 2
            f, fb = both(lambda: linear_attention(q, k, v, layout="blhd"), (q, k, v), do)
            row("linear_attn", f"(B,L,H,D) in place, T{T}", f, fb, B * T, 4 * P, 11 * P)

            def via_copies():
                qq, kk, vv = (x.permute(0, 2, 1, 3).contiguous() for x in (q, k, v))
                return linear_attention(qq, kk, vv).permute(0, 2, 1, 3).contiguous()
            f, fb = both(via_copies, (q, k, v), do)
            row("linear_attn", f"(B,L,H,D) via permutes, T{T}", f, fb, B * T, 4 * P, 11 * P)
    if args.op in ("all", "simple_la"):
        for (b, h, T, d) in ((4, 32, 32768, 128), (B, H, 32768, D)) + (((4, 32, 262144, 128),) if args.long else ()):
            q, k, v = gau(b, h, T, d), gau(b, h, T, d), gau(b, h, T, d)
            do = torch.randn_like(v)
            P = b * h * T * d * 2
            f, fb = both(lambda: simple_la(q, k, v), (q, k, v), do)
            row("simple_la", f"B{b} H{h} T{T} D{d}", f, fb, b * T, 4 * P, 11 * P)
    if args.op in ("all", "decoupled_la"):
        for T in (4096, 32768):
            q, k, qr, kr, v = pos(B, H, T, D), pos(B, H, T, D), gau(B, H, T, D), gau(B, H, T, D), gau(B, H, T, D)
            do = torch.randn_like(v)
            P = B * H * T * D * 2
            f, fb = both(lambda: decoupled_la(q, k, qr, kr, v), (q, k, qr, kr, v), do)
            row("decoupled_la", f"B{B} H{H} T{T} D{D}", f, fb, B * T, 6 * P, 16 * P)
    if args.op in ("all", "varlen"):
        g = torch.Generator().manual_seed(0)
        lengths = torch.randint(256, 16385, (32,), generator=g)
        cu = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)]).to(torch.int32).to(dev)
        tot, mx = int(lengths.sum()), int(lengths.max())
        q, k, v = pos(tot, H, D), pos(tot, H, D), gau(tot, H, D)
        do = torch.randn_like(v)
        P = tot * H * D * 2
        f, fb = both(lambda: varlen_linear_attention(q, k, v, cu, mx), (q, k, v), do)
        row("varlen", f"32 seqs, {tot} tok, H{H} D{D}", f, fb, tot, 4 * P, 11 * P)
    if args.op in ("all", "pisa"):
        b, h, T, d = 2, 24, 4608, 128
        q, k, v = gau(b, h, T, d), gau(b, h, T, d), gau(b, h, T, d)
        do = torch.randn_like(v)
        P = b * h * T * d * 2
        f, fb = both(lambda: piecewise_sparse_attention(q, k, v), (q, k, v), None if IMPL == "reference" else do)
        row("pisa", f"B{b} H{h} T{T} D{d} bs64 d0.1", f, fb, b * T, 7 * P, 7 * P)


if __name__ == "__main__":
    main()
