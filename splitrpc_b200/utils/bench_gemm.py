"""Times one GEMM or convolution shape on the tensor-core kernels.

    python -m splitrpc_b200.utils.bench_gemm --m 200704 --n 256 --k 64 [--residual] [--act relu] [--iters 20]
    python -m splitrpc_b200.utils.bench_gemm --conv 64,56,56,64,64,3,1,1     # n,h,w,cin,cout,k,stride,pad

Prints the CUDA-event time (L2 flushed between iterations), the achieved TFLOP/s
and GB/s and their fraction of the measured peaks.  With ``--iters 1`` it is a
small, self-ending command to capture under ``ncu``.
"""
from __future__ import annotations

import argparse

import torch

from .. import ops
from .profile_model import _peaks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--conv", default=None)
    ap.add_argument("--dual", default=None, help="two-input 1x1 convolution: n,oh,c1,h2,c2,cout,stride2")
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--act", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--graph", action="store_true", help="time graph replays of (flush, op) pairs minus the flushes alone")
    ap.add_argument("--library", action="store_true", help="time PyTorch's cuBLAS / cuDNN call for the same shape instead")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    hbm, tf, tag = _peaks()
    if args.dual:
        n, oh, c1, h2, c2, cout, s2 = (int(v) for v in args.dual.split(","))
        x1 = (torch.randn(n, oh, oh, c1, device="cuda") * 0.5).bfloat16()
        x2 = (torch.randn(n, h2, h2, c2, device="cuda") * 0.5).bfloat16()
        w1 = (torch.randn(cout, c1, device="cuda") * 0.1).bfloat16()
        w2 = (torch.randn(cout, c2, device="cuda") * 0.1).bfloat16()
        wt = torch.cat([w1, w2], dim=1).contiguous()
        bias = torch.randn(cout, device="cuda")
        out = torch.empty(n, oh, oh, cout, dtype=torch.bfloat16, device="cuda")
        fn = lambda: ops.conv1x1_dual(x1, x2, wt, bias=bias, stride2=s2, act=args.act, out=out)
        if args.library:
            import torch.nn.functional as F

            torch.backends.cudnn.benchmark = True
            x1l, x2l, bl = x1.permute(0, 3, 1, 2), x2.permute(0, 3, 1, 2), bias.bfloat16()
            w1l, w2l = w1.view(cout, c1, 1, 1), w2.view(cout, c2, 1, 1)
            fn = lambda: torch.relu_(F.conv2d(x1l, w1l, bl).add_(F.conv2d(x2l, w2l, None, s2)))
        flops = 2.0 * n * oh * oh * cout * (c1 + c2)
        nbytes = 2 * (x1.numel() + x2.numel() // (s2 * s2) + wt.numel() + out.numel())
        desc = f"two-input 1x1 conv {args.dual}"
    elif args.conv:
        n, h, w, cin, cout, k, s, pad = (int(v) for v in args.conv.split(","))
        x = (torch.randn(n, h, w, cin, device="cuda") * 0.5).bfloat16()
        wt = (torch.randn(cout, k, k, cin, device="cuda") * 0.1).bfloat16()
        bias = torch.randn(cout, device="cuda")
        oh, ow = (h + 2 * pad - k) // s + 1, (w + 2 * pad - k) // s + 1
        out = torch.empty(n, oh, ow, cout, dtype=torch.bfloat16, device="cuda")
        res = torch.randn_like(out) if args.residual else None
        fn = lambda: ops.conv2d_nhwc(x, wt, bias=bias, residual=res, stride=s, pad=pad, act=args.act, out=out)
        if args.library:
            import torch.nn.functional as F

            torch.backends.cudnn.benchmark = True
            xl = x.permute(0, 3, 1, 2)  # NHWC storage seen as NCHW = channels-last
            wl = wt.permute(0, 3, 1, 2)
            bl = bias.bfloat16()
            fn = lambda: F.conv2d(xl, wl, bl, s, pad)
        flops = 2.0 * n * oh * ow * cout * k * k * cin
        nbytes = 2 * (x.numel() + wt.numel() + out.numel() * (2 if args.residual else 1))
        desc = f"conv {args.conv}"
    else:
        M, N, K = args.m, args.n, args.k
        a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
        bias = torch.randn(N, device="cuda")
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        res = torch.randn(M, N, device="cuda").bfloat16() if args.residual else None
        fn = lambda: ops.gemm(a, b, bias=bias, residual=res, act=args.act, out=out)
        if args.library:
            bl = bias.bfloat16()
            fn = lambda: torch.nn.functional.linear(a, b, bl)
        flops = 2.0 * M * N * K
        nbytes = 2 * (M * K + N * K + M * N * (2 if args.residual else 1))
        desc = f"gemm M{M} N{N} K{K}"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(min(3, args.iters)):
        fn()
    torch.cuda.synchronize()
    times = []
    if args.graph:
        # Device time without host launch latency or event granularity: a graph of `iters` x (flush, op) minus a graph
        # of `iters` x (flush), each replayed five times.
        def replay_ms(with_op):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(args.iters):
                    flush.zero_()
                    if with_op:
                        fn()
            g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return sorted(ts)[2]

        times = [(replay_ms(True) - replay_ms(False)) / args.iters]
    else:
        for _ in range(args.iters):
            if not args.no_flush:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    ops.check_status()
    if args.library:
        desc = "library " + desc + (" (two convolutions + add + ReLU)" if args.dual else " (bias only, no activation or residual)")
    times.sort()
    ms = times[len(times) // 2]
    print(f"{desc}{' +res' if args.residual else ''}: median {ms * 1e3:.1f} us  {flops / ms / 1e9:.1f} TFLOP/s "
          f"({flops / ms / 1e9 / tf:.2f} {tag})  {nbytes / ms / 1e6:.0f} GB/s ({nbytes / ms / 1e6 / hbm:.2f} {tag})")


if __name__ == "__main__":
    main()
