"""Per-kernel timing of one model forward pass.

    python -m splitrpc_b200.utils.profile_model --model resnet50 --batch 64 [--iters 5] [--top 20]

Runs the model eagerly (one kernel launch per op), brackets every op of
``splitrpc_b200.ops`` with CUDA events on the launching stream and prints the
time, the algorithmic FLOPs / bytes and the achieved fraction of the measured
peaks (``MEASURED_PEAKS.json`` beside the package when present, otherwise the
stated fallback).  With ``--iters 1 --no-events`` it is the command to wrap in
``ncu`` for a kernel capture.
"""
from __future__ import annotations

import argparse
import json
import os
from collections import defaultdict

import torch

from .. import ops


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def _work(name, args, kwargs, out):
    """Algorithmic (flops, bytes) of one op call."""
    if name in ("gemm", "fc_skinny"):
        a, b = args[0], args[1]
        M, K = a.shape
        N = b.shape[0]
        by = 2 * (M * K + N * K + M * N) + (2 * M * N if kwargs.get("residual") is not None else 0)
        return 2.0 * M * N * K, by, f"M{M} N{N} K{K}"
    if name == "conv2d_nhwc":
        x, w = args[0], args[1]
        n, h, wd, cin = x.shape
        cout, r, s, _ = w.shape
        oh, ow = out.shape[1], out.shape[2]
        by = 2 * (x.numel() + w.numel() + out.numel()) + (2 * out.numel() if kwargs.get("residual") is not None else 0)
        return 2.0 * n * oh * ow * cout * r * s * cin, by, f"{n}x{h}x{wd}x{cin}->{cout} k{r} s{kwargs.get('stride', 1)}"
    if name == "conv1x1_dual":
        x1, x2, w = args[0], args[1], args[2]
        st = kwargs.get("stride2", 1)
        by = 2 * (x1.numel() + x2.numel() // (st * st) + w.numel() + out.numel())
        return 2.0 * out.numel() * w.shape[1], by, f"{tuple(x1.shape)}+{tuple(x2.shape)}/s{st}->{w.shape[0]}"
    if name == "stem_s2d":
        batch = args[1]
        return 0.0, batch * (3 * 224 * 224 * 4 + 115 * 115 * 16 * 2), f"b{batch}"
    if name == "stem_conv":
        batch = args[2]
        return 2.0 * batch * 12544 * 64 * 256, 2 * batch * (115 * 115 * 16 + 12544 * 64), f"b{batch} 4x1 taps x 64ch windows"
    if name == "stem_im2col":
        batch = args[1]
        return 0.0, batch * (3 * 224 * 224 * 4 + 112 * 112 * 192 * 2), f"b{batch}"
    if isinstance(out, torch.Tensor):
        by = out.numel() * out.element_size()
        for a in args:
            if isinstance(a, torch.Tensor):
                by += a.numel() * a.element_size()
        return 0.0, by, "x".join(str(d) for d in out.shape)
    return 0.0, 0, ""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "bert_base", "bert_large"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--no-events", action="store_true")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    if args.model == "resnet50":
        from ..models import ResNet50

        m = ResNet50(max_batch=args.batch)
        inp = dict(x=torch.randn(args.batch, 3, 224, 224, device="cuda"))
        out = torch.zeros(args.batch, 1000, device="cuda")
    else:
        from ..models import BERT_BASE, BERT_LARGE, BertClassifier

        cfg = BERT_BASE if args.model == "bert_base" else BERT_LARGE
        seq = args.seq or (128 if args.model == "bert_base" else 384)
        m = BertClassifier(cfg, seq=seq, max_batch=args.batch)
        inp = dict(ids=torch.randint(0, 30522, (args.batch, seq), device="cuda", dtype=torch.int32))
        out = torch.zeros(args.batch, 2, device="cuda")

    records = []
    if not args.no_events:
        for name in ("gemm", "fc_skinny", "conv2d_nhwc", "conv1x1_dual", "stem_im2col", "stem_s2d", "stem_conv", "maxpool3x3s2", "global_avgpool", "softmax_response", "layernorm",
                     "bert_embed_ln", "attention_d64"):
            fn = getattr(ops, name)

            def wrapped(*a, _fn=fn, _name=name, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = _fn(*a, **k)
                e1.record()
                o = r if isinstance(r, torch.Tensor) else k.get("out")
                records.append((_name, _work(_name, a, k, o), e0, e1))
                return r

            setattr(ops, name, wrapped)
    for it in range(args.iters):
        records.clear()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        m.forward(args.batch, out=out, **inp)
        t1.record()
        torch.cuda.synchronize()
    ops.check_status()
    total = t0.elapsed_time(t1)
    print(f"{args.model} batch {args.batch}: forward {total:.3f} ms ({args.batch / total * 1e3:.0f} req/s), "
          f"{len(records)} kernels")
    if args.no_events:
        return
    hbm, tf, tag = _peaks()
    rows, agg = [], defaultdict(float)
    for name, (fl, by, desc), e0, e1 in records:
        ms = e0.elapsed_time(e1)
        rows.append((ms, name, desc, fl, by))
        agg[name] += ms
    print("by op type:", ", ".join(f"{k} {v:.3f} ms" for k, v in sorted(agg.items(), key=lambda kv: -kv[1])))
    print(f"{'ms':>8} {'op':<16} {'shape':<34} {'TFLOP/s':>9} {'GB/s':>8} {'frac ' + tag:>18}")
    for ms, name, desc, fl, by in sorted(rows, key=lambda r: -r[0])[: args.top]:
        tfl = fl / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        gbs = by / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        frac = max(tfl / tf, gbs / hbm)
        print(f"{ms:8.4f} {name:<16} {desc:<34} {tfl:9.1f} {gbs:8.0f} {frac:18.2f}")
    tot_fl = sum(r[3] for r in rows)
    print(f"total algorithmic {tot_fl / 1e9:.1f} GFLOP -> {tot_fl / (total * 1e-3) / 1e12:.1f} TFLOP/s over the whole forward")


if __name__ == "__main__":
    main()
