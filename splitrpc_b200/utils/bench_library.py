"""Library stand-in for the original's model path: the same networks through PyTorch's cuDNN / cuBLAS / SDPA kernels.

    python -m splitrpc_b200.utils.bench_library [--model resnet50|bert_base] [--batch N] [--iters 30]

The original serves ResNet-50 and BERT through ONNX Runtime + TensorRT (reference ``src/apps/ort_app.h:477-527``),
which cannot be installed here.  This script times the closest thing the image offers: the same architecture and
the same (batch-norm-folded, random) weights evaluated in bf16 by PyTorch library kernels, channels-last for the
convolutions, captured into a CUDA graph so that no host launch time is counted.  It prints the CUDA-event time
per batch (L2 flushed between replays) next to this package's own forward under the same protocol.  None of this
package's kernels run on the library side.
"""
from __future__ import annotations

import argparse

import torch
import torch.nn.functional as F


def _resnet_library(model, x):
    p = model.params
    dt = torch.bfloat16
    mean = torch.tensor(model.mean, device=x.device, dtype=torch.float32).view(1, 3, 1, 1)
    inv = torch.tensor(model.inv_std, device=x.device, dtype=torch.float32).view(1, 3, 1, 1)
    w = {}

    def cw(name):  # [cout, r, s, cin] bf16 -> NCHW weight in channels-last memory format
        if name not in w:
            w[name] = (p[name + ".w"].permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last), p[name + ".b"].to(dt))
        return w[name]

    stem_w = p["stem.w_nchw"].to(dt).contiguous(memory_format=torch.channels_last)
    stem_b = p["stem.b"].to(dt)
    fc_w, fc_b = p["fc.w"].to(dt), p["fc.b"].to(dt)
    for name, cin, width, s, ds in model.blocks:
        for part in (".c1", ".c2", ".c3") + ((".ds",) if ds else ()):
            cw(name + part)

    def fwd():
        y = ((x - mean) * inv).to(dt).contiguous(memory_format=torch.channels_last)
        y = F.relu(F.conv2d(y, stem_w, stem_b, 2, 3))
        y = F.max_pool2d(y, 3, 2, 1)
        for name, cin, width, s, ds in model.blocks:
            t = F.relu(F.conv2d(y, *cw(name + ".c1")))
            t = F.relu(F.conv2d(t, *cw(name + ".c2"), s, 1))
            idn = F.conv2d(y, *cw(name + ".ds"), s) if ds else y
            y = F.relu(F.conv2d(t, *cw(name + ".c3")) + idn)
        y = y.mean((2, 3))
        return torch.softmax(F.linear(y, fc_w, fc_b).float(), -1)

    return fwd


def _bert_library(model, ids):
    cfg, p, S = model.cfg, model.params, model.seq
    H, B = cfg.hidden, ids.shape[0]
    dt = torch.bfloat16
    f = {k: v.to(dt) for k, v in p.items() if v.is_floating_point()}

    def fwd():
        x = f["emb.word"][ids.long()] + f["emb.pos"][:S].unsqueeze(0) + f["emb.type"][0]
        x = F.layer_norm(x, (H,), f["emb.ln.g"], f["emb.ln.b"], 1e-12).view(B * S, H)
        for l in range(cfg.layers):
            q = f"l{l}."
            qkv = F.linear(x, f[q + "qkv.w"], f[q + "qkv.b"])
            qh, kh, vh = (t.view(B, S, cfg.heads, 64).transpose(1, 2) for t in qkv.split(H, dim=1))
            ctx = F.scaled_dot_product_attention(qh, kh, vh).transpose(1, 2).reshape(B * S, H)
            x1 = F.layer_norm(F.linear(ctx, f[q + "o.w"], f[q + "o.b"]) + x, (H,), f[q + "ln1.g"], f[q + "ln1.b"], 1e-12)
            h = F.gelu(F.linear(x1, f[q + "f1.w"], f[q + "f1.b"]))
            x = F.layer_norm(F.linear(h, f[q + "f2.w"], f[q + "f2.b"]) + x1, (H,), f[q + "ln2.g"], f[q + "ln2.b"], 1e-12)
        cls = x.view(B, S, H)[:, 0]
        pooled = torch.tanh(F.linear(cls, f["pool.w"], f["pool.b"]))
        return torch.softmax(F.linear(pooled, f["cls.w"], f["cls.b"]).float()[:, : cfg.num_labels], -1)

    return fwd


def _time_graph(fn, iters, flush):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "bert_base"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--iters", type=int, default=30)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    torch.backends.cudnn.benchmark = True
    from ..models import BERT_BASE, BertClassifier, ResNet50
    from .. import ops

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    with torch.no_grad():
        if args.model == "resnet50":
            nb = args.batch or 64
            model = ResNet50(device=0, max_batch=nb)
            x = torch.randn(nb, 3, 224, 224, device="cuda")
            lib = _resnet_library(model, x)
            resp = torch.empty(nb, 1000, device="cuda")
            ours = lambda: model.forward(nb, x=x, out=resp)
        else:
            nb = args.batch or 32
            model = BertClassifier(BERT_BASE, seq=128, device=0, max_batch=nb)
            ids = torch.randint(0, 30522, (nb, 128), device="cuda", dtype=torch.int32)
            lib = _bert_library(model, ids)
            resp = torch.empty(nb, model.resp_size // 4, device="cuda")
            ours = lambda: model.forward(nb, ids=ids, out=resp)
        a, b = lib().float(), ours().float()
        torch.cuda.synchronize()
        ops.check_status()
        agree = float((a.argmax(-1) == b.argmax(-1)).float().mean())
        t_lib = _time_graph(lib, args.iters, flush)
        t_ours = _time_graph(ours, args.iters, flush)
    print(f"{args.model} batch {nb}, bf16, CUDA-graph replay, L2 flushed between replays")
    print(f"  PyTorch library kernels (cuDNN/cuBLAS/SDPA): {t_lib:.3f} ms  ({nb / t_lib * 1e3:.0f} req/s)")
    print(f"  this package (tcgen05 kernels):              {t_ours:.3f} ms  ({nb / t_ours * 1e3:.0f} req/s)  "
          f"x{t_lib / t_ours:.2f}")
    print(f"  top-1 agreement between the two on random inputs: {agree:.2f}")


if __name__ == "__main__":
    main()
