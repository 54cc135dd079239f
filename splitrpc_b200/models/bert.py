"""BERT encoder + sequence classifier in bf16 on this library's kernels.

Per layer: fused QKV GEMM, attention (head dim 64), output GEMM with the
residual added in its epilogue, LayerNorm, FFN GEMM with GELU in the epilogue,
second FFN GEMM with the residual in its epilogue, LayerNorm.  The embedding
gather reads the int32 token ids of the request window through the device stub
and applies the embedding LayerNorm in the same kernel; the classifier's
softmax writes into the response window.  Requests carry ``seq`` int32 ids (mask
all ones); responses are ``num_labels`` fp32 probabilities.

The original serves BERT-SQuAD through ONNX Runtime
(reference ``src/apps/ort_defs.h:141-190``, ``src/apps/ort_app.h:477-527``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops


@dataclass(frozen=True)
class BertConfig:
    layers: int
    hidden: int
    heads: int
    ffn: int
    vocab: int = 30522
    max_pos: int = 512
    num_labels: int = 2


BERT_BASE = BertConfig(12, 768, 12, 3072)
BERT_LARGE = BertConfig(24, 1024, 16, 4096)


class BertClassifier:
    def __init__(self, cfg: BertConfig = BERT_BASE, seq: int = 128, device: int = 0, max_batch: int = 32, seed: int = 0,
                 attention: str = "tensor_core"):
        assert cfg.hidden == cfg.heads * 64, "attention kernel is specialised for head dim 64"
        self.cfg, self.seq, self.max_batch = cfg, seq, max_batch
        self.attention = attention  # "tensor_core" (tcgen05 kernel) or "simt"
        self.device = torch.device("cuda", device)
        self.req_size = seq * 4
        self.resp_size = cfg.num_labels * 4
        g = torch.Generator(device="cpu").manual_seed(seed)
        H, F = cfg.hidden, cfg.ffn
        bf, dev = torch.bfloat16, self.device

        def mat(n, k, std=0.02):
            return (torch.randn((n, k), generator=g) * std).to(dev, bf).contiguous()

        def vec(n, std=0.02, base=0.0):
            return (torch.randn((n,), generator=g) * std + base).to(dev, torch.float32)

        p = self.params = {}
        p["emb.word"], p["emb.pos"], p["emb.type"] = mat(cfg.vocab, H), mat(cfg.max_pos, H), mat(2, H)
        p["emb.ln.g"], p["emb.ln.b"] = vec(H, 0.02, 1.0), vec(H)
        for l in range(cfg.layers):
            q = f"l{l}."
            p[q + "qkv.w"], p[q + "qkv.b"] = mat(3 * H, H), vec(3 * H)
            p[q + "o.w"], p[q + "o.b"] = mat(H, H), vec(H)
            p[q + "ln1.g"], p[q + "ln1.b"] = vec(H, 0.02, 1.0), vec(H)
            p[q + "f1.w"], p[q + "f1.b"] = mat(F, H), vec(F)
            p[q + "f2.w"], p[q + "f2.b"] = mat(H, F), vec(H)
            p[q + "ln2.g"], p[q + "ln2.b"] = vec(H, 0.02, 1.0), vec(H)
        p["pool.w"], p["pool.b"] = mat(H, H), vec(H)
        p["cls.w"], p["cls.b"] = mat(8, H, 0.2), vec(8, 0.1)  # rows >= num_labels are padding
        T = max_batch * seq
        self.buf = {
            "x": torch.empty((T, H), dtype=bf, device=dev), "qkv": torch.empty((T, 3 * H), dtype=bf, device=dev),
            "ctx": torch.empty((T, H), dtype=bf, device=dev), "attn": torch.empty((T, H), dtype=bf, device=dev),
            "x1": torch.empty((T, H), dtype=bf, device=dev), "ffn": torch.empty((T, F), dtype=bf, device=dev),
            "y": torch.empty((T, H), dtype=bf, device=dev), "pooled": torch.empty((max_batch, H), dtype=bf, device=dev),
            "logits": torch.empty((max_batch, 8), dtype=torch.float32, device=dev),
        }
        self.kernels_per_forward = 1 + 7 * cfg.layers + 3

    def forward(self, batch: int, ids: torch.Tensor | None = None, d_stub: int = 0, out: torch.Tensor | None = None,
                flag_ptr: int = 0, flag_value: int = 0, counter: torch.Tensor | None = None, d_push: int = 0) -> torch.Tensor:
        cfg, p, b, S = self.cfg, self.params, self.buf, self.seq
        T = batch * S
        x, qkv, ctx, attn, x1, ffn, y = (b[k][:T] for k in ("x", "qkv", "ctx", "attn", "x1", "ffn", "y"))
        ops.bert_embed_ln(x, batch, S, p["emb.word"], p["emb.pos"], p["emb.type"], p["emb.ln.g"], p["emb.ln.b"], ids=ids,
                          d_stub=d_stub, req_stride=self.req_size)
        for l in range(cfg.layers):
            q = f"l{l}."
            if self.attention == "tensor_core":
                # one fused Q|K|V projection; the attention kernel reads V in place (MN-major operand of P.V)
                ops.gemm(x, p[q + "qkv.w"], bias=p[q + "qkv.b"], out=qkv)
                ops.attention_tc_qkv(qkv, batch, S, cfg.heads, out=ctx)
            else:
                ops.gemm(x, p[q + "qkv.w"], bias=p[q + "qkv.b"], out=qkv)
                ops.attention_d64(qkv, batch, S, cfg.heads, out=ctx)
            ops.gemm(ctx, p[q + "o.w"], bias=p[q + "o.b"], residual=x, out=attn)
            ops.layernorm(attn, p[q + "ln1.g"], p[q + "ln1.b"], out=x1)
            ops.gemm(x1, p[q + "f1.w"], bias=p[q + "f1.b"], act="gelu", out=ffn)
            ops.gemm(ffn, p[q + "f2.w"], bias=p[q + "f2.b"], residual=x1, out=y)
            ops.layernorm(y, p[q + "ln2.g"], p[q + "ln2.b"], out=x)
        cls_rows = x.view(batch, S * cfg.hidden)[:, : cfg.hidden]  # first token of every sequence, row stride S*H
        ops.gemm(cls_rows, p["pool.w"], bias=p["pool.b"], act="tanh", out=b["pooled"][:batch])
        ops.gemm(b["pooled"][:batch], p["cls.w"], bias=p["cls.b"], out=b["logits"][:batch])
        logits = b["logits"][:batch, : cfg.num_labels]
        ops.softmax_response(logits, batch, out=out, d_stub=0 if out is not None else d_stub, resp_stride=self.resp_size,
                             counter=counter, flag_ptr=flag_ptr, flag_value=flag_value, d_push=0 if out is not None else d_push)
        return logits

    __call__ = forward

    @torch.no_grad()
    def reference_forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Plain PyTorch fp32 evaluation with the same weights; returns softmax rows ``[batch, num_labels]``."""
        import torch.nn.functional as Fn

        cfg, p, S = self.cfg, self.params, self.seq
        H = cfg.hidden
        B = ids.shape[0]
        f = lambda k: p[k].float()
        x = f("emb.word")[ids.long().clamp(0, cfg.vocab - 1)] + f("emb.pos")[:S].unsqueeze(0) + f("emb.type")[0]
        x = Fn.layer_norm(x, (H,), f("emb.ln.g"), f("emb.ln.b"), 1e-12).view(B * S, H)
        for l in range(cfg.layers):
            q = f"l{l}."
            qkv = x @ f(q + "qkv.w").t() + f(q + "qkv.b")
            qh, kh, vh = (t.view(B, S, cfg.heads, 64).transpose(1, 2) for t in qkv.split(H, dim=1))
            att = torch.softmax(qh @ kh.transpose(-1, -2) / 8.0, -1) @ vh
            ctx = att.transpose(1, 2).reshape(B * S, H)
            x1 = Fn.layer_norm(ctx @ f(q + "o.w").t() + f(q + "o.b") + x, (H,), f(q + "ln1.g"), f(q + "ln1.b"), 1e-12)
            h = Fn.gelu(x1 @ f(q + "f1.w").t() + f(q + "f1.b"))
            x = Fn.layer_norm(h @ f(q + "f2.w").t() + f(q + "f2.b") + x1, (H,), f(q + "ln2.g"), f(q + "ln2.b"), 1e-12)
        cls = x.view(B, S, H)[:, 0]
        pooled = torch.tanh(cls @ f("pool.w").t() + f("pool.b"))
        logits = pooled @ f("cls.w").t()[:, : cfg.num_labels] + f("cls.b")[: cfg.num_labels]
        return torch.softmax(logits, -1)
