"""Tensor-parallel BERT classifier (BERT-large, seq 384 by default) over NVLink.

Attention heads and the FFN are split over the ranks; activations between
blocks are sharded by rows.  Every collective is fused into a kernel of this
library: all-gather into the QKV / FFN-up GEMM, reduce-scatter into the
attention-output / FFN-down GEMM epilogue, and the reduction itself into the
LayerNorm that follows (see ``splitrpc_b200.parallel.tp``).  All ranks are given
the same token ids (the ingress fans a batch out to every rank of the group) and
end with the same logits.  Weights are the shards of the same random-init model
that ``BertClassifier`` builds for a given seed, so the two can be compared.
"""
from __future__ import annotations

import torch

from .. import ops
from ..parallel.tp import TensorParallel
from .bert import BERT_LARGE, BertClassifier, BertConfig


class BertClassifierTP:
    def __init__(self, cfg: BertConfig = BERT_LARGE, seq: int = 384, device: int = 0, batch: int = 16, seed: int = 0,
                 n_copy: int | None = None, group=None):
        import torch.distributed as dist

        self.cfg, self.seq, self.batch = cfg, seq, batch
        self.device = torch.device("cuda", device)
        self.tp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        tp, r = self.tp, self.rank
        assert cfg.heads % tp == 0 and batch % tp == 0
        self.req_size, self.resp_size = seq * 4, cfg.num_labels * 4
        H, F = cfg.hidden, cfg.ffn
        Hl, Fl = H // tp, F // tp
        self.Hl, self.Fl, self.heads_local = Hl, Fl, cfg.heads // tp
        # Full model on this GPU only long enough to cut the shards (same seed on every rank).
        full = BertClassifier(cfg, seq=seq, device=device, max_batch=1, seed=seed, attention="tensor_core")
        fp = full.params
        p = self.params = {k: fp[k] for k in ("emb.word", "emb.pos", "emb.type", "emb.ln.g", "emb.ln.b", "pool.w", "pool.b",
                                              "cls.w", "cls.b")}
        sl = slice(r * Hl, (r + 1) * Hl)
        for l in range(cfg.layers):
            q = f"l{l}."
            w, bq = fp[q + "qkv.w"], fp[q + "qkv.b"]
            # this rank's heads of Q, K and V as one [3*Hl, H] projection (Q | K | V thirds)
            p[q + "qkv.w"] = torch.cat([w[:H][sl], w[H:2 * H][sl], w[2 * H:][sl]]).contiguous()
            p[q + "qkv.b"] = torch.cat([bq[:H][sl], bq[H:2 * H][sl], bq[2 * H:][sl]]).contiguous()
            p[q + "o.w"] = fp[q + "o.w"][:, sl].contiguous()
            p[q + "o.b"] = fp[q + "o.b"]
            p[q + "f1.w"] = fp[q + "f1.w"][r * Fl:(r + 1) * Fl].contiguous()
            p[q + "f1.b"] = fp[q + "f1.b"][r * Fl:(r + 1) * Fl].contiguous()
            p[q + "f2.w"] = fp[q + "f2.w"][:, r * Fl:(r + 1) * Fl].contiguous()
            p[q + "f2.b"] = fp[q + "f2.b"]
            for k in ("ln1.g", "ln1.b", "ln2.g", "ln2.b"):
                p[q + k] = fp[q + k]
        del full
        torch.cuda.empty_cache()
        T = batch * seq
        self.T = T
        self.tpc = TensorParallel(T, H, self.device, n_copy=n_copy, group=group)
        bf, dev = torch.bfloat16, self.device
        self.buf = {"qkv": torch.empty((T, 3 * Hl), dtype=bf, device=dev),
                    "ctx": torch.empty((T, Hl), dtype=bf, device=dev), "ffn": torch.empty((T, Fl), dtype=bf, device=dev),
                    "pooled": torch.empty((batch, H), dtype=bf, device=dev),
                    "logits": torch.empty((batch, 8), dtype=torch.float32, device=dev)}
        self.kernels_per_forward = 3 + 7 * cfg.layers + 5

    def forward(self, ids: torch.Tensor, out: torch.Tensor | None = None, d_stub: int = 0, d_push: int = 0,
                n_resp: int | None = None, resp_stride: int | None = None) -> torch.Tensor:
        """``ids``: int32 ``[batch, seq]`` (identical on every rank).  Returns fp32 logits ``[batch, num_labels]``.

        ``out``: probabilities go there.  ``d_stub`` / ``d_push`` (the serving app's stub and response-push block):
        the first ``n_resp`` rows go to the app's response slots, ``resp_stride`` bytes apart, and the kernel completes
        the slots when the server has enabled that."""
        cfg, p, b, S, t = self.cfg, self.params, self.buf, self.seq, self.tpc
        B, r, tp = self.batch, self.rank, self.tp
        bl = B // tp
        t.begin_step()
        ops.bert_embed_ln(t.shard("A"), bl, S, p["emb.word"], p["emb.pos"], p["emb.type"], p["emb.ln.g"], p["emb.ln.b"],
                          ids=ids[r * bl:(r + 1) * bl], req_stride=S * 4)
        t.signal("A", 1)
        for l in range(cfg.layers):
            q = f"l{l}."
            e = l + 1
            t.ag_gemm("A", p[q + "qkv.w"], e, bias=p[q + "qkv.b"], out=b["qkv"])
            ops.attention_tc_qkv(b["qkv"], B, S, self.heads_local, out=b["ctx"])  # V in place, no transposed copy
            t.gemm_rs(b["ctx"], p[q + "o.w"], "RS1", e)
            t.ln_reduce("RS1", e, p[q + "o.b"], t.shard("A"), p[q + "ln1.g"], p[q + "ln1.b"], out=t.shard("B"), signal=("B", e))
            t.ag_gemm("B", p[q + "f1.w"], e, bias=p[q + "f1.b"], act="gelu", out=b["ffn"])
            t.gemm_rs(b["ffn"], p[q + "f2.w"], "RS2", e)
            t.ln_reduce("RS2", e, p[q + "f2.b"], t.shard("B"), p[q + "ln2.g"], p[q + "ln2.b"], out=t.shard("A"),
                        signal=("A", e + 1))
        t.ag_gemm("A", None, cfg.layers + 1)  # plain all-gather of the final hidden states
        t.end_step()
        x = t.gathered["A"]
        cls_rows = x.view(B, S * cfg.hidden)[:, : cfg.hidden]
        ops.gemm(cls_rows, p["pool.w"], bias=p["pool.b"], act="tanh", out=b["pooled"])
        ops.gemm(b["pooled"], p["cls.w"], bias=p["cls.b"], out=b["logits"])
        logits = b["logits"][:, : cfg.num_labels]
        if out is not None or d_stub:
            ops.softmax_response(logits, B if n_resp is None else n_resp, out=out, d_stub=0 if out is not None else d_stub,
                                 resp_stride=resp_stride or self.resp_size, d_push=0 if out is not None else d_push)
        return logits

    __call__ = forward
