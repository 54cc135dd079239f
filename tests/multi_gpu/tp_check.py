"""Run under torchrun on 2+ GPUs: checks the fused tensor-parallel kernels and the cross-GPU
scatter-gather against single-GPU references.  Prints ``MULTI_GPU_OK`` on rank 0 when everything matches."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from splitrpc_b200 import _C, ops
from splitrpc_b200.models import BertClassifier, BertClassifierTP
from splitrpc_b200.models.bert import BertConfig
from splitrpc_b200.parallel import SymmetricArena, TensorParallel, init_distributed


def check_fused_linear(rank, world, dev):
    """all-gather->GEMM and GEMM->reduce-scatter + reduce/LayerNorm against plain matmuls on the full tensors."""
    T, H, N = 128 * world * 3, 512, 768
    tpc = TensorParallel(T, H, dev, n_copy=4)
    g = torch.Generator(device="cpu").manual_seed(5)
    x_full = (torch.randn((T, H), generator=g) * 0.5).to(dev, torch.bfloat16)
    w_col = (torch.randn((N * world, H), generator=g) * 0.05).to(dev, torch.bfloat16)
    bias_col = torch.randn((N * world,), generator=g).to(dev)
    w_row = (torch.randn((H, N * world), generator=g) * 0.05).to(dev, torch.bfloat16)
    bias_row = torch.randn((H,), generator=g).to(dev)
    gamma, beta = torch.rand((H,), generator=g).to(dev) + 0.5, torch.randn((H,), generator=g).to(dev)
    rows = T // world
    for step in range(3):  # several passes: step numbers advance, buffers are reused
        tpc.begin_step()
        tpc.shard("A").copy_(x_full[rank * rows:(rank + 1) * rows] * (step + 1))
        tpc.signal("A", 1)
        y = tpc.ag_gemm("A", w_col[rank * N:(rank + 1) * N], 1, bias=bias_col[rank * N:(rank + 1) * N], act="gelu")
        tpc.gemm_rs(y, w_row[:, rank * N:(rank + 1) * N].contiguous(), "RS1", 1)
        out = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
        tpc.ln_reduce("RS1", 1, bias_row, tpc.shard("A"), gamma, beta, out)
        tpc.end_step()
        torch.cuda.synchronize()
        ops.check_status()
        xs = x_full.float() * (step + 1)
        y_ref = torch.nn.functional.gelu(xs @ w_col.float().t() + bias_col)
        torch.testing.assert_close(y.float(), y_ref[:, rank * N:(rank + 1) * N], rtol=3e-2, atol=3e-2)
        assert torch.equal(tpc.gathered["A"].float(), xs.bfloat16().float()), "all-gather mismatch"
        z = y_ref.bfloat16().float() @ w_row.float().t() + bias_row + xs.bfloat16().float()
        ref = torch.nn.functional.layer_norm(z, (H,), gamma, beta, 1e-12)[rank * rows:(rank + 1) * rows]
        torch.testing.assert_close(out.float(), ref, rtol=5e-2, atol=5e-2)
    dist.barrier()


def check_bert_tp(rank, world, dev):
    cfg = BertConfig(layers=2, hidden=512, heads=8, ffn=2048)
    B, S = 2 * world, 128
    tp_model = BertClassifierTP(cfg, seq=S, device=dev.index, batch=B, seed=3, n_copy=4)
    ref_model = BertClassifier(cfg, seq=S, device=dev.index, max_batch=B, seed=3)
    g = torch.Generator(device="cpu").manual_seed(9)
    for _ in range(2):
        ids = torch.randint(0, 30522, (B, S), generator=g, dtype=torch.int32).to(dev)
        logits = tp_model.forward(ids).clone()
        out = torch.zeros(B, 2, device=dev)
        ref_logits = ref_model.forward(B, ids=ids, out=out).clone()
        torch.cuda.synchronize()
        ops.check_status()
        torch.testing.assert_close(logits, ref_logits, rtol=5e-2, atol=5e-2)
    dist.barrier()


def check_tp_server(rank, world, dev):
    """Requests through the RPC front end of rank 0, every rank stepping the tensor-parallel graph; responses against
    a single-GPU evaluation of the same weights on the same token ids."""
    import numpy as np

    from splitrpc_b200.serving.tp_server import TensorParallelServer

    cfg = BertConfig(layers=2, hidden=512, heads=8, ffn=2048)
    B, S = 2 * world, 128
    tp_model = BertClassifierTP(cfg, seq=S, device=dev.index, batch=B, seed=5, n_copy=4)
    srv = TensorParallelServer(tp_model, outstanding=2 * B)
    if rank == 0:
        total = 6 * B + 1  # the last batch is a short one
        with srv:
            cli = srv.client(total=total, warmup=0, payload="ids", n_payloads=4, verify=True)  # verify keeps the responses
            assert cli.run_closed_loop(2 * B), "closed loop did not finish"
            assert cli.received == total
        ref_model = BertClassifier(cfg, seq=S, device=dev.index, max_batch=B, seed=5)
        for k in (0, 3, total - 1):
            ids = torch.from_numpy(np.frombuffer(cli.payload(k % 4), dtype=np.int32).copy()).view(1, S).to(dev)
            out = torch.zeros(1, 2, device=dev)
            ref_model.forward(1, ids=ids, out=out)
            torch.cuda.synchronize()
            got = torch.from_numpy(np.frombuffer(cli.response(k), dtype=np.float32).copy())[:2]
            torch.testing.assert_close(got, out[0].cpu(), rtol=5e-2, atol=5e-2)
    else:
        assert srv.serve_forever() >= 6
    ops.check_status()
    dist.barrier()


def check_cross_gpu_sg(rank, world, dev):
    """Rank k pulls 8 KB fragments out of rank 0's arena into its own buffer and pushes an echo back into rank 0."""
    frag, n_frag = 8192, 64
    arena = SymmetricArena(2 * world * frag * n_frag + 4096, dev)
    rx = arena.alloc("rx", (world, n_frag * frag), torch.uint8)
    tx = arena.alloc("tx", (world, n_frag * frag), torch.uint8)
    if rank == 0:
        rx.copy_(torch.randint(0, 256, rx.shape, dtype=torch.uint8, device=dev))
    arena.barrier()
    local = torch.zeros(n_frag * frag, dtype=torch.uint8, device=dev)
    src0 = arena.ptr("rx", 0, rank * n_frag * frag)
    _C.sg_copy([(src0 + i * frag, local.data_ptr() + i * frag, frag) for i in range(n_frag)], 0)
    dst0 = arena.ptr("tx", 0, rank * n_frag * frag)
    _C.sg_copy([(local.data_ptr() + i * frag, dst0 + i * frag, frag) for i in range(n_frag)], 1)
    arena.barrier()
    if rank == 0:
        assert torch.equal(tx, rx), "cross-GPU echo mismatch"
    arena.barrier()


def main():
    rank, world, local_rank = init_distributed()
    dev = torch.device("cuda", local_rank)
    check_cross_gpu_sg(rank, world, dev)
    check_fused_linear(rank, world, dev)
    check_bert_tp(rank, world, dev)
    check_tp_server(rank, world, dev)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
