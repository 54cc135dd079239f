"""Times the fused tensor-parallel kernels against their NCCL + GEMM baselines (run under torchrun).

    torchrun --nproc-per-node N -m splitrpc_b200.parallel.bench_tp [--tokens 6144] [--hidden 1024] [--ffn 4096]

For each of the two fused ops it prints, max over ranks of the CUDA-event time:
  all-gather -> GEMM          fused kernel   vs   ncclAllGather + this library's GEMM
  GEMM -> reduce-scatter (+LN) fused kernels  vs   GEMM + ncclReduceScatter + LayerNorm
and the fraction of the roofline: the slower of FLOPs / measured GEMM peak and NVLink bytes / 770 GB/s.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from .. import ops
from ..utils.profile_model import _peaks
from .symm import init_distributed
from .tp import TensorParallel

NVLINK_GBS = 770.0


def _time(fn, iters, pre=None, graph=True):
    """Median CUDA-event time of ``fn`` (max over ranks).  With ``graph`` the launches of ``fn`` are captured once and
    replayed, so the figure is the device time of the kernels and not the host's launch rate."""
    fn()
    torch.cuda.synchronize()
    dist.barrier()
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        fn = g.replay
        fn()
        torch.cuda.synchronize()
        dist.barrier()
    ts = []
    for _ in range(iters):
        if pre:
            pre()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=6144)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--n-copy", type=int, default=None)
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of graph replays")
    args = ap.parse_args()
    rank, world, local_rank = init_distributed()
    dev = torch.device("cuda", local_rank)
    T, H, F = args.tokens, args.hidden, args.ffn
    Fl = F // world
    rows = T // world
    tpc = TensorParallel(T, H, dev, n_copy=args.n_copy)
    hbm, tf, tag = _peaks()
    g = torch.Generator(device="cpu").manual_seed(1)
    x_shard = (torch.randn((rows, H), generator=g) * 0.5).to(dev, torch.bfloat16)
    w1 = (torch.randn((Fl, H), generator=g) * 0.03).to(dev, torch.bfloat16)
    b1 = torch.randn((Fl,), generator=g).to(dev)
    w2 = (torch.randn((H, Fl), generator=g) * 0.03).to(dev, torch.bfloat16)
    b2 = torch.randn((H,), generator=g).to(dev)
    gamma, beta = torch.ones(H, device=dev), torch.zeros(H, device=dev)
    y = torch.empty((T, Fl), dtype=torch.bfloat16, device=dev)
    out = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    use_graph = not args.no_graph

    # ---- fused all-gather -> GEMM
    def fused_ag():
        tpc.begin_step()
        tpc.signal("A", 1)
        tpc.ag_gemm("A", w1, 1, bias=b1, act="gelu", out=y)
        tpc.end_step()

    tpc.shard("A").copy_(x_shard)
    t_ag = _time(fused_ag, args.iters, pre=flush.zero_, graph=use_graph)
    # baseline: NCCL all-gather then the same GEMM kernel on local memory
    gathered = torch.empty((T, H), dtype=torch.bfloat16, device=dev)

    def nccl_ag():
        dist.all_gather_into_tensor(gathered, x_shard)
        ops.gemm(gathered, w1, bias=b1, act="gelu", out=y)

    t_ag_base = _time(nccl_ag, args.iters, pre=flush.zero_, graph=use_graph)
    t_ag_gemm = _time(lambda: ops.gemm(gathered, w1, bias=b1, act="gelu", out=y), args.iters, pre=flush.zero_, graph=use_graph)

    # ---- fused GEMM -> reduce-scatter + reduce/LayerNorm
    def fused_rs():
        tpc.begin_step()
        tpc.gemm_rs(y, w2, "RS1", 1)
        tpc.ln_reduce("RS1", 1, b2, tpc.shard("A"), gamma, beta, out)
        tpc.end_step()

    t_rs = _time(fused_rs, args.iters, pre=flush.zero_, graph=use_graph)
    partial = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    red = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)

    def nccl_rs():
        ops.gemm(y, w2, out=partial)
        dist.reduce_scatter_tensor(red, partial)
        ops.layernorm(red, gamma, beta, residual=x_shard, out=out)

    t_rs_base = _time(nccl_rs, args.iters, pre=flush.zero_, graph=use_graph)
    t_rs_gemm = _time(lambda: ops.gemm(y, w2, out=partial), args.iters, pre=flush.zero_, graph=use_graph)
    ops.check_status()
    if rank == 0:
        fl = 2.0 * T * Fl * H
        nv_ag = (world - 1) * rows * H * 2          # bytes each rank pulls over NVLink
        nv_rs = (world - 1) * rows * H * 2          # bytes each rank pushes
        roof_ag = max(fl / (tf * 1e12), nv_ag / (NVLINK_GBS * 1e9)) * 1e3
        roof_rs = max(fl / (tf * 1e12), nv_rs / (NVLINK_GBS * 1e9)) * 1e3
        print(f"tp={world} tokens={T} hidden={H} ffn={F} (local {Fl}), {'graph replays' if use_graph else 'eager launches'}")
        print(f"the two GEMMs alone on local memory: {t_ag_gemm * 1e3:.1f} us ({fl / t_ag_gemm / 1e9:.0f} TFLOP/s), "
              f"{t_rs_gemm * 1e3:.1f} us ({fl / t_rs_gemm / 1e9:.0f} TFLOP/s)")
        print(f"all-gather->GEMM      fused {t_ag * 1e3:8.1f} us   NCCL all-gather + GEMM {t_ag_base * 1e3:8.1f} us   "
              f"roofline {roof_ag * 1e3:6.1f} us -> {roof_ag / t_ag:.2f} of roofline ({tag} GEMM peak, 770 GB/s NVLink)")
        print(f"GEMM->reduce-scatter+LN fused {t_rs * 1e3:8.1f} us   GEMM + NCCL reduce-scatter + LN {t_rs_base * 1e3:8.1f} us   "
              f"roofline {roof_rs * 1e3:6.1f} us -> {roof_rs / t_rs:.2f} of roofline")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
