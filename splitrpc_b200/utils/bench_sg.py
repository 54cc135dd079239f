"""Scatter-gather / echo microbenchmark: payloads of 64 B - 4 MB split into 8 KB fragments.

    python -m splitrpc_b200.utils.bench_sg [--source pinned|device] [--batch 64] [--impl 0|1] [--sizes 64,4096,...]
    torchrun --nproc-per-node N -m splitrpc_b200.utils.bench_sg --source peer     # every rank pulls from GPU 0

For each payload size a batch of requests is gathered from its fragments (in the
pinned receive arena, in local HBM, or in GPU 0's memory over NVLink) into a
contiguous batch buffer and echoed back, with this library's copy kernels and,
as the baseline, with one cudaMemcpyAsync per fragment (the copy-engine path of
the original, reference src/transport/g_copy_ng.cu:194-199).  Times are CUDA
events on the launching stream (max over ranks when distributed), L2 flushed
between iterations.
"""
from __future__ import annotations

import argparse
import os

import torch

from .. import _C

FRAG = 8192


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default="pinned", choices=["pinned", "device", "peer"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--impl", type=int, default=0, help="0 = SIMT vector kernel, 1 = cp.async.bulk pipeline")
    ap.add_argument("--sizes", default=",".join(str(1 << p) for p in range(6, 23, 2)))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-baseline", action="store_true")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local_rank = 0, 0
    dist = None
    if world > 1 or args.source == "peer":
        import torch.distributed as dist

        from ..parallel import SymmetricArena, init_distributed

        rank, world, local_rank = init_distributed()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sizes = [int(s) for s in args.sizes.split(",")]
    max_bytes = max(sizes) * args.batch
    if args.source == "pinned":
        src_t = torch.empty(max_bytes, dtype=torch.uint8).pin_memory()
        src_t.random_(0, 256)
        src_ptr = src_t.data_ptr()
        peak = 55.0  # PCIe 5.0 x16 practical GB/s (context only)
    elif args.source == "device":
        src_t = torch.randint(0, 256, (max_bytes,), dtype=torch.uint8, device=dev)
        src_ptr = src_t.data_ptr()
        peak = 6536.0 / 2
    else:
        arena = SymmetricArena(max_bytes + 4096, dev)
        src_t = arena.alloc("rx", (max_bytes,), torch.uint8)
        if rank == 0:
            src_t.random_(0, 256)
        arena.barrier()
        src_ptr = arena.ptr("rx", 0)
        peak = 770.0
    batch_buf = torch.zeros(max_bytes, dtype=torch.uint8, device=dev)
    echo_buf = torch.zeros(max_bytes, dtype=torch.uint8, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            if dist:
                torch.cuda.synchronize()
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
        if dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if rank == 0:
        print(f"source={args.source} batch={args.batch} impl={args.impl} ranks={world}  (GB/s is per rank, gather direction)")
        print(f"{'payload':>9} {'frags':>6} {'gather us':>10} {'GB/s':>8} {'frac':>6} {'echo us':>9} {'memcpy/frag us':>15}")
    for size in sizes:
        items, back = [], []
        for r in range(args.batch):
            off = 0
            while off < size:
                ln = min(FRAG, size - off)
                items.append((src_ptr + r * size + off, batch_buf.data_ptr() + r * size + off, ln))
                back.append((batch_buf.data_ptr() + r * size + off, echo_buf.data_ptr() + r * size + off, ln))
                off += ln
        n = len(items)
        if n > 8000:
            continue
        h_in, h_back = _C.sg_list_create(items), _C.sg_list_create(back)
        t_g = timed(lambda: _C.sg_list_launch(h_in, args.impl, 0, stream))
        t_e = timed(lambda: (_C.sg_list_launch(h_in, args.impl, 0, stream), _C.sg_list_launch(h_back, args.impl, 0, stream)))
        torch.cuda.synchronize()
        if size == sizes[0] and args.source != "peer":
            assert torch.equal(echo_buf[: size * args.batch].cpu(), src_t[: size * args.batch].cpu()), "echo mismatch"
        t_m = float("nan")
        if not args.no_baseline and n <= 2048:
            def memcpy_per_frag():
                for s, d, ln in items:
                    _C.memcpy_async(d, s, ln, stream)
            t_m = timed(memcpy_per_frag)
        _C.sg_list_destroy(h_in)
        _C.sg_list_destroy(h_back)
        if rank == 0:
            gbs = size * args.batch / t_g / 1e6
            print(f"{size:9d} {n:6d} {t_g * 1e3:10.1f} {gbs:8.1f} {gbs / peak:6.2f} {t_e * 1e3:9.1f} {t_m * 1e3:15.1f}")
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
