"""Headline benchmark: requests/s of dynamic-batched model serving, per GPU replica.

    python bench.py --gpus N --steps K --warmup W [--config resnet50|bert_base|lenet5|echo]

One process per GPU (launched under torchrun for N > 1; RANK/LOCAL_RANK/WORLD_SIZE
come from the environment).  Every rank serves one data-parallel replica of the
model on its GPU.  A "step" is one full batch (``max_batch`` requests) through
the serving path.  Two numbers are produced:

* ``value``: device-timed.  K steps of {scatter-gather kernel that pulls the
  batch's 8 KB fragments out of the pinned receive arena into the request ring,
  the model's CUDA graph, the response scatter kernel into the pinned transmit
  arena}, bracketed by CUDA events on the serving stream, max over ranks.
* ``e2e``: the same metric through the public serving API: the load generator
  sends fragmented requests over the loopback transport (an emulated NIC that
  DMA-writes into pinned host rings), the native server reassembles, gathers,
  batches dynamically, runs the graphs and sends responses, and the client
  receives them on the host.  The host->device bytes are the request fragments
  the GPU pulls from pinned memory; the device->host bytes are the responses.

Rank 0 prints one JSON line.  ``--impl reference`` reports why the original
server cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

CONFIGS = {
    "resnet50": dict(model="ResNet-50 v1.5 bf16 (BN folded), 3x224x224 fp32 requests in 8 KB fragments", max_batch=64,
                     payload="normal", seq=None),
    "bert_base": dict(model="BERT-base bf16 classifier, seq 128 int32 ids", max_batch=32, payload="ids", seq=128),
    "bert_large_tp": dict(model="BERT-large bf16 classifier, seq 384 int32 ids, tensor parallel over all GPUs",
                          max_batch=16, payload="ids", seq=384),
}


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.samples, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([f.strip() for f in line.split(",")])

    def stop(self) -> dict:
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
                for n, v in zip(names, s[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_model(config: str, device: int):
    if config == "resnet50":
        from splitrpc_b200.models import ResNet50

        return ResNet50(device=device, max_batch=CONFIGS[config]["max_batch"])
    if config == "lenet5":
        raise SystemExit("lenet5 is served by the built-in app: see tests/test_gpu_sg.py and serving.smoke_test")
    if config == "bert_base":
        from splitrpc_b200.models import BertClassifier, BERT_BASE

        return BertClassifier(BERT_BASE, seq=128, device=device, max_batch=CONFIGS[config]["max_batch"])
    raise SystemExit(f"unknown config {config}")


def device_timed(srv, steps: int, warmup: int):
    """K steps of gather -> graph -> response scatter, timed with CUDA events on the serving stream.

    The step is issued the way the server issues it: the gather of batch i+1 runs on the scatter-gather stream while
    the model graph of batch i runs on the work stream, over two windows of the request/response rings.  The timed
    region starts with both streams idle and ends when the last response scatter has finished, so it contains K
    gathers, K graphs, K scatters and K L2 flushes.
    """
    import torch

    from splitrpc_b200 import _C

    app, nb = srv.app, srv.max_batch
    req, resp = srv.req_size, srv.resp_size
    mtu = 8192
    n_sets = 2
    # Two batches worth of fragments in pinned, GPU-mapped host memory, one per ring window.
    pinned = torch.empty(n_sets * nb * req, dtype=torch.uint8).pin_memory()
    pinned.random_(0, 256) if req < 4096 else pinned.view(torch.float32).normal_()
    if srv.model.__class__.__name__ == "BertClassifier":
        pinned.view(torch.int32).random_(0, 30522)
    tx = torch.empty(n_sets * nb * max(resp, 16), dtype=torch.uint8).pin_memory()
    req_base, _, _ = app.req_ring
    resp_base, _, _ = app.resp_ring
    stubs = torch.empty(n_sets, 2, dtype=torch.int64).pin_memory()  # (request window, response window) per set
    lists, out_lists = [], []
    for s in range(n_sets):
        items = []
        for r in range(nb):
            off = 0
            while off < req:  # one item per 8 KB fragment, as the reassembly delivers them
                ln = min(mtu, req - off)
                items.append((pinned.data_ptr() + (s * nb + r) * req + off, req_base + (s * nb + r) * req + off, ln))
                off += ln
        lists.append(_C.sg_list_create(items))
        out_lists.append(_C.sg_list_create(
            [(resp_base + (s * nb + r) * resp, tx.data_ptr() + (s * nb + r) * resp, resp) for r in range(nb)]))
        stubs[s, 0] = req_base + s * nb * req
        stubs[s, 1] = resp_base + s * nb * resp
    stream = srv.stream
    sg_stream = torch.cuda.Stream(device=srv.device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=f"cuda:{srv.device}")
    total = warmup + steps
    gathered = [torch.cuda.Event() for _ in range(total)]
    done = [torch.cuda.Event() for _ in range(total)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def step(i):
        w = i % n_sets
        if i >= n_sets:
            sg_stream.wait_event(done[i - n_sets])  # the window's previous batch has been answered
        # PCIe-bound: a few 1024-thread blocks on the SMs that the model's persistent kernels leave free
        gb = -srv.reserve_sms if srv.reserve_sms > 0 else 48
        if srv.fused_ingress:  # gather + deserialise in one kernel, as the server's engine does
            _C.sg_list_launch_stem_s2d(lists[w], req_base, req, srv.ingress["mean"], srv.ingress["inv_std"], gb, sg_stream.cuda_stream)
        else:
            _C.sg_list_launch(lists[w], 0, gb, sg_stream.cuda_stream)
        gathered[i].record(sg_stream)
        stream.wait_event(gathered[i])
        # the stub is re-pointed in stream order, as the stream-armed server mode does
        _C.memcpy_async(app.d_stub, stubs[w].data_ptr(), 16, stream.cuda_stream)
        app.launch(nb)
        _C.sg_list_launch(out_lists[w], 0, 0, stream.cuda_stream)
        with torch.cuda.stream(stream):
            flush.zero_()  # L2 flush between iterations (inside the timed region)
        done[i].record(stream)

    for i in range(warmup):
        step(i)
    stream.synchronize()
    sg_stream.synchronize()
    t0.record(stream)
    sg_stream.wait_event(t0)
    for i in range(warmup, total):
        step(i)
    t1.record(stream)
    stream.synchronize()
    sg_stream.synchronize()
    app.set_stub()
    ms_total = t0.elapsed_time(t1)
    for h in lists + out_lists:
        _C.sg_list_destroy(h)
    return [ms_total / steps] * steps


def run_ours(args, rank: int, world: int, local_rank: int) -> dict:
    import torch

    from splitrpc_b200 import ops
    from splitrpc_b200.serving import ModelServer

    cfg = CONFIGS[args.config]
    nb = cfg["max_batch"]
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    model = build_model(args.config, local_rank)
    outstanding = 3 * nb  # closed-loop depth: one batch running, one being gathered, one in the clients' hands
    srv = ModelServer(model, device=local_rank, max_batch=nb, server_mode=2, copy_type=2, outstanding=outstanding)

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = device_timed(srv, args.steps, max(args.warmup, 3))
    barrier()
    total_ms = sum(ms)
    t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_total_ms = float(t.item())
    ops.check_status()
    value = world * nb * args.steps / (max_total_ms / 1e3)

    # ---- end to end through the public API
    barrier()
    n_req = nb * args.steps
    n_warm = nb * max(args.warmup, 3)
    srv.start()
    # Requests are sent by reference: the payload pool sits in pinned, GPU-mapped host memory (as a NIC's registered
    # buffers would) and only headers + descriptors cross the emulated wire; the GPU pulls every fragment of every
    # request out of that host memory each step.
    cli = srv.client(total=n_req + n_warm, warmup=n_warm, payload=cfg["payload"], n_payloads=outstanding, send_by_reference=True)
    barrier()
    ok = cli.run_closed_loop(outstanding)
    st = cli.post_process()
    clocks = sampler.stop()
    ws = srv.server.worker_stats(0)
    srv.stop()
    e2e_rps = st.get("throughput_est", 0.0) if ok else 0.0
    t2 = torch.tensor([e2e_rps, st.get("p50_sojournTime_us", 0.0), st.get("p99_sojournTime_us", 0.0)], device="cuda",
                      dtype=torch.float64)
    if dist:
        s = t2.clone()
        dist.all_reduce(s, op=dist.ReduceOp.SUM)
        m = t2.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX)
        e2e_total, p50, p99 = float(s[0]), float(m[1]), float(m[2])
    else:
        e2e_total, p50, p99 = float(t2[0]), float(t2[1]), float(t2[2])
    hist = ws["batch_hist"]
    mean_bs = sum(k * v for k, v in hist.items()) / max(1, sum(hist.values()))
    launches_per_step = 2 + model.kernels_per_forward
    wns = ws["work_ns"][len(ws["work_ns"]) // 4:]
    work_ms = sum(wns) / max(1, len(wns)) / 1e6  # host-observed graph launch + wait per batch on the worker thread
    result = {
        "metric": "req/s (dynamic batching, device-timed, max over ranks)", "value": round(value, 1), "unit": "req/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(max_total_ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "splitrpc_b200",
        "config": {"model": cfg["model"], "global_batch": nb * world, "seq_len": cfg["seq"], "parallelism": f"dp{world}",
                   "step": f"one batch of {nb} requests per GPU: gather fragments from pinned host arena + model graph + response scatter; the gather of batch i+1 overlaps the graph of batch i on a second stream, as in the server",
                   "l2": "256 MiB buffer written between iterations, inside the timed region; inputs alternate between two pinned host sets",
                   "weights": "random init"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_total, 1), "unit": "req/s", "h2d_bytes_per_step": nb * srv.req_size,
                "d2h_bytes_per_step": nb * srv.resp_size, "p50_us": round(p50, 1), "p99_us": round(p99, 1),
                "mean_batch": round(mean_bs, 2), "worker_ms_per_batch": round(work_ms, 3), "requests": n_req, "outstanding": outstanding,
                "path": "loadgen (fragments in pinned host memory, sent by reference) -> loopback NIC -> native server "
                        "(reassembly, steering, dynamic batching) -> SG kernel pulls fragments over PCIe -> CUDA graph -> "
                        "SG kernel writes responses to the pinned transmit arena -> client"},
        "gpu_launches": launches_per_step * args.steps,
    }
    if dist:
        dist.destroy_process_group()
    return result


def run_tp(args, rank: int, world: int, local_rank: int) -> dict:
    """BERT-large, one batch of 16 x 384 tokens per step, all GPUs cooperating on every batch (tensor parallel)."""
    import torch
    import torch.distributed as dist

    from splitrpc_b200 import ops
    from splitrpc_b200.models import BERT_LARGE, BertClassifierTP
    from splitrpc_b200.parallel import init_distributed

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    init_distributed()
    cfg = CONFIGS[args.config]
    B, S = cfg["max_batch"], cfg["seq"]
    model = BertClassifierTP(BERT_LARGE, seq=S, device=local_rank, batch=B)
    dev = torch.device("cuda", local_rank)
    warm = max(args.warmup, 3)
    n_sets = 4
    ids_host = [torch.randint(0, 30522, (B, S), dtype=torch.int32, generator=torch.Generator().manual_seed(i)).pin_memory()
                for i in range(n_sets)]
    ids_dev = torch.zeros((B, S), dtype=torch.int32, device=dev)
    probs = torch.zeros((B, 2), dtype=torch.float32, device=dev)
    probs_host = torch.zeros((B, 2), dtype=torch.float32).pin_memory()
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        model.forward(ids_dev, out=probs)  # warm-up outside capture (sets kernel attributes)
        stream.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            model.forward(ids_dev, out=probs)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sampler = ClockSampler(local_rank)

    def one_step(i):
        graph.replay()

    results = {}
    with torch.cuda.stream(stream):
        for i in range(warm):
            one_step(i)
        stream.synchronize()
        dist.barrier()
        sampler.start()
        evs = []
        for i in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            one_step(i)
            e1.record(stream)
            evs.append((e0, e1))
        stream.synchronize()
        dist.barrier()
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results["device"] = float(t.item())
    # ---- end to end: closed-loop clients -> RPC front end on rank 0 -> control broadcast -> TP graph on every rank
    from splitrpc_b200.serving.tp_server import TensorParallelServer

    srv = TensorParallelServer(model, outstanding=2 * B)
    n_req, n_warm = B * args.steps, B * warm
    stats = torch.zeros(4, dtype=torch.float64, device=dev)
    if rank == 0:
        with srv:
            cli = srv.client(total=n_req + n_warm, warmup=n_warm, payload="ids", n_payloads=2 * B, send_by_reference=True)
            ok = cli.run_closed_loop(2 * B)
            st = cli.post_process()
        if ok:
            stats[0], stats[1], stats[2] = st.get("throughput_est", 0.0), st.get("p50_sojournTime_us", 0.0), st.get("p99_sojournTime_us", 0.0)
        stats[3] = srv.served_batches
    else:
        srv.serve_forever()
    dist.barrier()
    dist.broadcast(stats, src=0)
    e2e_rps, e2e_p50, e2e_p99, e2e_batches = (float(v) for v in stats)
    clocks = sampler.stop()
    ops.check_status()
    value = B * args.steps / (results["device"] / 1e3)
    res = {
        "metric": "req/s (tensor-parallel batch serving, device-timed, max over ranks)", "value": round(value, 1),
        "unit": "req/s", "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(results["device"] / args.steps, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "splitrpc_b200",
        "config": {"model": cfg["model"], "global_batch": B, "seq_len": S, "parallelism": f"tp{world}",
                   "step": "one batch of 16 sequences through the tensor-parallel CUDA graph on all ranks",
                   "l2": "256 MiB buffer written between timed iterations", "weights": "random init"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_rps, 1), "unit": "req/s", "h2d_bytes_per_step": B * S * 4, "d2h_bytes_per_step": B * 16,
                "p50_us": round(e2e_p50, 1), "p99_us": round(e2e_p99, 1),
                "mean_batch": round((n_req + n_warm) / max(1.0, e2e_batches), 2), "outstanding": 2 * B,
                "path": "loadgen (ids in pinned host memory, sent by reference) -> loopback NIC -> native server on rank 0 "
                        "(reassembly, dynamic batching, SG kernel pulls the ids over PCIe) -> control broadcast to the "
                        "peers -> TP graph on every rank -> probabilities to the pinned transmit arena -> client"},
        "gpu_launches": model.kernels_per_forward * args.steps,
    }
    dist.barrier()
    dist.destroy_process_group()
    return res


def run_reference(args, rank: int, world: int, local_rank: int) -> dict:
    """The original's data path, re-hosted: see baseline/reference_arm.py.  Imports nothing of this package."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    try:
        import reference_arm

        return reference_arm.run(args, rank, world, local_rank, CONFIGS[args.config])
    except Exception as e:  # noqa: BLE001 - the arm must answer with one JSON line and exit 0
        return {"impl": "reference", "unavailable": f"reference arm failed: {type(e).__name__}: {str(e)[:300]}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="resnet50", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        res = run_reference(args, rank, world, local_rank)
        if rank == 0:
            print(json.dumps(res), flush=True)
        return
    res = run_tp(args, rank, world, local_rank) if args.config == "bert_large_tp" else run_ours(args, rank, world, local_rank)
    if rank == 0:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
