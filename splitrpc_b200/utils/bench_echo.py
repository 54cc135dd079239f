"""Echo / scatter-gather sweep through the public serving path (``bench.py --config echo``).

For every payload size from 64 B to 4 MB (powers of two) the requests are cut into 8 KB fragments, sent over the
loopback transport, reassembled by rank 0, gathered by GPU 0's scatter-gather kernel into the request ring of an
echo app on one of the N GPUs (its own, or a peer's over NVLink), echoed by that GPU and returned: single-fragment
responses are stored into the ingress transmit arena by the serving GPU itself, larger ones are read back from the
response ring (for a peer: over NVLink) by GPU 0's scatter kernel.  Every reply is verified byte for byte.  One
process per GPU; rank 0 is the ingress.  The original's counterpart is its echo app behind the copy engine
(reference ``src/apps/echo_rpc_bench.cc:25-36``, ``src/transport/g_copy_ng.cu:114-144``).
"""
from __future__ import annotations

import os
import tempfile
import time

MTU = 8192
FUNC = 4242
PCIE_GBS = 55.0


def _path(rank: int, size: int) -> str:
    return os.path.join(tempfile.gettempdir(), f"splitrpc_echo_{os.environ.get('MASTER_PORT', str(os.getpid()))}_{rank}_{size}.sock")


def device_timed_echo(app, size: int, batch: int, device: int, iters: int = 12) -> float:
    """Server-side rate of one GPU without the emulated wire and the client: for a batch of `batch` requests of `size`
    bytes, the gather kernel pulls the 8 KB fragments out of pinned host memory into the request ring, the echo app
    copies them into the response ring, the scatter kernel writes the responses back to pinned host memory in 8 KB
    fragments; two windows alternate so that the host-to-device traffic of one batch overlaps the device-to-host traffic
    of the other.  Returns payload GB/s (request bytes per second), CUDA events.  This is what the original's echo
    figure measures (its copy kernels and its echo copy, no network)."""
    import torch

    from .. import _C

    torch.cuda.set_device(device)
    app.disable_device_completion()
    app.reset_slots()
    req_base, resp_base = app.req_ring[0], app.resp_ring[0]
    n_win = 2
    src = torch.empty(n_win * batch * size, dtype=torch.uint8).pin_memory()
    dst = torch.zeros(n_win * batch * size, dtype=torch.uint8).pin_memory()
    src.random_(0, 256)
    work = torch.cuda.ExternalStream(app.work_stream, device=torch.device("cuda", device))
    side = [torch.cuda.Stream(device=device) for _ in range(n_win)]
    gathers, scatters = [], []
    for w in range(n_win):
        gi, si = [], []
        for r in range(batch):
            off = 0
            while off < size:
                ln = min(MTU, size - off)
                k = (w * batch + r) * size + off
                gi.append((src.data_ptr() + k, req_base + k, ln))
                si.append((resp_base + k, dst.data_ptr() + k, ln))
                off += ln
        gathers.append(_C.sg_list_create(gi))
        scatters.append(_C.sg_list_create(si))
    ev_g = [torch.cuda.Event() for _ in range(n_win)]
    ev_a = [torch.cuda.Event() for _ in range(n_win)]
    ev_s = [torch.cuda.Event() for _ in range(n_win)]

    def step(i):
        w = i % n_win
        s = side[w]
        s.wait_event(ev_s[w]) if i >= n_win else None
        _C.sg_list_launch(gathers[w], 0, 48, s.cuda_stream)
        ev_g[w].record(s)
        work.wait_event(ev_g[w])
        app.stage_window(req_base + w * batch * size, resp_base + w * batch * size, w * batch, batch)
        app.launch(batch)
        ev_a[w].record(work)
        s.wait_event(ev_a[w])
        _C.sg_list_launch(scatters[w], 0, 48, s.cuda_stream)
        ev_s[w].record(s)

    for i in range(4):
        step(i)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(work)
    for s in side:
        s.wait_event(t0)
    for i in range(4, 4 + iters):
        step(i)
    for s in side:
        work.wait_stream(s)
    t1.record(work)
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    ok = bool(torch.equal(src, dst))
    for h in gathers + scatters:
        _C.sg_list_destroy(h)
    app.reset_slots()
    if not ok:
        raise RuntimeError("device-timed echo: the scattered responses differ from the requests")
    return iters * batch * size / (ms * 1e-3) / 1e9


def run_echo(args, rank: int, world: int, local_rank: int, sizes=None) -> dict | None:
    import torch

    from .. import _C, ops

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("gloo")
    _C.set_rpc_mtu(MTU)
    sizes = sizes or [1 << k for k in range(6, 23)]
    sweep = []
    for size in sizes:
        frags = (size + MTU - 1) // MTU
        batch = 64 if size <= (1 << 18) else (16 if size <= (1 << 20) else 8)
        outstanding = 2 * batch * world
        pool = max(64, 4 * batch)
        app = _C.make_app("echo", local_rank, size, size, [], pool, 1, batch, "gpu", 2)
        dev_gbs = device_timed_echo(app, size, batch, local_rank) if rank == 0 else None
        bs = None
        if rank > 0:
            bs = _C.BatchedServer(app, _path(rank, size), func_id=FUNC, server_mode=2, max_batch=batch)
            bs.start()
        if dist:
            dist.barrier()
        if rank == 0:
            n_slots = max(1024, 3 * outstanding * frags)
            sp, cp = _C.make_loopback_pair(MTU, n_slots, "shm_pinned")
            srv = _C.Server(sp, req_size=size, resp_size=size, server_mode=2, max_batch=batch, gather_burst=batch,
                            rr_pool_size=max(1023, 4 * outstanding))
            srv.add_replica(app)
            for r in range(1, world):
                srv.add_remote_replica(_path(r, size), func_id=FUNC, ingress_device=local_rank, copy_type=2)
            srv.start()
            # about a third of a second per size at the PCIe rate, at least a few batches per replica
            n_req = int(max(8 * batch * world, min(200000, 0.3 * PCIE_GBS * 1e9 / max(size, 4096))))
            n_warm = max(batch * world, n_req // 10)
            cli = _C.Client(cp, req_size=size, resp_size=size, total=n_req + n_warm, warmup=n_warm, payload="echo", verify=True,
                            n_payloads=min(outstanding, 64), send_by_reference=True)
            t0 = time.perf_counter()
            ok = cli.run_closed_loop(outstanding)
            wall = time.perf_counter() - t0
            st = cli.post_process()
            ss = srv.stats()
            srv.stop()
            srv.release_remotes()
            rps = st.get("throughput_est", 0.0) if ok else 0.0
            sweep.append({"bytes": size, "fragments": frags, "batch": batch, "req_s": round(rps, 1),
                          "gather_gbs": round(rps * size / 1e9, 3), "p50_us": round(st.get("p50_sojournTime_us", 0.0), 1),
                          "p99_us": round(st.get("p99_sojournTime_us", 0.0), 1), "verified": bool(ok and cli.verify_failures == 0),
                          "pushed": sum(r["pushed"] for r in ss["replicas"]), "steered": [r["steered"] for r in ss["replicas"]],
                          "of_pcie": round(rps * size / 1e9 / PCIE_GBS, 3), "seconds": round(wall, 3),
                          "server_side_gbs": round(dev_gbs, 3)})
            del cli, srv, sp, cp
        if dist:
            dist.barrier()
        if bs is not None:
            bs.stop()
        del app
    ops.check_status()
    res = None
    if rank == 0:
        big = max(sweep, key=lambda s: s["gather_gbs"])
        big_dev = max(sweep, key=lambda s: s["server_side_gbs"])
        res = {"metric": "payload GB/s gathered into GPU batch buffers and echoed (best size of the sweep), end to end", "value": big["gather_gbs"],
               "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "uint8", "data": "synthetic",
               "impl": "splitrpc_b200",
               "config": {"model": "echo app on every GPU behind one ingress, 64 B - 4 MB payloads in 8 KB fragments", "global_batch": None,
                          "seq_len": None, "parallelism": f"dp{world}, single ingress" if world > 1 else "dp1",
                          "roofline": f"every request crosses GPU 0's PCIe link once in and once out: {PCIE_GBS} GB/s measured per direction"},
               "server_side": {"value": big_dev["server_side_gbs"], "unit": "GB/s", "bytes": big_dev["bytes"],
                               "what": "GPU 0 alone, CUDA events: gather kernel from pinned host memory -> echo app -> scatter kernel "
                                       "back to pinned host memory, two batches in flight (no emulated wire, no client): the "
                                       "quantity the original's echo figure measures"},
               "sweep": sweep, "all_verified": all(s["verified"] for s in sweep)}
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return res
