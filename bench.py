"""Headline benchmark: requests/s of dynamic-batched model serving behind ONE ingress.

    python bench.py --gpus N --steps K --warmup W [--config resnet50|bert_base|bert_large_tp|lenet5|echo]
                    [--impl ours|reference] [--slo-ms 10]

One process per GPU (launched under torchrun for N > 1; RANK/LOCAL_RANK/WORLD_SIZE come from the environment).
Rank 0 is the ingress: it owns the loopback transport (an emulated NIC that DMA-writes into pinned host rings which
GPU 0 maps), parses headers, reassembles and steers.  Every rank serves one data-parallel replica of the model on its
GPU; the replicas of ranks > 0 sit behind batched servers that handed their request rings and slot doorbells to rank 0.
A "step" is one full batch (``max_batch`` requests) per GPU.  Numbers:

* ``value`` (device-timed, single ingress): K steps of one batch per GPU, no host thread between a batch's first
  doorbell and its last completion; CUDA events on every rank's serving stream, max over ranks.  For N > 1 two ways of
  feeding the replicas of ranks > 0 are measured (``--ingress both``) and the faster is the headline, the other is
  reported under ``ingress_push`` / ``ingress_pull``:
  push  GPU 0's scatter-gather kernel pulls a batch's 8 KB fragments out of the pinned arena, deserialises them,
        stores them into the serving GPU's request ring over NVLink and rings the slot doorbells; the serving GPU's
        stream, parked on the last doorbell, runs the model's CUDA graph, whose last kernel stores the responses into
        the ingress transmit arena and completes the slots.  Every request crosses GPU 0's PCIe link.
  pull  rank 0 shares its payload memory with the replicas (descriptors at ALLOC time) and only describes each
        request; every serving GPU's own gather kernel fetches its batch over its own PCIe link, beside the graph of
        the previous batch.  Responses are stored and completed the same way.
* ``e2e``: the same metric through the public serving API: the load generator sends fragmented requests over the
  loopback transport, the native server reassembles, steers, gathers; the replicas batch dynamically and answer; the
  client receives the responses on the host.  Host->device bytes are the request fragments GPU 0 pulls from pinned
  memory; device->host bytes are the responses.  Run for about two seconds, with the payloads handed over by
  reference (registered buffers) and, for comparison, copied into the receive arena by the emulated DMA.
* ``ingress_per_gpu``: the earlier arrangement, every GPU with its own transport, server and load generator (N
  independent single-GPU servers), device-timed and end to end, as a second, labelled number.

Rank 0 prints one JSON line.  ``--impl reference`` runs the original's data path (see baseline/reference_arm.py).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

CONFIGS = {
    "resnet50": dict(model="ResNet-50 v1.5 bf16 (BN folded), 3x224x224 fp32 requests in 8 KB fragments", max_batch=64,
                     payload="normal", seq=None),
    "bert_base": dict(model="BERT-base bf16 classifier, seq 128 int32 ids", max_batch=32, payload="ids", seq=128),
    "bert_large_tp": dict(model="BERT-large bf16 classifier, seq 384 int32 ids, tensor parallel over all GPUs",
                          max_batch=16, payload="ids", seq=384),
    "lenet5": dict(model="LeNet-5 fp32 on the CPU device, 1x28x28 fp32 requests (3136 B, one fragment)", max_batch=32,
                   payload="uniform", seq=None),
    "echo": dict(model="echo / scatter-gather microbenchmark, 64 B - 4 MB payloads in 8 KB fragments", max_batch=64,
                 payload="echo", seq=None),
}
RX_COMPLETE, WORK_COMPLETE = 1, 2
PCIE_GBS = 55.0      # measured rate of one large pinned-host -> GPU copy on these machines
NVLINK_GBS = 770.0   # measured peer copy rate per direction
DMA_LANES = 4        # copy threads of the emulated NIC in the copy-mode end-to-end run


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
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), [f.strip() for f in line.split(",")]))

    def mark(self) -> float:
        return time.perf_counter()

    def summary(self, t_from: float | None = None, t_to: float | None = None, _widened: bool = False) -> dict:
        sm, mx, pw, reasons = [], 0, [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for t, s in list(self.samples):
            if (t_from is not None and t < t_from) or (t_to is not None and t > t_to):
                continue
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
                pw.append(float(s[2]))
                for n, v in zip(names, s[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        out = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
               "samples": len(sm), "power_w_max": max(pw) if pw else None}
        if not sm and t_from is not None and t_to is not None and not _widened:
            # a timed region shorter than the sampling period: the samples just around it (the GPU is under the same
            # load right before, in the warm-up steps, and right after)
            out = self.summary(t_from - 0.3, t_to + 0.3, _widened=True)
            out["window"] = "within 0.3 s of the timed region (none fell inside it)"
        return out

    def stop(self) -> dict:
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return self.summary()


def build_model(config: str, device: int):
    if config == "resnet50":
        from splitrpc_b200.models import ResNet50

        return ResNet50(device=device, max_batch=CONFIGS[config]["max_batch"])
    if config == "bert_base":
        from splitrpc_b200.models import BertClassifier, BERT_BASE

        return BertClassifier(BERT_BASE, seq=128, device=device, max_batch=CONFIGS[config]["max_batch"])
    raise SystemExit(f"unknown model config {config}")


def sock_path(rank: int) -> str:
    return os.path.join(tempfile.gettempdir(), f"splitrpc_bench_{os.environ.get('MASTER_PORT', str(os.getpid()))}_{rank}.sock")


# ----------------------------------------------------------------------------------------------- device-timed
def device_timed_single_ingress(node, rank: int, world: int, steps: int, warmup: int, barrier, payload_kind: str):
    """K steps of the doorbell-driven pipeline described in the module docstring.  ``node`` is the ModelServer (rank 0,
    remotes already added, server not started) or the ModelReplica (ranks > 0, batched server without a worker).
    Returns this rank's CUDA-event time for the K steps in ms and the number of kernels it launched in them."""
    import torch

    from splitrpc_b200 import _C

    app, nb, req, resp = node.app, node.max_batch, node.req_size, node.resp_size
    dev = torch.device("cuda", node.device)
    # three ring windows per replica: one being computed, one gathered and waiting, one being gathered
    n_sets, mtu, total = 3, 8192, warmup + steps
    stream = node.stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    req_base, resp_base = app.req_ring[0], app.resp_ring[0]
    if rank == 0:
        app.reset_slots()
    launches = 0
    produce = None
    lists = []
    if rank == 0:
        srv = node.server
        _, tx_dev, tx_bytes, tx_slot = srv.tx_arena
        assert world * n_sets * nb * tx_slot <= tx_bytes, "transmit arena too small for the timing loop"
        pinned = torch.empty(n_sets * world * nb * req, dtype=torch.uint8).pin_memory()
        if payload_kind == "ids":
            pinned.view(torch.int32).random_(0, 30522)
        else:
            pinned.view(torch.float32).normal_()
        sg_streams = [torch.cuda.Stream(device=dev) for _ in range(world)]  # one per replica: no head-of-line blocking
        rings = [dict(req_base=req_base, states_dev=app.states_dev)] + [srv.remote_rings(r - 1) for r in range(1, world)]
        for r in range(world):
            per_w = []
            for w in range(n_sets):
                items, bells = [], []
                for j in range(nb):
                    src = pinned.data_ptr() + ((w * world + r) * nb + j) * req
                    dst = rings[r]["req_base"] + (w * nb + j) * req
                    off = 0
                    while off < req:  # one item per 8 KB fragment, as the reassembly delivers them
                        ln = min(mtu, req - off)
                        items.append((src + off, dst + off, ln))
                        off += ln
                    bells.append(rings[r]["states_dev"] + 4 * (w * nb + j))
                    tx_off = ((r * n_sets + w) * nb + j) * tx_slot
                    if r == 0:
                        app.set_tx_off(w * nb + j, tx_off)
                    else:
                        srv.remote_set_tx_off(r - 1, w * nb + j, tx_off)
                per_w.append(_C.sg_list_create(items, bells))
            lists.append(per_w)
        gb = -node.reserve_sms if node.reserve_sms > 0 else 48  # PCIe-bound: a few fat blocks on the reserved SMs

        def produce(i):
            w = i % n_sets
            for r in range(world):
                sg = sg_streams[r].cuda_stream
                if i >= n_sets:  # the replica has consumed what this window held n_sets steps ago
                    _C.stream_wait32(sg, rings[r]["states_dev"] + 4 * (w * nb + nb - 1), WORK_COMPLETE)
                if node.fused_ingress:  # gather + deserialise + doorbells in one kernel, as the server's engine does
                    _C.sg_list_launch_stem_s2d(lists[r][w], rings[r]["req_base"], req, node.ingress["mean"], node.ingress["inv_std"],
                                               gb, sg, bell_value=RX_COMPLETE)
                else:
                    _C.sg_list_launch(lists[r][w], 0, gb, sg, bell_value=RX_COMPLETE)
            return world

    def consume(i):
        w = i % n_sets
        st = stream.cuda_stream
        _C.stream_wait32(st, app.states_dev + 4 * (w * nb + nb - 1), RX_COMPLETE)
        # re-point what the graph's kernels read (request / response window, first slot, where each response goes) in
        # stream order: one small kernel behind the doorbell wait, as the stream-armed worker queues it
        app.stage_window(req_base + w * nb * req, resp_base + w * nb * resp, w * nb, nb, armed=True)
        app.launch(nb)  # the graph; its last kernel stores the responses into rank 0's arena and completes the slots
        with torch.cuda.stream(stream):
            flush.zero_()  # L2 flush between iterations (inside the timed region)
        return node.model.kernels_per_forward + 1  # + the window update

    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        flush.zero_()  # loads the fill kernel before the stream is first parked on a doorbell
    stream.synchronize()
    for i in range(warmup):
        if produce:
            produce(i)
        consume(i)
    stream.synchronize()
    barrier()
    t0.record(stream)
    for i in range(warmup, total):
        if produce:
            launches += produce(i)
        launches += consume(i)
    t1.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    barrier()
    ok = all(app.slot_state(s) == WORK_COMPLETE for s in range(n_sets * nb))
    for per_w in lists:
        for h in per_w:
            _C.sg_list_destroy(h)
    if not ok:
        raise RuntimeError("device-timed loop: a slot was not completed by the serving GPU")
    return ms, launches


def fill_payload(host_addr: int, nbytes: int, kind: str):
    """Synthetic request bytes at a host address (a shared region that torch did not allocate)."""
    import ctypes

    import numpy as np

    buf = np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(host_addr))
    rng = np.random.default_rng(7)
    if kind == "ids":
        buf.view(np.int32)[:] = rng.integers(0, 30522, nbytes // 4, dtype=np.int32)
    else:
        buf.view(np.float32)[:] = rng.standard_normal(nbytes // 4, dtype=np.float32)


def device_timed_per_gpu(srv, steps: int, warmup: int, src_base: int | None = None, tx_off0: int = 0, tx_slot: int | None = None):
    """This GPU gathers its own batches from pinned host memory over its own PCIe link (gather of batch i+1 on a second
    stream beside the graph of batch i) and runs the graph, whose last kernel stores the responses into the transmit
    arena.  CUDA events on the serving stream.  ``src_base``: device-side address of 2 x max_batch requests in host
    memory (the ingress's shared payload region, as this process maps it); None: a pinned buffer of this process (the
    independent arrangement).  ``tx_off0`` / ``tx_slot``: where this GPU's responses go in the transmit arena."""
    import torch

    from splitrpc_b200 import _C

    app, nb, req, resp = srv.app, srv.max_batch, srv.req_size, srv.resp_size
    mtu, n_sets = 8192, 2
    if src_base is None:
        pinned = torch.empty(n_sets * nb * req, dtype=torch.uint8).pin_memory()
        pinned.view(torch.float32).normal_() if req >= 4096 else pinned.view(torch.int32).random_(0, 30522)
        src_base = pinned.data_ptr()
    req_base, resp_base = app.req_ring[0], app.resp_ring[0]
    if tx_slot is None:
        tx_slot = srv.server.tx_arena[3]
    app.reset_slots()
    stubs = torch.empty(n_sets, 2, dtype=torch.int64).pin_memory()
    first = torch.empty(n_sets, dtype=torch.int32).pin_memory()
    lists = []
    for s in range(n_sets):
        items = []
        for r in range(nb):
            off = 0
            while off < req:
                ln = min(mtu, req - off)
                items.append((src_base + (s * nb + r) * req + off, req_base + (s * nb + r) * req + off, ln))
                off += ln
            app.set_tx_off(s * nb + r, tx_off0 + (s * nb + r) * tx_slot)
        lists.append(_C.sg_list_create(items))
        stubs[s, 0], stubs[s, 1], first[s] = req_base + s * nb * req, resp_base + s * nb * resp, s * nb
    stream = srv.stream
    sg_stream = torch.cuda.Stream(device=srv.device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=f"cuda:{srv.device}")
    total = warmup + steps
    gathered = [torch.cuda.Event() for _ in range(total)]
    done = [torch.cuda.Event() for _ in range(total)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gb = -srv.reserve_sms if srv.reserve_sms > 0 else 48

    def step(i):
        w = i % n_sets
        if i >= n_sets:
            sg_stream.wait_event(done[i - n_sets])
        if srv.fused_ingress:
            _C.sg_list_launch_stem_s2d(lists[w], req_base, req, srv.ingress["mean"], srv.ingress["inv_std"], gb, sg_stream.cuda_stream)
        else:
            _C.sg_list_launch(lists[w], 0, gb, sg_stream.cuda_stream)
        gathered[i].record(sg_stream)
        stream.wait_event(gathered[i])
        app.stage_window(int(stubs[w, 0]), int(stubs[w, 1]), int(first[w]), nb)
        app.launch(nb)
        with torch.cuda.stream(stream):
            flush.zero_()
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
    ms = t0.elapsed_time(t1)
    ok = all(app.slot_state(s) == WORK_COMPLETE for s in range(n_sets * nb))
    app.reset_slots()
    for h in lists:
        _C.sg_list_destroy(h)
    if not ok:
        raise RuntimeError("device-timed loop: a slot was not completed by the serving GPU")
    return ms


# ----------------------------------------------------------------------------------------------- end to end
def closed_loop(srv, n_req: int, n_warm: int, outstanding: int, payload: str, by_reference: bool) -> dict:
    cli = srv.client(total=n_req + n_warm, warmup=n_warm, payload=payload, n_payloads=min(outstanding, 256),
                     send_by_reference=by_reference)
    t0 = time.perf_counter()
    ok = cli.run_closed_loop(outstanding)
    wall = time.perf_counter() - t0
    st = cli.post_process()
    # throughput_est = completed measured requests / (last completion - first dispatch): it stays meaningful when a
    # handful of requests never complete (the loop then ends by its drain timeout and `ok` is false); more than 0.1 %
    # lost counts as a failed run
    received, total = int(cli.received), n_req + n_warm
    usable = ok or received >= 0.999 * total
    return {"ok": bool(ok), "rps": st.get("throughput_est", 0.0) if usable else 0.0, "p50_us": st.get("p50_sojournTime_us", 0.0),
            "p99_us": st.get("p99_sojournTime_us", 0.0), "requests": n_req, "seconds": round(wall, 3), "received": received,
            "lost": total - received}


class PerGpuIngress:
    """A per-GPU ingress around the already captured app of a ModelReplica (second, labelled number of the bench)."""

    def __init__(self, rep, outstanding: int):
        import math

        from splitrpc_b200 import _C

        self.app, self.model, self.device, self.max_batch = rep.app, rep.model, rep.device, rep.max_batch
        self.stream, self.req_size, self.resp_size = rep.stream, rep.req_size, rep.resp_size
        self.fused_ingress, self.ingress, self.reserve_sms = rep.fused_ingress, rep.ingress, rep.reserve_sms
        self.app.reset_slots()
        frags = math.ceil(self.req_size / 8192) + math.ceil(self.resp_size / 8192)
        self.server_port, self.client_port = _C.make_loopback_pair(8192, max(1024, 2 * outstanding * frags), "shm_pinned")
        if self.fused_ingress:
            self.app.set_ingress_stem_s2d(self.ingress["mean"], self.ingress["inv_std"])
        self.server = _C.Server(self.server_port, req_size=self.req_size, resp_size=self.resp_size, server_mode=2,
                                max_batch=self.max_batch, rr_pool_size=max(1023, 4 * outstanding), gather_burst=self.max_batch)
        self.server.add_replica(self.app)

    def start(self):
        self.server.start()

    def stop(self):
        self.server.stop()

    def client(self, total, warmup, payload, **kw):
        from splitrpc_b200 import _C

        return _C.Client(self.client_port, req_size=self.req_size, resp_size=self.resp_size, total=total, warmup=warmup,
                         payload=payload, verify=False, **kw)


def run_ours(args, rank: int, world: int, local_rank: int) -> dict:
    import torch

    from splitrpc_b200 import _C, ops
    from splitrpc_b200.serving import ModelReplica, ModelServer

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    cfg = CONFIGS[args.config]
    nb = cfg["max_batch"]
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    warm = max(args.warmup, 3)
    model = build_model(args.config, local_rank)
    # closed-loop depth per replica: one batch running, one being gathered, one in the clients' hands
    outstanding = 3 * nb * world
    pool = max(256, 4 * nb)

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()

    def allmax(v: float) -> float:
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def allsum(v: float) -> float:
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if dist:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- roles: rank 0 = ingress + replica, the others = replicas behind batched servers
    if rank == 0:
        # When GPU 0 gathers for every replica ("push"), the gather that also deserialises ResNet images needs about 24
        # SMs to run at the PCIe rate (12 are enough when it only feeds its own replica), so the model kernels of GPU 0
        # leave 24 SMs to it; when every replica fetches its own requests ("pull"), every GPU leaves 12.
        node = ModelServer(model, device=local_rank, max_batch=nb, server_mode=2, copy_type=2, outstanding=outstanding,
                           pool_size=pool, n_replicas=world, reserve_sms=12 if world == 1 else 24,
                           steer_policy=0 if world == 1 else 1)
    else:
        node = ModelReplica(model, sock_path(rank), device=local_rank, max_batch=nb, server_mode=-1, pool_size=pool,
                            reserve_sms=12)
    sampler = ClockSampler(local_rank)
    sampler.start()
    mtu, n_sets = 8192, 2

    def measure(mode: str) -> dict:
        """Device-timed loop and end-to-end run with the replicas of ranks > 0 fed in `mode`: "push" = GPU 0's gather
        kernel stores every request into the serving GPU's ring over NVLink; "pull" = rank 0 only describes where the
        fragments are and every serving GPU fetches them from the shared host memory over its own PCIe link."""
        pull = mode == "pull"
        out = {"mode": mode}
        src_dev = 0
        if rank == 0:
            node.recapture(12 if pull or world == 1 else 24)
            node.new_server(server_mode=2, outstanding=outstanding, n_replicas=world, steer_policy=0 if world == 1 else 1)
            if pull:
                # the requests of the timing loop: one shared, pinned region of the ingress port, 2 windows per GPU
                region = _C.alloc_dma_region(node.client_port, world * n_sets * nb * node.req_size)
                fill_payload(region[0], region[2], cfg["payload"])
                src_dev = region[1]
        else:
            node.serve(server_mode=-1)
            node.start()
        barrier()
        if rank == 0:
            for r in range(1, world):
                node.add_remote(sock_path(r), pull=pull)
                if bool(node.server.remote_info(r - 1)["pull"]) != pull:
                    raise RuntimeError("the replica did not accept the requested ingress mode")
        barrier()
        m0 = sampler.mark()
        if pull:
            if rank > 0:
                src_dev = node.batched.regions()[1][0]  # region 0 is the receive arena, 1 the buffer allocated above
            per_rank = n_sets * nb
            ms = device_timed_per_gpu(node, args.steps, warm, src_base=src_dev + rank * per_rank * node.req_size,
                                      tx_off0=rank * per_rank * mtu, tx_slot=mtu)
            launches = (model.kernels_per_forward + 2) * args.steps
        else:
            ms, launches = device_timed_single_ingress(node, rank, world, args.steps, warm, barrier, cfg["payload"])
        m1 = sampler.mark()
        out["max_ms"] = allmax(ms)
        out["launches"] = int(allsum(launches))
        out["clocks"] = sampler.summary(m0, m1)
        ops.check_status()
        out["value"] = world * nb * args.steps / (out["max_ms"] / 1e3)

        # ---- end to end through the public API
        if rank == 0:
            node.stop()  # releases the worker-less batched servers
        barrier()
        if rank > 0:
            node.serve(server_mode=2)
            node.start()
        barrier()
        e2e = {}
        n_req = int(min(400000, max(nb * args.steps * world, args.e2e_seconds * out["value"])))
        n_warm = max(nb * warm * world, n_req // 20)
        m2 = m3 = sampler.mark()
        if rank == 0:
            node.new_server(server_mode=2, outstanding=outstanding, n_replicas=world, steer_policy=0 if world == 1 else 1)
            for r in range(1, world):
                node.add_remote(sock_path(r), pull=pull)
            node.start()
            m2 = sampler.mark()
            e2e["ref"] = closed_loop(node, n_req, n_warm, outstanding, cfg["payload"], True)
            m3 = sampler.mark()
            st = node.server.stats()
            ws = [node.server.worker_stats(i) for i in range(world)]
            lat = sorted(node.server.device_latency_ns())
            e2e["dev_lat"] = [lat[round(q * (len(lat) - 1))] / 1e3 if lat else None for q in (0.5, 0.99)] + [len(lat)]
            # the emulated NIC writes the fragments of a request with four copy lanes (a NIC's DMA engines do not run on
            # the sending thread either)
            _C.set_loopback_dma_lanes(node.client_port, DMA_LANES)
            e2e["copy"] = closed_loop(node, max(nb * world * 4, n_req // 4), max(nb, n_warm // 4), outstanding, cfg["payload"], False)
            _C.set_loopback_dma_lanes(node.client_port, 1)
            e2e["pushed"] = sum(r["pushed"] for r in st["replicas"])
            e2e["steered"] = [r["steered"] for r in st["replicas"]]
            e2e["sg_errors"] = st["sg_errors"]
            hist = ws[0]["batch_hist"]
            e2e["mean_batch_replica0"] = sum(k * v for k, v in hist.items()) / max(1, sum(hist.values()))
            e2e["batches"] = [w["num_batches"] for w in ws]
            node.stop()
        barrier()
        out["clocks_e2e"] = sampler.summary(m2, m3)
        if rank > 0:
            node.stop()
        out["e2e"] = e2e
        out["n_req"] = n_req
        return out

    modes = ["push"] if world == 1 else (["pull", "push"] if args.ingress == "both" else [args.ingress])
    runs = {m: measure(m) for m in modes}
    head = max(runs.values(), key=lambda r: r["value"])  # the same on every rank (all-reduced values)
    other = [r for r in runs.values() if r is not head]
    value, max_ms, total_launches, e2e = head["value"], head["max_ms"], head["launches"], head["e2e"]
    clocks_dev, clocks_e2e = head["clocks"], head["clocks_e2e"]
    pull_head = head["mode"] == "pull"

    # ---- the independent arrangement (every GPU its own ingress), as a second number
    per_gpu = None
    if world > 1:
        if rank == 0:
            srv2 = node
            srv2.new_server(server_mode=2, outstanding=3 * nb, n_replicas=1)
        else:
            srv2 = PerGpuIngress(node, outstanding=3 * nb)
        barrier()
        ms2 = allmax(device_timed_per_gpu(srv2, args.steps, warm))
        barrier()
        srv2.start()
        r2 = closed_loop(srv2, max(nb * args.steps, int(0.5 * value / world)), nb * warm, 3 * nb, cfg["payload"], True)
        srv2.stop()
        per_gpu = {"value": round(world * nb * args.steps / (ms2 / 1e3), 1), "ms_per_step": round(ms2 / args.steps, 4),
                   "e2e": round(allsum(r2["rps"]), 1), "e2e_p99_us": round(allmax(r2["p99_us"]), 1),
                   "parallelism": f"dp{world}, one ingress (transport, server, load generator) per GPU"}
    clocks = sampler.stop()

    result = None
    if rank == 0:
        req_bytes, resp_bytes = node.req_size, node.resp_size
        # requests/s that fit through the PCIe links that carry them: GPU 0's alone, or every GPU's own
        ingress_cap = PCIE_GBS * 1e9 / req_bytes * (world if pull_head else 1)
        step_push = (f"one batch of {nb} requests per GPU: GPU 0 gathers the fragments from the pinned host arena "
                     "into the serving GPU's ring (NVLink for the other GPUs) and rings the slot doorbells; the serving "
                     "stream waits on the doorbell and replays the model graph, whose last kernel stores the responses "
                     "into the ingress transmit arena and completes the slots")
        step_pull = (f"one batch of {nb} requests per GPU: every GPU's own gather kernel fetches the batch's 8 KB fragments from "
                     "the ingress's shared pinned host memory over its own PCIe link into its request ring (next batch beside "
                     "the running graph), then replays the model graph, whose last kernel stores the responses into the "
                     "ingress transmit arena and completes the slots")
        path_push = ("loadgen (fragments in pinned host memory, sent by reference) -> loopback NIC -> native server on rank 0 "
                     "(reassembly, steering) -> GPU 0 gather kernel pulls the fragments over PCIe, writes the serving GPU's ring "
                     "and rings its doorbells -> worker (dynamic batching) -> CUDA graph -> last kernel stores the responses into "
                     "the pinned transmit arena and completes the slots -> client")
        path_pull = ("loadgen (fragments in shared pinned host memory, sent by reference) -> loopback NIC -> native server on rank 0 "
                     "(reassembly, steering; writes each request's fragment list into the slot's descriptor block) -> the serving "
                     "process's fetch thread launches its GPU's gather kernel, which pulls the fragments over that GPU's PCIe link "
                     "and rings the doorbells -> worker (dynamic batching) -> CUDA graph -> last kernel stores the responses into "
                     "the ingress's pinned transmit arena and completes the slots -> client")

        def e2e_block(run):
            e, ce = run["e2e"], run["clocks_e2e"]
            rf, cpm = e["ref"], e["copy"]
            sm = ce.get("sm_mhz") or 0
            return {"value": round(rf["rps"], 1), "unit": "req/s", "h2d_bytes_per_step": nb * world * req_bytes,
                    "d2h_bytes_per_step": nb * world * resp_bytes, "p50_us": round(rf["p50_us"], 1), "p99_us": round(rf["p99_us"], 1),
                    "slo_ms": args.slo_ms, "slo_met": bool(rf["ok"] and rf["p99_us"] <= args.slo_ms * 1e3),
                    "requests": rf["requests"], "lost": rf["lost"], "seconds": rf["seconds"], "outstanding": outstanding,
                    "sm_mhz_median": ce.get("sm_mhz"), "reasons": ce.get("reasons"),
                    "value_at_max_clock": round(rf["rps"] * 1965.0 / sm, 1) if sm else None,
                    "copy_mode": {"value": round(cpm["rps"], 1), "p50_us": round(cpm["p50_us"], 1), "p99_us": round(cpm["p99_us"], 1),
                                  "requests": cpm["requests"], "dma_lanes": DMA_LANES, "note": "the emulated NIC DMA writes every fragment into the receive arena (CPU memcpy, spread over the copy lanes)"},
                    "device_timed_latency": {"p50_us": e["dev_lat"][0], "p99_us": e["dev_lat"][1], "samples": e["dev_lat"][2],
                                             "span": "the gather rings the slot's doorbell -> the serving GPU has stored the response "
                                                     "(device timers; across two GPUs corrected by their measured offset)"},
                    "responses_pushed_by_serving_gpu": e["pushed"], "steered": e["steered"], "sg_errors": e["sg_errors"],
                    "mean_batch_replica0": round(e["mean_batch_replica0"], 2), "batches": e["batches"],
                    "path": path_pull if run["mode"] == "pull" else path_push}

        result = {
            "metric": "req/s (dynamic batching, device-timed, max over ranks)", "value": round(value, 1), "unit": "req/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(max_ms / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "splitrpc_b200",
            "config": {"model": cfg["model"], "global_batch": nb * world, "seq_len": cfg["seq"],
                       "parallelism": (f"dp{world}, single ingress, " + ("replicas fetch their requests (pull)" if pull_head else
                                                                        "GPU 0 pushes over NVLink")) if world > 1 else "dp1",
                       "step": step_pull if pull_head else step_push,
                       "l2": "256 MiB buffer written between iterations, inside the timed region; inputs alternate between two pinned host sets",
                       "weights": "random init"},
            "clocks": {**clocks_dev, "whole_run": clocks},
            "roofline": {"ingress_pcie_req_s": round(ingress_cap, 0), "value_over_ingress_cap": round(value / ingress_cap, 3),
                         "note": (f"every GPU fetches its requests over its own PCIe link ({PCIE_GBS} GB/s measured each): "
                                  f"{req_bytes} B per request" if pull_head else
                                  f"one ingress pulls every request over GPU 0's PCIe link ({PCIE_GBS} GB/s measured): "
                                  f"{req_bytes} B per request; the NVLink hop ({NVLINK_GBS} GB/s measured per direction) is not the limit")},
            "e2e": e2e_block(head),
            "gpu_launches": total_launches,
        }
        for o in other:
            result["ingress_" + o["mode"]] = {"value": round(o["value"], 1), "ms_per_step": round(o["max_ms"] / args.steps, 4),
                                              "gpu_launches": o["launches"], "clocks": o["clocks"],
                                              "step": step_pull if o["mode"] == "pull" else step_push, "e2e": e2e_block(o)}
        if per_gpu:
            result["ingress_per_gpu"] = per_gpu
    barrier()
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
    ids_dev = torch.zeros((B, S), dtype=torch.int32, device=dev)
    probs = torch.zeros((B, 2), dtype=torch.float32, device=dev)
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
    results = {}
    with torch.cuda.stream(stream):
        for i in range(warm):
            graph.replay()
        stream.synchronize()
        dist.barrier()
        sampler.start()
        evs = []
        for i in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            evs.append((e0, e1))
        stream.synchronize()
        dist.barrier()
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results["device"] = float(t.item())
    # ---- end to end: closed-loop clients -> RPC front end on rank 0 -> fan-out kernel + doorbells -> TP graph on every rank
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
                        "(reassembly, dynamic batching, SG kernel pulls the ids over PCIe) -> rank 0's graph: fan-out kernel "
                        "stores the ids into every rank's buffer over NVLink and rings the ranks' doorbells (their streams are "
                        "parked on them with the TP graph queued behind) -> TP graph on every rank -> last kernel stores the "
                        "probabilities into the pinned transmit arena and completes the slots -> client"},
        "gpu_launches": model.kernels_per_forward * args.steps,
    }
    dist.barrier()
    dist.destroy_process_group()
    return res


def run_lenet5_cpu(args) -> dict:
    """Plumbing configuration that needs no GPU: LeNet-5 on the CPU device behind the loopback transport."""
    import numpy as np

    from splitrpc_b200 import _C
    from splitrpc_b200.serving import lenet5_random_weights

    cfg = CONFIGS["lenet5"]
    nb = cfg["max_batch"]
    _C.set_rpc_mtu(8192)
    w = lenet5_random_weights()
    sp, cp = _C.make_loopback_pair(8192, 4096)
    app = _C.make_app("lenet5", -1, 3136, 40, w, 256, 1, nb, "cpu")
    srv = _C.Server(sp, req_size=3136, resp_size=40, server_mode=2, max_batch=nb)
    srv.add_replica(app)
    srv.start()
    n_req, n_warm = nb * args.steps * 8, nb * max(args.warmup, 3)
    cli = _C.Client(cp, req_size=3136, resp_size=40, total=n_req + n_warm, warmup=n_warm, payload="uniform", verify=True)
    t0 = time.perf_counter()
    ok = cli.run_closed_loop(48)
    wall = time.perf_counter() - t0
    st = cli.post_process()
    ws = srv.worker_stats(0)
    srv.stop()
    x = np.frombuffer(cli.payload(3), dtype=np.float32)
    oracle_ok = bool(np.allclose(np.frombuffer(cli.response(3), dtype=np.float32), _C.cpu_lenet5(w, x)[0], rtol=1e-4, atol=1e-5))
    hist = ws["batch_hist"]
    rps = st.get("throughput_est", 0.0) if ok else 0.0
    # the comparison system on the same app: gRPC in front of the copy path, batching what queues up
    copy_path = None
    try:
        from splitrpc_b200.utils.grpc_baseline import GrpcClient, GrpcCopyPathServer

        app2 = _C.make_app("lenet5", -1, 3136, 40, w, 256, 1, nb, "cpu")
        with GrpcCopyPathServer(app2, nb) as gs:
            gc = GrpcClient(gs.address, 3136)
            g = gc.run_closed_loop(outstanding=48, total=min(n_req, 4000), warmup=200)
            gc.close()
            t = gs.times()
        copy_path = {"value": round(g["req_per_s"], 1), "unit": "req/s", "p50_us": round(g["p50_us"], 1), "p99_us": round(g["p99_us"], 1),
                     "errors": g["errors"], "mean_batch": round(t["requests"] / max(1, t["batches"]), 2),
                     "copy_in_us_per_req": round(t["h2d_ns"] / max(1, t["requests"]) / 1e3, 2),
                     "run_us_per_req": round(t["run_ns"] / max(1, t["requests"]) / 1e3, 2),
                     "copy_out_us_per_req": round(t["d2h_ns"] / max(1, t["requests"]) / 1e3, 2),
                     "note": "Python grpcio server and client threads: understates what gRPC's C++ server does"}
    except Exception as e:  # noqa: BLE001 - grpcio is optional
        copy_path = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
    return {"metric": "req/s (dynamic batching, CPU device, host clock)", "value": round(rps, 1), "unit": "req/s", "n_gpus": 0,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(1e3 * nb / rps, 4) if rps else None,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "splitrpc_b200",
            "config": {"model": cfg["model"], "global_batch": nb, "seq_len": None, "parallelism": "cpu"},
            "e2e": {"value": round(rps, 1), "unit": "req/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "p50_us": round(st.get("p50_sojournTime_us", 0.0), 1), "p99_us": round(st.get("p99_sojournTime_us", 0.0), 1),
                    "requests": n_req, "seconds": round(wall, 3), "oracle_match": oracle_ok,
                    "mean_batch": round(sum(k * v for k, v in hist.items()) / max(1, sum(hist.values())), 2)},
            "grpc_copy_path": copy_path, "gpu_launches": 0}


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
    ap.add_argument("--slo-ms", type=float, default=10.0, help="p99 latency objective of the end-to-end phase")
    ap.add_argument("--e2e-seconds", type=float, default=2.0, help="target length of the end-to-end phase")
    ap.add_argument("--ingress", default="both", choices=["both", "pull", "push"],
                    help="N > 1: how the replicas of ranks > 0 get their requests (both: measure both, report the faster first)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # Standard output carries the result line and nothing else: libraries that write to descriptor 1 themselves (NCCL
    # prints its version there) are pointed at standard error for the length of the run.
    sys.stdout.flush()
    result_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        res = run_reference(args, rank, world, local_rank)
    elif args.config == "lenet5":
        res = run_lenet5_cpu(args) if rank == 0 else None
    elif args.config == "echo":
        from splitrpc_b200.utils.bench_echo import run_echo

        res = run_echo(args, rank, world, local_rank)
    elif args.config == "bert_large_tp":
        res = run_tp(args, rank, world, local_rank)
    else:
        res = run_ours(args, rank, world, local_rank)
    sys.stdout.flush()
    if rank == 0 and res is not None:
        result_out.write(json.dumps(res) + "\n")
        result_out.flush()


if __name__ == "__main__":
    main()
