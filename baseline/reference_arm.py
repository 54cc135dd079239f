"""Reference arm of ``bench.py``: the original's own data path, re-hosted, for the same metric and configuration.

What runs here, and what does not:

* Scatter-gather: the ORIGINAL code.  ``baseline/_ref/libsplitrpc_ref.so`` is built from the unmodified
  ``src/transport/g_copy_ng.cu`` and headers of the original tree (see ``baseline/build_ref.py``); every request is
  gathered by the original's ``gather_skbs`` + ``sg_on_gpu`` + ``WaitForAppRunComplete`` and every response scattered
  the same way, one request at a time on a shunter thread, as in ``src/splitrpc_server/p2p_rpc_dpdk_server.cc:108-190``.
  Copy type 2 (``CopyKernel``, one block per buffer) by default, copy type 0 (one ``cudaMemcpyAsync`` per buffer) with
  ``SPLITRPC_REF_COPY_TYPE=0``.  The resident single-block kernel (copy type 1) spins on its doorbell without a bound
  and is left out.
* Model: the original hands the batch to ONNX Runtime -> TensorRT/cuDNN/cuBLAS (``src/apps/ort_app.h:511-516``),
  none of which exist offline.  The declared stand-in is the same architecture through PyTorch's library kernels
  (cuDNN / cuBLAS / SDPA) in bf16, captured once into a CUDA graph (a TensorRT engine has no per-layer host cost
  either) and replayed by a worker thread with a stream synchronise per batch as ``do_batch_work_sync`` does
  (``src/p2p_rpc_async_app_server.h:213-218``).
* The fragments sit in pinned host memory 8 KB apart plus a 128-byte gap (an mbuf's headroom), so they do not coalesce,
  as with a DPDK buffer pool; responses go to pinned host memory.

Nothing from ``splitrpc_b200`` is imported.  One replica per GPU for N > 1.
"""
from __future__ import annotations

import ctypes
import os
import queue
import statistics
import subprocess
import threading
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
MTU = 8192
MBUF_GAP = 128

REFERENCE_CLASS = "re-hosted original copy path (g_copy_ng.cu, unmodified) + library model (ORT/TensorRT unavailable offline: PyTorch bf16 cuDNN/cuBLAS/SDPA in a CUDA graph)"


def load_library():
    import sys

    sys.path.insert(0, str(HERE))
    import build_ref

    try:
        lib_path = build_ref.build()
    except Exception as e:  # build problems are reported as unavailability, not as a crash
        return None, f"the original's copy engine did not build: {str(e).splitlines()[0][:160]}"
    if lib_path is None or not Path(lib_path).exists():
        return None, "baseline/_ref/libsplitrpc_ref.so is missing and the original tree is not on this machine"
    lib = ctypes.CDLL(str(lib_path))
    lib.ref_engine_create.restype = ctypes.c_void_p
    lib.ref_engine_create.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.ref_gather_batch.restype = ctypes.c_int
    lib.ref_gather_batch.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32,
                                     ctypes.c_uint32, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int]
    lib.ref_scatter_batch.restype = ctypes.c_int
    lib.ref_scatter_batch.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                      ctypes.c_int]
    lib.ref_scatter_batch_frags.restype = ctypes.c_int
    lib.ref_scatter_batch_frags.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                            ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int]
    lib.ref_items_per_request.restype = ctypes.c_int
    lib.ref_items_per_request.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32,
                                          ctypes.c_int]
    lib.ref_engine_destroy.argtypes = [ctypes.c_void_p]
    return lib, ""


# ----------------------------------------------------------------------------- library models (random weights)
def make_resnet50(dev, nb):
    """ResNet-50 v1.5 with batch norm folded into the convolutions (what TensorRT serves), bf16, channels-last."""
    import torch
    import torch.nn.functional as F

    g = torch.Generator().manual_seed(0)
    dt = torch.bfloat16

    def conv(cout, cin, k):
        w = torch.randn(cout, cin, k, k, generator=g) * (2.0 / (cin * k * k)) ** 0.5
        return (w.to(dev, dt).contiguous(memory_format=torch.channels_last), (torch.randn(cout, generator=g) * 0.01).to(dev, dt))

    stem = conv(64, 3, 7)
    blocks, cin = [], 64
    for stage, (width, n, stride) in enumerate(((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2))):
        for b in range(n):
            s = stride if b == 0 else 1
            ds = conv(width * 4, cin, 1) if (b == 0) else None
            blocks.append((conv(width, cin, 1), conv(width, width, 3), conv(width * 4, width, 1), ds, s))
            cin = width * 4
    fc_w = (torch.randn(1000, 2048, generator=g) * 0.01).to(dev, dt)
    fc_b = torch.zeros(1000, device=dev, dtype=dt)
    mean = torch.tensor([0.485, 0.456, 0.406], device=dev).view(1, 3, 1, 1)
    inv = 1.0 / torch.tensor([0.229, 0.224, 0.225], device=dev).view(1, 3, 1, 1)

    def forward(x_fp32, out):  # x: [b, 3, 224, 224] fp32 view of the request ring; out: [b, 1000] fp32 response ring
        y = ((x_fp32 - mean) * inv).to(dt).contiguous(memory_format=torch.channels_last)
        y = F.relu(F.conv2d(y, stem[0], stem[1], 2, 3))
        y = F.max_pool2d(y, 3, 2, 1)
        for c1, c2, c3, ds, s in blocks:
            t = F.relu(F.conv2d(y, *c1))
            t = F.relu(F.conv2d(t, *c2, s, 1))
            idn = F.conv2d(y, *ds, s) if ds is not None else y
            y = F.relu(F.conv2d(t, *c3) + idn)
        y = y.mean((2, 3))
        out.copy_(torch.softmax(F.linear(y, fc_w, fc_b).float(), -1))

    return dict(forward=forward, req_size=3 * 224 * 224 * 4, resp_size=4000,
                view_req=lambda t, b: t.view(torch.float32).view(b, 3, 224, 224),
                view_resp=lambda t, b: t.view(torch.float32).view(b, 1000),
                fill=lambda t: t.view(torch.float32).normal_())


def make_bert(dev, nb, layers=12, hidden=768, heads=12, ffn=3072, seq=128, labels=2):
    import torch
    import torch.nn.functional as F

    g = torch.Generator().manual_seed(0)
    dt = torch.bfloat16

    def mat(n, k, std=0.02):
        return (torch.randn(n, k, generator=g) * std).to(dev, dt)

    def vec(n, base=0.0):
        return (torch.randn(n, generator=g) * 0.02 + base).to(dev, dt)

    word, pos, typ = mat(30522, hidden), mat(512, hidden), mat(2, hidden)
    eg, eb = vec(hidden, 1.0), vec(hidden)
    L = [dict(qkv=(mat(3 * hidden, hidden), vec(3 * hidden)), o=(mat(hidden, hidden), vec(hidden)), ln1=(vec(hidden, 1.0), vec(hidden)),
              f1=(mat(ffn, hidden), vec(ffn)), f2=(mat(hidden, ffn), vec(hidden)), ln2=(vec(hidden, 1.0), vec(hidden)))
         for _ in range(layers)]
    pool, cls = (mat(hidden, hidden), vec(hidden)), (mat(labels, hidden, 0.2), vec(labels))

    def forward(ids, out):  # ids: [b, seq] int32 view of the request ring; out: [b, labels] fp32
        B = ids.shape[0]
        x = word[ids.long()] + pos[:seq].unsqueeze(0) + typ[0]
        x = F.layer_norm(x, (hidden,), eg, eb, 1e-12).view(B * seq, hidden)
        for l in L:
            qkv = F.linear(x, *l["qkv"])
            qh, kh, vh = (t.view(B, seq, heads, 64).transpose(1, 2) for t in qkv.split(hidden, dim=1))
            ctx = F.scaled_dot_product_attention(qh, kh, vh).transpose(1, 2).reshape(B * seq, hidden)
            x1 = F.layer_norm(F.linear(ctx, *l["o"]) + x, (hidden,), *l["ln1"], 1e-12)
            h = F.gelu(F.linear(x1, *l["f1"]))
            x = F.layer_norm(F.linear(h, *l["f2"]) + x1, (hidden,), *l["ln2"], 1e-12)
        c = torch.tanh(F.linear(x.view(B, seq, hidden)[:, 0], *pool))
        out.copy_(torch.softmax(F.linear(c, *cls).float(), -1))

    return dict(forward=forward, req_size=seq * 4, resp_size=labels * 4,
                view_req=lambda t, b: t.view(torch.int32).view(b, seq),
                view_resp=lambda t, b: t.view(torch.float32).view(b, labels),
                fill=lambda t: t.view(torch.int32).random_(0, 30522))


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.gpu, self.samples, self.proc = gpu, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: [self.samples.append([f.strip() for f in l.split(",")]) for l in self.proc.stdout],
                             daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
                for n, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


class Pipeline:
    """Shunter thread (original gather/scatter, one request at a time) + worker thread (library model, sync per batch)."""

    def __init__(self, lib, model, dev_index, nb, copy_type):
        import torch

        self.torch, self.lib, self.model, self.nb = torch, lib, model, nb
        self.dev = torch.device("cuda", dev_index)
        self.req, self.resp = model["req_size"], model["resp_size"]
        self.frags = (self.req + MTU - 1) // MTU
        self.last = self.req - (self.frags - 1) * MTU
        self.frag_stride = MTU + MBUF_GAP
        self.req_stride = self.frags * self.frag_stride
        self.n_sets = 2
        self.rx = torch.empty(self.n_sets * nb * self.req_stride, dtype=torch.uint8).pin_memory()
        for s in range(self.n_sets * nb):
            for f in range(self.frags):  # the payload bytes of each fragment
                o = s * self.req_stride + f * self.frag_stride
                model["fill"](self.rx[o:o + (MTU if f < self.frags - 1 else self.last)])
        self.tx_stride = max(64, (self.resp + 63) // 64 * 64)
        self.tx = torch.zeros(self.n_sets * nb * self.tx_stride, dtype=torch.uint8).pin_memory()
        self.req_ring = torch.zeros(self.n_sets * nb * self.req, dtype=torch.uint8, device=self.dev)
        self.resp_ring = torch.zeros(self.n_sets * nb * self.resp, dtype=torch.uint8, device=self.dev)
        self.engine = lib.ref_engine_create(dev_index, copy_type)
        if not self.engine:
            raise RuntimeError("ref_engine_create failed")
        self.items = lib.ref_items_per_request(self.engine, self.rx.data_ptr(), self.frag_stride, MTU, self.last, self.frags)
        self.work_stream = torch.cuda.Stream(device=self.dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        self.batch_latency_s = []
        # one CUDA graph of the library model per ring window (the tensors alias the ring, so the addresses are fixed)
        self.graphs = []
        with torch.cuda.stream(self.work_stream), torch.no_grad():
            for w in range(self.n_sets):
                x = model["view_req"](self.req_ring[w * nb * self.req:(w + 1) * nb * self.req], nb)
                out = model["view_resp"](self.resp_ring[w * nb * self.resp:(w + 1) * nb * self.resp], nb)
                for _ in range(3):  # lets cuDNN pick its algorithms before the capture
                    model["forward"](x, out)
                self.work_stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.work_stream):
                    model["forward"](x, out)
                self.graphs.append(g)
        self.work_stream.synchronize()

    def gather(self, w):
        rc = self.lib.ref_gather_batch(self.engine, self.rx.data_ptr() + w * self.nb * self.req_stride, self.req_stride,
                                       self.frag_stride, MTU, self.last, self.frags,
                                       self.req_ring.data_ptr() + w * self.nb * self.req, self.req, self.nb)
        if rc:
            raise RuntimeError(f"original sg_on_gpu failed on request {rc}")

    def scatter(self, w):
        rc = self.lib.ref_scatter_batch(self.engine, self.resp_ring.data_ptr() + w * self.nb * self.resp, self.resp,
                                        self.tx.data_ptr() + w * self.nb * self.tx_stride, self.tx_stride, self.nb)
        if rc:
            raise RuntimeError(f"original sg_on_gpu (scatter) failed on response {rc}")

    def work(self, w):
        torch = self.torch
        with torch.cuda.stream(self.work_stream), torch.no_grad():
            self.graphs[w].replay()
            self.flush.zero_()  # L2 flush between iterations, inside the timed region
        self.work_stream.synchronize()

    def run(self, steps):
        """Runs `steps` batches through the two-thread pipeline; returns when the last response is in host memory."""
        ready, done, err = queue.Queue(), [threading.Event() for _ in range(steps)], []
        starts = [0.0] * steps
        self.torch.cuda.set_device(self.dev)

        def worker():
            try:
                self.torch.cuda.set_device(self.dev)
                for _ in range(steps):
                    i = ready.get()
                    if i is None:
                        return
                    self.work(i % self.n_sets)
                    done[i].set()
            except Exception as e:  # noqa: BLE001
                err.append(e)
                for d in done:
                    d.set()

        t = threading.Thread(target=worker)
        t.start()
        try:
            for i in range(steps):
                starts[i] = time.perf_counter()
                self.gather(i % self.n_sets)
                ready.put(i)
                if i >= 1:
                    done[i - 1].wait()
                    self.scatter((i - 1) % self.n_sets)
                    self.batch_latency_s.append(time.perf_counter() - starts[i - 1])
            done[steps - 1].wait()
            self.scatter((steps - 1) % self.n_sets)
            self.batch_latency_s.append(time.perf_counter() - starts[steps - 1])
        finally:
            ready.put(None)
            t.join()
        if err:
            raise err[0]

    def close(self):
        self.lib.ref_engine_destroy(self.engine)


def run_echo(lib, args, rank, world, local_rank):
    """Echo sweep on the original's copy path: per request gather (list builder + CopyKernel + sync), the echo app's
    device-to-device cudaMemcpyAsync (src/apps/echo_rpc_bench.cc:25-36) + sync per batch, per response scatter + sync.
    The original serves one GPU; with N > 1 every rank runs this by itself and the rates are summed."""
    import torch

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("gloo")
    copy_type = int(os.environ.get("SPLITRPC_REF_COPY_TYPE", "2"))
    engine = lib.ref_engine_create(local_rank, copy_type)
    dev = torch.device("cuda", local_rank)
    stride = MTU + MBUF_GAP
    sweep = []
    for size in [1 << k for k in range(6, 23)]:
        frags = (size + MTU - 1) // MTU
        last = size - (frags - 1) * MTU
        frag_len = min(MTU, size)
        batch = 64 if size <= (1 << 18) else (16 if size <= (1 << 20) else 8)
        rx = torch.randint(0, 256, (batch * frags * stride,), dtype=torch.uint8).pin_memory()
        tx = torch.zeros(batch * frags * stride, dtype=torch.uint8).pin_memory()
        req_ring = torch.zeros(batch * size, dtype=torch.uint8, device=dev)
        resp_ring = torch.zeros(batch * size, dtype=torch.uint8, device=dev)
        n_batches = int(max(3, min(200, 0.3 * 13e9 / (batch * max(size, 4096)))))

        def one_batch():
            rc = lib.ref_gather_batch(engine, rx.data_ptr(), frags * stride, stride, frag_len, last, frags, req_ring.data_ptr(), size, batch)
            resp_ring.copy_(req_ring, non_blocking=True)
            torch.cuda.synchronize()
            rc |= lib.ref_scatter_batch_frags(engine, resp_ring.data_ptr(), size, tx.data_ptr(), frags * stride, stride, frag_len, last, frags, batch)
            if rc:
                raise RuntimeError("original copy engine failed")

        one_batch()
        t0 = time.perf_counter()
        for _ in range(n_batches):
            one_batch()
        wall = time.perf_counter() - t0
        ok = all(bool(torch.equal(tx[f * stride:f * stride + (frag_len if f < frags - 1 else last)],
                                  rx[f * stride:f * stride + (frag_len if f < frags - 1 else last)])) for f in range(min(frags, 3)))
        rps = batch * n_batches / wall
        sweep.append({"bytes": size, "fragments": frags, "batch": batch, "req_s": round(rps, 1), "gather_gbs": round(rps * size / 1e9, 3),
                      "verified": ok})
    lib.ref_engine_destroy(engine)
    if dist:
        import torch.distributed as dist2

        for s in sweep:
            t = torch.tensor([s["req_s"], s["gather_gbs"]], dtype=torch.float64)
            dist2.all_reduce(t)
            s["req_s"], s["gather_gbs"] = round(float(t[0]), 1), round(float(t[1]), 3)
        dist2.barrier()
        dist2.destroy_process_group()
    best = max(sweep, key=lambda s: s["gather_gbs"])
    return {"metric": "payload GB/s gathered into GPU batch buffers and echoed (best size of the sweep), end to end", "value": best["gather_gbs"],
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "uint8", "data": "synthetic", "impl": "reference",
            "reference_class": "re-hosted original copy path (g_copy_ng.cu, unmodified) + its echo app's device memcpy; host clock",
            "config": {"model": "echo, 64 B - 4 MB payloads in 8 KB fragments", "global_batch": None, "seq_len": None,
                       "parallelism": f"dp{world}, one independent copy engine per GPU" if world > 1 else "dp1",
                       "copy_type": copy_type},
            "sweep": sweep, "all_verified": all(s["verified"] for s in sweep)}


def run(args, rank, world, local_rank, cfg):
    """Returns the JSON dict of the reference arm (or an ``unavailable`` dict)."""
    lib, why = load_library()
    if lib is None:
        return {"impl": "reference", "unavailable": why}
    if args.config == "lenet5":
        return {"impl": "reference", "unavailable": "the original has no CPU device: its LeNet is a set of generated GPU kernels "
                "behind the DPDK server, so the GPU-less plumbing configuration has no counterpart to run"}
    if args.config == "echo":
        return run_echo(lib, args, rank, world, local_rank)
    if args.config == "bert_large_tp":
        return {"impl": "reference", "unavailable": "the original has no multi-GPU path at all (no NCCL, no peer copies); its "
                "library stand-in for tensor parallelism (NCCL all-gather / reduce-scatter + cuBLAS) is timed per operation by "
                "python -m splitrpc_b200.parallel.bench_tp"}
    import torch

    torch.cuda.set_device(local_rank)
    torch.backends.cudnn.benchmark = True
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nb = cfg["max_batch"]
    dev = torch.device("cuda", local_rank)
    model = make_resnet50(dev, nb) if args.config == "resnet50" else make_bert(dev, nb)
    copy_type = int(os.environ.get("SPLITRPC_REF_COPY_TYPE", "2"))
    pipe = Pipeline(lib, model, local_rank, nb, copy_type)
    warm = max(args.warmup, 3)

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    pipe.run(warm)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pipe.run(args.steps)
    torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)
    barrier()
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * nb * args.steps / (ms_max / 1e3)
    # end to end: the same path for longer, on the host clock, every response read on the host
    e2e_steps = max(args.steps, min(20 * args.steps, int(2.0 / max(1e-4, ms_max / 1e3 / args.steps))))
    pipe.batch_latency_s.clear()
    barrier()
    w0 = time.perf_counter()
    pipe.run(e2e_steps)
    checksum = float(pipe.tx.view(torch.float32)[:16].sum())
    wall = time.perf_counter() - w0
    clocks = sampler.stop()
    lat = sorted(pipe.batch_latency_s)
    t2 = torch.tensor([nb * e2e_steps / wall, lat[len(lat) // 2] * 1e6, lat[min(len(lat) - 1, round(0.99 * (len(lat) - 1)))] * 1e6],
                      device="cuda", dtype=torch.float64)
    if dist:
        s, m = t2.clone(), t2.clone()
        dist.all_reduce(s, op=dist.ReduceOp.SUM)
        dist.all_reduce(m, op=dist.ReduceOp.MAX)
        e2e_total, p50, p99 = float(s[0]), float(m[1]), float(m[2])
    else:
        e2e_total, p50, p99 = (float(v) for v in t2)
    res = {
        "metric": "req/s (dynamic batching, device-timed, max over ranks)", "value": round(value, 1), "unit": "req/s",
        "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(ms_max / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference", "reference_class": REFERENCE_CLASS,
        "config": {"model": cfg["model"], "global_batch": nb * world, "seq_len": cfg["seq"],
                   "parallelism": f"dp{world}" if world > 1 else "dp1",
                   "step": f"one batch of {nb} requests per GPU: per request gather_skbs + sg_on_gpu (copy type {copy_type}, "
                           f"{pipe.items} buffers per request) + stream sync on the shunter thread; library model + stream sync on "
                           "the worker thread (CUDA graph); per response scatter + sync; gather of batch i+1 overlaps the model of batch i",
                   "l2": "256 MiB buffer written between iterations, inside the timed region; inputs alternate between two pinned host sets",
                   "weights": "random init"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_total, 1), "unit": "req/s", "h2d_bytes_per_step": nb * pipe.req, "d2h_bytes_per_step": nb * pipe.resp,
                "p50_us": round(p50, 1), "p99_us": round(p99, 1), "latency": "per batch, gather start to last response in host memory",
                "requests": nb * e2e_steps, "seconds": round(wall, 3), "response_checksum": checksum,
                "path": "fragments in pinned host memory -> original gather (per request) -> library model -> original scatter "
                        "(per response) -> pinned host memory, host clock"},
        "gpu_launches": args.steps * nb * (2 if copy_type == 2 else pipe.items + 1),
    }
    pipe.close()
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return res
