"""Model serving engine: a model built from this library's kernels behind the native server.

``ModelServer`` owns the loopback transport (pinned receive/transmit arenas the GPU
maps), a graph app whose CUDA graphs hold the model's forward pass for every batch
size, and the native server threads.  Python is only involved in building and
capturing; the request hot path is native code and GPU kernels.
"""
from __future__ import annotations

import math

import torch

from .. import _C

MTU = 8192


class ModelServer:
    def __init__(self, model, device: int = 0, max_batch: int = 64, server_mode: int = 2, copy_type: int = 2,
                 outstanding: int | None = None, pool_size: int | None = None, batch_sizes=None, reserve_sms: int = 12,
                 fused_ingress: bool = True):
        """``reserve_sms``: SMs that the model's persistent kernels leave out of their grids, for the scatter-gather
        kernel that pulls the next batch out of host memory while the current one is computed.  A persistent kernel
        counts on one block per SM: with a foreign block on only a few SMs it takes twice as long (ResNet-50 graph
        1.98 ms instead of 1.63 ms), with twelve SMs set aside it runs at 1.68 ms beside the copy."""
        self.model, self.device, self.max_batch = model, device, max_batch
        self.reserve_sms = reserve_sms
        _C.gemm_reserve_sms(reserve_sms)  # process-wide; must precede the graph captures below
        self.req_size, self.resp_size = model.req_size, model.resp_size
        _C.set_rpc_mtu(MTU)
        torch.cuda.set_device(device)
        self.outstanding = outstanding or 2 * max_batch
        frags = math.ceil(self.req_size / MTU) + math.ceil(self.resp_size / MTU)
        n_slots = max(1024, 2 * self.outstanding * frags)
        self.server_port, self.client_port = _C.make_loopback_pair(MTU, n_slots, "pinned")
        self.pool_size = pool_size or max(256, 4 * max_batch)
        self.app = _C.make_graph_app(device, self.req_size, self.resp_size, self.pool_size, max_batch, "gpu", copy_type)
        self.stream = torch.cuda.ExternalStream(self.app.work_stream, device=torch.device("cuda", device))
        self.batch_sizes = list(batch_sizes) if batch_sizes else list(range(1, max_batch + 1))
        # Fused ingress: the gather that pulls a request's fragments into the ring also deserialises them for the
        # model's first layer (models that offer enable_fused_ingress; GPU engine with one kernel per list).
        self.fused_ingress = False
        if fused_ingress and copy_type == 2 and hasattr(model, "enable_fused_ingress"):
            base, nbytes, doubled = self.app.req_ring
            slots = nbytes * (2 if doubled else 1) // self.req_size
            tr = model.enable_fused_ingress(base, slots, self.req_size)
            _C.memset_async(base, 0, nbytes, self.app.work_stream)  # borders and padding channels stay zero for good
            self.stream.synchronize()
            if not self.app.set_ingress_stem_s2d(tr["mean"], tr["inv_std"]):
                raise RuntimeError("the scatter-gather engine does not support the fused ingress transform")
            self.fused_ingress = True
            self.ingress = tr
        self._capture()
        self.server = _C.Server(self.server_port, req_size=self.req_size, resp_size=self.resp_size, server_mode=server_mode,
                                max_batch=max_batch, rr_pool_size=max(1023, 4 * self.outstanding), gather_burst=max_batch)
        self.server.add_replica(self.app)
        self._running = False

    def _capture(self) -> None:
        """Warm-up run, then one captured graph per batch size; kernels read the ring through the stub."""
        self.app.set_stub()
        with torch.cuda.stream(self.stream):
            self.model.forward(min(2, self.max_batch), d_stub=self.app.d_stub)
        self.stream.synchronize()
        for bs in self.batch_sizes:
            with torch.cuda.stream(self.stream):
                self.app.capture_begin()
                try:
                    self.model.forward(bs, d_stub=self.app.d_stub)
                finally:
                    self.app.capture_end(bs)
        self.stream.synchronize()

    def start(self) -> None:
        if not self._running:
            self.server.start()
            self._running = True

    def stop(self) -> None:
        if self._running:
            self.server.stop()
            self._running = False

    def client(self, total: int, warmup: int, payload: str, verify: bool = False, **kw):
        return _C.Client(self.client_port, req_size=self.req_size, resp_size=self.resp_size, total=total, warmup=warmup,
                         payload=payload, verify=verify, **kw)

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()
