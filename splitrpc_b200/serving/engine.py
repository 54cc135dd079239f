"""Model serving engine: a model built from this library's kernels behind the native server.

Two roles, one per process:

``ModelServer``   the ingress.  Owns the loopback transport (receive/transmit arenas in pinned host memory that
                  the GPUs map), the native server threads (header parsing, reassembly, flow steering) and
                  one replica of the model on its own GPU.  Replicas on other
                  GPUs are added with ``add_remote(path)``: either the scatter-gather kernel of the ingress GPU
                  writes their request rings over NVLink and rings their slot doorbells itself (push), or the
                  ingress only describes each request and the replica's GPU fetches the fragments from the shared
                  host memory over its own PCIe link (``pull=True``).
``ModelReplica``  a replica on another GPU (another process): the model's graphs behind a batched server that
                  hands its rings and doorbells to the ingress (``buf_mon`` ALLOC handshake) and runs the worker.

In both, the model's last kernel stores each response into the ingress transmit arena and completes the slot, so
neither a scatter kernel nor a host thread sits between the result and the (emulated) NIC.  Python is only involved
in building and capturing; the request hot path is native code and GPU kernels.
"""
from __future__ import annotations

import math

import torch

from .. import _C

MTU = 8192
FUNC_ID = 1234


class _GraphModelApp:
    """A graph app for ``model`` on ``device``: rings, fused ingress set-up, one captured graph per batch size."""

    def __init__(self, model, device: int, max_batch: int, copy_type: int, pool_size: int | None, batch_sizes,
                 reserve_sms: int, fused_ingress: bool):
        self.model, self.device, self.max_batch = model, device, max_batch
        self.reserve_sms = reserve_sms
        _C.gemm_reserve_sms(reserve_sms)  # process-wide; must precede the graph captures below
        self.req_size, self.resp_size = model.req_size, model.resp_size
        _C.set_rpc_mtu(MTU)
        torch.cuda.set_device(device)
        self.pool_size = pool_size or max(256, 4 * max_batch)
        self.app = _C.make_graph_app(device, self.req_size, self.resp_size, self.pool_size, max_batch, "gpu", copy_type)
        self.stream = torch.cuda.ExternalStream(self.app.work_stream, device=torch.device("cuda", device))
        self.batch_sizes = list(batch_sizes) if batch_sizes else list(range(1, max_batch + 1))
        # Fused ingress: the gather that pulls a request's fragments into the ring also deserialises them for the
        # model's first layer (models that offer enable_fused_ingress; GPU engine with one kernel per list).
        self.fused_ingress = False
        self.ingress = None
        if fused_ingress and copy_type == 2 and hasattr(model, "enable_fused_ingress"):
            base, nbytes, doubled = self.app.req_ring
            slots = nbytes * (2 if doubled else 1) // self.req_size
            self.ingress = model.enable_fused_ingress(base, slots, self.req_size)
            _C.memset_async(base, 0, nbytes, self.app.work_stream)  # borders and padding channels stay zero for good
            self.stream.synchronize()
            self.fused_ingress = True
        self._capture()

    def _capture(self) -> None:
        """Warm-up run, then one captured graph per batch size.  Kernels read the ring through the stub and the
        response destinations through the push block, so one graph serves every ring position and every producer."""
        self.app.set_stub()
        kw = dict(d_stub=self.app.d_stub, d_push=self.app.d_push)
        with torch.cuda.stream(self.stream):
            self.model.forward(min(2, self.max_batch), **kw)
        self.stream.synchronize()
        for bs in self.batch_sizes:
            with torch.cuda.stream(self.stream):
                self.app.capture_begin()
                try:
                    self.model.forward(bs, **kw)
                finally:
                    self.app.capture_end(bs)
        self.stream.synchronize()
        self.app.set_self_push(True)  # the graphs' last kernel stores responses and completes slots

    def recapture(self, reserve_sms: int) -> None:
        """Captures the graphs again with another number of SMs left out of the model's persistent kernels (no server
        or worker may be running).  A GPU that gathers for every replica needs more of them than one that only feeds
        itself."""
        if reserve_sms == self.reserve_sms:
            return
        self.reserve_sms = reserve_sms
        _C.gemm_reserve_sms(reserve_sms)
        self._capture()


class ModelServer(_GraphModelApp):
    def __init__(self, model, device: int = 0, max_batch: int = 64, server_mode: int = 2, copy_type: int = 2,
                 outstanding: int | None = None, pool_size: int | None = None, batch_sizes=None, reserve_sms: int = 12,
                 fused_ingress: bool = True, n_replicas: int = 1, steer_policy: int = 0, device_completion: bool = True,
                 port=None):
        """``reserve_sms``: SMs that the model's persistent kernels leave out of their grids, for the scatter-gather
        kernel that pulls the next batch out of host memory while the current one is computed.  A persistent kernel
        counts on one block per SM: with a foreign block on only a few SMs it takes twice as long (ResNet-50 graph
        1.98 ms instead of 1.63 ms), with twelve SMs set aside it runs at 1.68 ms beside the copy.

        ``n_replicas``: how many replicas this ingress will feed in total (sizes the arenas and the request pool)."""
        super().__init__(model, device, max_batch, copy_type, pool_size, batch_sizes, reserve_sms, fused_ingress)
        self.copy_type = copy_type
        self.server = None
        self.n_remote = 0
        self._running = False
        self.new_server(server_mode=server_mode, outstanding=outstanding, n_replicas=n_replicas, steer_policy=steer_policy,
                        device_completion=device_completion, port=port)

    def new_server(self, server_mode: int = 2, outstanding: int | None = None, n_replicas: int = 1, steer_policy: int = 0,
                   device_completion: bool = True, port=None) -> None:
        """(Re)creates the transport and the native server around the already captured model: a fresh loopback link
        (or ``port``, a transport port made by the caller, e.g. ``_C.make_udp_port(..., mem="shm_pinned")``), a fresh
        request pool, this GPU's replica added.  Remote replicas of an earlier server are released first."""
        self.stop()
        self.server = None
        self.app.reset_slots()
        self.outstanding = outstanding or 2 * self.max_batch * n_replicas
        frags = math.ceil(self.req_size / MTU) + math.ceil(self.resp_size / MTU)
        n_slots = max(1024, 2 * self.outstanding * frags)
        # "shm_pinned": pinned and GPU-mapped like a NIC's registered rings, and a shared mapping, so that replicas
        # in other processes can register the transmit arena with their GPUs and store responses into it
        if port is not None:
            self.server_port, self.client_port = port, None
        else:
            self.server_port, self.client_port = _C.make_loopback_pair(MTU, n_slots, "shm_pinned")
        if self.fused_ingress and not self.app.set_ingress_stem_s2d(self.ingress["mean"], self.ingress["inv_std"]):
            raise RuntimeError("the scatter-gather engine does not support the fused ingress transform")
        self.server = _C.Server(self.server_port, req_size=self.req_size, resp_size=self.resp_size, server_mode=server_mode,
                                max_batch=self.max_batch, rr_pool_size=max(1023, 4 * self.outstanding),
                                gather_burst=self.max_batch, steer_policy=steer_policy,
                                device_completion=1 if device_completion else 0)
        self.server.add_replica(self.app)

    def add_remote(self, path: str, timeout_ms: int = 60000, pull: bool = False) -> int:
        """Connects to the ``ModelReplica`` listening at ``path`` and adds it to flow steering.

        ``pull=False``: this GPU's gather kernel stores the replica's requests into its ring over NVLink and rings
        its doorbells.  ``pull=True``: this process shares its payload memory with the replica and only describes
        each request (where its fragments are); the replica's own GPU fetches them over its own PCIe link, so the
        ingress GPU's link stops being the bound when several replicas are fed."""
        idx = self.server.add_remote_replica(path, func_id=FUNC_ID, ingress_device=self.device, copy_type=self.copy_type,
                                             timeout_ms=timeout_ms, pull=pull)
        self.n_remote += 1
        return idx

    def start(self) -> None:
        if not self._running:
            self.server.start()
            self._running = True

    def stop(self) -> None:
        if self._running:
            self.server.stop()
            self._running = False
        if self.n_remote:
            self.server.release_remotes()
            self.n_remote = 0

    def client(self, total: int, warmup: int, payload: str, verify: bool = False, **kw):
        return _C.Client(self.client_port, req_size=self.req_size, resp_size=self.resp_size, total=total, warmup=warmup,
                         payload=payload, verify=verify, **kw)

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()


class ModelReplica(_GraphModelApp):
    """One replica of ``model`` on ``device`` for an ingress in another process (see ``ModelServer.add_remote``).

    ``server_mode``: 0 fixed batch, 1 stream armed, 2 dynamic batching; negative = no worker (the caller consumes the
    slots itself, e.g. a timing loop)."""

    def __init__(self, model, path: str, device: int = 0, max_batch: int = 64, server_mode: int = 2, copy_type: int = 2,
                 pool_size: int | None = None, batch_sizes=None, reserve_sms: int = 0, fused_ingress: bool = True):
        super().__init__(model, device, max_batch, copy_type, pool_size, batch_sizes, reserve_sms, fused_ingress)
        self.path = path
        self.batched = None
        self.serve(server_mode)

    def serve(self, server_mode: int = 2) -> None:
        """(Re)creates the batched server in the given worker mode; call ``start()`` afterwards."""
        if self.batched is not None:
            self.batched.stop()
        self.batched = _C.BatchedServer(self.app, self.path, func_id=FUNC_ID, server_mode=server_mode, max_batch=self.max_batch)
        if self.fused_ingress:
            self.batched.set_ingress_stem_s2d(self.ingress["mean"], self.ingress["inv_std"])

    def start(self) -> None:
        self.batched.start()

    def stop(self) -> None:
        self.batched.stop()

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()
