"""RPC front end for a tensor-parallel model: rank 0 owns the transport, every rank steps the model.

The original serves one model on one GPU per process (reference ``src/utils/config_utils.h:42-44``).  Here a
tensor-parallel group serves as one replica: rank 0 runs the native server (reassembly, dynamic batching, gather of
the token ids into its request ring); for every batch its worker thread broadcasts a small control tensor
``[command, batch, ids...]`` to the peers over NCCL, and then all ranks replay the same captured CUDA graph of the
tensor-parallel model, whose kernels keep in step through the flags in peer memory.  Only rank 0 writes responses.

    srv = TensorParallelServer(model)            # on every rank
    if srv.rank == 0:
        with srv:                                # starts the front end
            cli = srv.client(total=..., warmup=..., payload="ids"); cli.run_closed_loop(16)
    else:
        srv.serve_forever()                      # returns when rank 0 leaves the ``with`` block
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _C

MTU = 8192
CMD_STOP, CMD_RUN = 0, 1


class TensorParallelServer:
    def __init__(self, model, outstanding: int | None = None, pool_size: int = 256, resp_size: int = 16, group=None):
        self.model, self.group = model, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.B, self.S = model.batch, model.seq
        self.device = model.device if isinstance(model.device, torch.device) else torch.device("cuda", model.device)
        self.req_size, self.resp_size = self.S * 4, resp_size
        assert resp_size % 8 == 0 and resp_size >= 8
        torch.cuda.set_device(self.device)
        dev = self.device
        self.ctrl = torch.zeros(2 + self.B * self.S, dtype=torch.int32, device=dev)
        self.ctrl_host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self.ids = torch.zeros((self.B, self.S), dtype=torch.int32, device=dev)
        self.probs = torch.zeros((self.B, 2), dtype=torch.float32, device=dev)
        self.outstanding = outstanding or 2 * self.B
        self.served_batches = 0
        if self.rank == 0:
            _C.set_rpc_mtu(MTU)
            self.server_port, self.client_port = _C.make_loopback_pair(MTU, max(1024, 4 * self.outstanding), "pinned")
            self.app = _C.make_python_app(self._run, dev.index, self.req_size, self.resp_size, pool_size, 1, self.B, "gpu", 2)
            self.stream = torch.cuda.ExternalStream(self.app.work_stream, device=dev)
        else:
            self.app = None
            self.stream = torch.cuda.Stream(device=dev)
        # one captured graph of the whole tensor-parallel forward (the same on every rank)
        with torch.cuda.stream(self.stream):
            model.forward(self.ids, out=self.probs)
            self.stream.synchronize()
            dist.barrier(group)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                model.forward(self.ids, out=self.probs)
        self.stream.synchronize()
        dist.barrier(group)
        if self.rank == 0:
            self.server = _C.Server(self.server_port, req_size=self.req_size, resp_size=self.resp_size, server_mode=2,
                                    max_batch=self.B, rr_pool_size=max(1023, 4 * self.outstanding), gather_burst=self.B)
            self.server.add_replica(self.app)
        self._running = False

    # ------------------------------------------------------------------ every rank: one batch
    def _step(self) -> None:
        """Runs on the stream after ``ctrl`` holds the batch: ids into place, then the graph."""
        self.ids.copy_(self.ctrl[2:].view(self.B, self.S), non_blocking=True)
        self.graph.replay()

    # ------------------------------------------------------------------ rank 0: called by the native worker thread
    def _run(self, req_ptr: int, resp_ptr: int, batch: int, stream: int, d_stub: int) -> None:
        torch.cuda.set_device(self.device)
        with torch.cuda.stream(self.stream):
            self.ctrl_host[0], self.ctrl_host[1] = CMD_RUN, batch
            self.ctrl[:2].copy_(self.ctrl_host, non_blocking=True)
            if batch < self.B:
                self.ctrl[2 + batch * self.S:].zero_()  # padding sequences of a short batch
            _C.memcpy_async(self.ctrl.data_ptr() + 8, req_ptr, batch * self.req_size, stream)
            dist.broadcast(self.ctrl, src=0, group=self.group)
            self._step()
            # probabilities of the first `batch` sequences into their response slots (resp_size bytes apart)
            _C.memcpy2d_async(resp_ptr, self.resp_size, self.probs.data_ptr(), 8, 8, batch, stream)
        self.served_batches += 1

    # ------------------------------------------------------------------ other ranks
    def serve_forever(self) -> int:
        """Follows rank 0 batch by batch; returns the number of batches when rank 0 stops."""
        assert self.rank != 0
        n = 0
        with torch.cuda.stream(self.stream):
            while True:
                dist.broadcast(self.ctrl, src=0, group=self.group)
                self.ctrl_host.copy_(self.ctrl[:2], non_blocking=True)
                self.stream.synchronize()
                if int(self.ctrl_host[0]) == CMD_STOP:
                    break
                self._step()
                n += 1
        self.stream.synchronize()
        self.served_batches = n
        return n

    # ------------------------------------------------------------------ rank 0: life cycle
    def start(self) -> None:
        assert self.rank == 0
        if not self._running:
            self.server.start()
            self._running = True

    def stop(self) -> None:
        assert self.rank == 0
        if self._running:
            self.server.stop()
            self._running = False
        with torch.cuda.stream(self.stream):
            self.ctrl_host[0], self.ctrl_host[1] = CMD_STOP, 0
            self.ctrl[:2].copy_(self.ctrl_host, non_blocking=True)
            dist.broadcast(self.ctrl, src=0, group=self.group)
        self.stream.synchronize()

    def client(self, total: int, warmup: int, payload: str = "ids", verify: bool = False, **kw):
        assert self.rank == 0
        return _C.Client(self.client_port, req_size=self.req_size, resp_size=self.resp_size, total=total, warmup=warmup,
                         payload=payload, verify=verify, **kw)

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()
