"""RPC front end for a tensor-parallel model: rank 0 owns the transport, every rank steps the model.

The original serves one model on one GPU per process (reference ``src/utils/config_utils.h:42-44``).  Here a
tensor-parallel group serves as one replica.  Rank 0 runs the native server (reassembly, dynamic batching, gather of
the token ids into its request ring) around a graph app: the graph of a batch of ``n`` requests is

    fan-out kernel   stores the batch's ids into every rank's input buffer over NVLink peer memory (its own included),
                     then a {command, batch} record and, with a system-scope release store, the next sequence number
                     into every rank's doorbell word;
    model forward    the tensor-parallel model, whose kernels keep in step through the flags in peer memory;
    response writer  the last kernel stores the ``n`` responses into the transmit arena and completes the slots.

The other ranks keep their streams parked on the doorbell word (``cuStreamWaitValue32``, >=) with the model's graph
queued behind it, a few batches ahead; their host threads only refill that queue.  No collective library call and no
host thread sits between the arrival of a batch on rank 0 and the start of the model on any rank.

    srv = TensorParallelServer(model)            # on every rank
    if srv.rank == 0:
        with srv:                                # starts the front end
            cli = srv.client(total=..., warmup=..., payload="ids"); cli.run_closed_loop(16)
    else:
        srv.serve_forever()                      # returns when rank 0 leaves the ``with`` block
"""
from __future__ import annotations

import collections

import torch
import torch.distributed as dist

from .. import _C

MTU = 8192
CMD_STOP, CMD_RUN = 0, 1


class TensorParallelServer:
    def __init__(self, model, outstanding: int | None = None, pool_size: int = 256, resp_size: int = 16, group=None,
                 ahead: int = 2):
        self.model, self.group, self.ahead = model, group, ahead
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.B, self.S = model.batch, model.seq
        self.device = model.device if isinstance(model.device, torch.device) else torch.device("cuda", model.device)
        self.req_size, self.resp_size = self.S * 4, resp_size
        assert resp_size % 8 == 0 and resp_size >= 8 and self.req_size % 16 == 0
        torch.cuda.set_device(self.device)
        dev = self.device
        # per rank, at the same offsets of the group's symmetric memory: input ids, control record, doorbell word
        arena = model.tpc.arena
        self.ids = arena.alloc("fan_ids", (self.B, self.S), torch.int32)
        self.ctrl = arena.alloc("fan_ctrl", (8,), torch.int32)
        self.bell = arena.alloc("fan_bell", (8,), torch.int32)
        self.ids.zero_()
        self.ctrl.zero_()
        self.bell.zero_()
        arena.barrier()
        self.probs = torch.zeros((self.B, 2), dtype=torch.float32, device=dev)
        self.outstanding = outstanding or 2 * self.B
        self.served_batches = 0
        self._fan = dict(dst=[arena.ptr("fan_ids", r) for r in range(self.world)],
                         ctrl=[arena.ptr("fan_ctrl", r) for r in range(self.world)],
                         doorbell=[arena.ptr("fan_bell", r) for r in range(self.world)])
        if self.rank == 0:
            _C.set_rpc_mtu(MTU)
            self.seq = torch.zeros(1, dtype=torch.int32, device=dev)
            self.arrivals = torch.zeros(1, dtype=torch.int32, device=dev)
            self.app = _C.make_graph_app(dev.index, self.req_size, self.resp_size, pool_size, self.B, "gpu", 2)
            self.stream = torch.cuda.ExternalStream(self.app.work_stream, device=dev)
        else:
            self.app = None
            self.stream = torch.cuda.Stream(device=dev)
        # one run of the model on every rank together (sets kernel attributes), then the captures
        with torch.cuda.stream(self.stream):
            model.forward(self.ids, out=self.probs)
        self.stream.synchronize()
        dist.barrier(group)
        if self.rank == 0:
            self.app.set_stub()
            for n in range(1, self.B + 1):
                with torch.cuda.stream(self.stream):
                    self.app.capture_begin()
                    try:
                        self._fanout(CMD_RUN, n)
                        model.forward(self.ids, d_stub=self.app.d_stub, d_push=self.app.d_push, n_resp=n, resp_stride=self.resp_size)
                    finally:
                        self.app.capture_end(n)
            self.app.set_self_push(True)
            self.server_port, self.client_port = _C.make_loopback_pair(MTU, max(1024, 4 * self.outstanding), "pinned")
            self.server = _C.Server(self.server_port, req_size=self.req_size, resp_size=self.resp_size, server_mode=2,
                                    max_batch=self.B, rr_pool_size=max(1023, 4 * self.outstanding), gather_burst=self.B)
            self.server.add_replica(self.app)
        else:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                model.forward(self.ids, out=self.probs)
        self.stream.synchronize()
        dist.barrier(group)
        self._running = False

    def _fanout(self, command: int, batch: int) -> None:
        """Rank 0, on the current stream: ids of the window the app's stub names -> every rank, then doorbells."""
        _C.tp_fanout(self.app.d_stub, self.req_size, batch, self.B, command, self._fan["dst"], self._fan["ctrl"],
                     self._fan["doorbell"], self.seq.data_ptr(), self.arrivals.data_ptr(), torch.cuda.current_stream().cuda_stream)

    # ------------------------------------------------------------------ other ranks
    def serve_forever(self) -> int:
        """Keeps `ahead` {doorbell wait, model graph} pairs queued on the stream; returns the number of batches served
        when rank 0 stops."""
        assert self.rank != 0
        n, seq = 0, 0
        queued = collections.deque()
        hosts = [torch.zeros(2, dtype=torch.int32).pin_memory() for _ in range(self.ahead + 1)]
        st = self.stream.cuda_stream
        stopping = False
        with torch.cuda.stream(self.stream):
            while True:
                while not stopping and len(queued) < self.ahead:
                    seq += 1
                    _C.stream_wait32(st, self.bell.data_ptr(), seq, geq=True)
                    host = hosts[seq % len(hosts)]
                    host.copy_(self.ctrl[:2], non_blocking=True)  # the record that came with this doorbell
                    self.graph.replay()
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                    queued.append((ev, host))
                if not queued:
                    break
                ev, host = queued.popleft()
                ev.synchronize()
                if int(host[0]) == CMD_STOP:
                    stopping = True  # what is still queued belongs to rank 0's remaining stop steps
                else:
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
        # one stop step per step the other ranks keep queued: each releases one doorbell wait and runs the model once
        # on every rank, so that every queued graph finds its partners
        with torch.cuda.stream(self.stream):
            self.app.set_stub()
            for _ in range(self.ahead):
                self._fanout(CMD_STOP, 0)
                self.model.forward(self.ids, out=self.probs)
        self.stream.synchronize()
        self.served_batches = self.server.worker_stats(0)["num_batches"]

    def client(self, total: int, warmup: int, payload: str = "ids", verify: bool = False, **kw):
        assert self.rank == 0
        return _C.Client(self.client_port, req_size=self.req_size, resp_size=self.resp_size, total=total, warmup=warmup,
                         payload=payload, verify=verify, **kw)

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()
