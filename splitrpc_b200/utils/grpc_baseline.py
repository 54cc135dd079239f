"""The comparison system: the same apps behind a general-purpose RPC library with the copy path.

The original measures itself against gRPC servers that receive a request into ordinary host memory, copy it to the GPU,
run the app and copy the response back (reference ``src/grpc_bench/grpc_handler.h:15-222`` per request,
``src/grpc_bench/batched_grpc_handler.h:18-328`` with an app-worker thread that batches, client
``src/lib_loadgen/grpc_client.h:18-233``).  This module is that system on this package's apps:

* the wire format is the original's ``doinference.Scheduler/runJob`` with ``ScheduleRequest`` / ``ScheduleReply``
  ``{uint64 guid = 1; uint32 funcid = 2; bytes payload = 3; uint32 size = 4}`` (reference
  ``src/grpc_bench/infer.proto:8-26``), encoded here by hand so that no code generator is needed; a client or server
  built from the original's ``.proto`` interoperates;
* the data path (copy in per request, one app run per batch, copy out per request, a timer per phase, the batching
  worker thread) is native: ``_C.CopyPathBatcher``;
* the RPC library is ``grpcio``.  Its Python server costs more per call than the C++ asynchronous server of the
  original, so requests per second through it understate what gRPC can do; the per-phase timers and the comparison at
  equal client settings are what carries over.

    srv = GrpcCopyPathServer(app, max_batch=8); srv.start()
    stats = GrpcClient(srv.address, req_size).run_closed_loop(outstanding=8, total=2000, warmup=200)
    srv.stop()

Command line (same environment knobs as the other mains):
``python -m splitrpc_b200.utils.grpc_baseline server`` / ``... client``.
"""
from __future__ import annotations

import os
import sys
import threading
import time
from concurrent import futures

METHOD = "/doinference.Scheduler/runJob"
MAX_MSG = 64 << 20


# ------------------------------------------------------------------ proto3 wire format of the two messages
def _varint(v: int) -> bytes:
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def encode_message(guid: int, funcid: int, payload: bytes, size: int | None = None) -> bytes:
    """``{guid = 1, funcid = 2, payload = 3, size = 4}``; zero-valued fields are left out, as proto3 does."""
    size = len(payload) if size is None else size
    parts = []
    if guid:
        parts.append(b"\x08" + _varint(guid))
    if funcid:
        parts.append(b"\x10" + _varint(funcid))
    if payload:
        parts.append(b"\x1a" + _varint(len(payload)) + payload)
    if size:
        parts.append(b"\x20" + _varint(size))
    return b"".join(parts)


def decode_message(buf: bytes) -> tuple[int, int, bytes, int]:
    """Returns ``(guid, funcid, payload, size)``; unknown fields are skipped, a malformed message raises ValueError."""
    guid = funcid = size = 0
    payload = b""
    i, n = 0, len(buf)

    def varint(i):
        v = shift = 0
        while True:
            if i >= n or shift > 63:
                raise ValueError("truncated varint")
            b = buf[i]
            i += 1
            v |= (b & 0x7F) << shift
            if not b & 0x80:
                return v, i
            shift += 7

    while i < n:
        key, i = varint(i)
        field, wt = key >> 3, key & 7
        if wt == 0:
            v, i = varint(i)
            if field == 1:
                guid = v
            elif field == 2:
                funcid = v & 0xFFFFFFFF
            elif field == 4:
                size = v & 0xFFFFFFFF
        elif wt == 2:
            ln, i = varint(i)
            if i + ln > n:
                raise ValueError("truncated bytes field")
            if field == 3:
                payload = bytes(buf[i:i + ln])
            i += ln
        elif wt == 1:
            i += 8
        elif wt == 5:
            i += 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        if i > n:
            raise ValueError("truncated message")
    return guid, funcid, payload, size


# ------------------------------------------------------------------ server
class GrpcCopyPathServer:
    """gRPC front end + native copy path around one app.  ``max_batch`` 1 is the original's per-request handler, more
    is its batched handler (whatever has queued up while the previous batch ran, at most ``max_batch``)."""

    def __init__(self, app, max_batch: int = 1, address: str = "127.0.0.1:0", threads: int | None = None):
        import grpc

        from .. import _C

        self.batcher = _C.CopyPathBatcher(app, max_batch)
        self.calls = 0
        self.errors = 0
        batcher = self.batcher

        def run_job(request: bytes, context):
            try:
                guid, funcid, payload, _ = decode_message(request)
                out = batcher.submit(payload)
            except Exception as e:  # malformed message or a failed batch
                self.errors += 1
                context.abort(grpc.StatusCode.INTERNAL, str(e))
            self.calls += 1
            return encode_message(guid, funcid, out)

        handler = grpc.method_handlers_generic_handler(
            "doinference.Scheduler", {"runJob": grpc.unary_unary_rpc_method_handler(run_job)})
        # enough handler threads that a whole batch can wait in the worker at once
        self.server = grpc.server(futures.ThreadPoolExecutor(max_workers=threads or max(4, 2 * max_batch)),
                                  options=[("grpc.max_receive_message_length", MAX_MSG),
                                           ("grpc.max_send_message_length", MAX_MSG)])
        self.server.add_generic_rpc_handlers((handler,))
        port = self.server.add_insecure_port(address)
        if port == 0:
            raise RuntimeError(f"cannot listen on {address}")
        self.address = address.rsplit(":", 1)[0] + f":{port}"

    def start(self):
        self.server.start()
        return self

    def stop(self):
        self.server.stop(grace=1.0).wait()
        self.batcher.stop()

    def times(self) -> dict:
        """Nanoseconds spent copying in, running and copying out, with the number of batches and requests."""
        return dict(self.batcher.times())

    __enter__ = start

    def __exit__(self, *exc):
        self.stop()


# ------------------------------------------------------------------ client (client type 1 of the load generator)
class GrpcClient:
    def __init__(self, address: str, req_size: int, funcid: int = 1, seed: int = 12345):
        import grpc
        import numpy as np

        self.channel = grpc.insecure_channel(address, options=[("grpc.max_receive_message_length", MAX_MSG),
                                                               ("grpc.max_send_message_length", MAX_MSG)])
        self.call = self.channel.unary_unary(METHOD)  # bytes in, bytes out
        self.req_size, self.funcid = req_size, funcid
        rng = np.random.default_rng(seed)
        self.payloads = [rng.integers(0, 256, req_size, dtype=np.uint8).tobytes() for _ in range(8)]
        self.responses: dict[int, bytes] = {}

    def one(self, guid: int, payload: bytes | None = None) -> bytes:
        p = self.payloads[guid % len(self.payloads)] if payload is None else payload
        g, f, out, _ = decode_message(self.call(encode_message(guid, self.funcid, p)))
        if g != guid or f != self.funcid:
            raise RuntimeError(f"reply for call {g}/{f}, expected {guid}/{self.funcid}")
        return out

    def run_closed_loop(self, outstanding: int, total: int, warmup: int = 0, keep: int = 0) -> dict:
        """``outstanding`` callers, ``warmup + total`` calls in all; statistics over the last ``total``.  The first
        ``keep`` responses (by guid) stay in ``self.responses``."""
        import numpy as np

        lock = threading.Lock()
        state = {"next": 0, "t0": None, "errors": 0}
        lat: list[float] = []
        n_all = warmup + total

        def worker():
            while True:
                with lock:
                    guid = state["next"]
                    if guid >= n_all:
                        return
                    state["next"] += 1
                    if guid == warmup:
                        state["t0"] = time.perf_counter()
                t = time.perf_counter()
                try:
                    out = self.one(guid + 1)
                except Exception:
                    with lock:
                        state["errors"] += 1
                    continue
                dt = time.perf_counter() - t
                with lock:
                    if guid >= warmup:
                        lat.append(dt)
                    if guid < keep:
                        self.responses[guid + 1] = out

        threads = [threading.Thread(target=worker) for _ in range(outstanding)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        t1 = time.perf_counter()
        a = np.asarray(lat) * 1e6
        span = t1 - (state["t0"] or t1)
        return {"received": len(lat), "errors": state["errors"], "req_per_s": len(lat) / span if span > 0 else 0.0,
                "p50_us": float(np.percentile(a, 50)) if len(a) else 0.0,
                "p99_us": float(np.percentile(a, 99)) if len(a) else 0.0, "mean_us": float(a.mean()) if len(a) else 0.0}

    def close(self):
        self.channel.close()


# ------------------------------------------------------------------ command line
def _env(name, default):
    return type(default)(os.environ.get(name, default))


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    role = argv[0] if argv else "server"
    uri = os.environ.get("P2P_RPC_URI", "127.0.0.1:50051")
    req, resp = _env("P2P_RPC_REQ_SIZE", 784), _env("P2P_RPC_RESP_SIZE", 40)
    if role == "server":
        from .. import _C

        name, device = os.environ.get("P2P_RPC_APP", "echo"), _env("P2P_RPC_CUDA_DEVICE_ID", -1)
        batch = _env("P2P_RPC_ORT_BATCH_SIZE", _env("P2P_RPC_MAX_BATCH_SIZE", 1))  # the original's name first
        app = _C.make_app(name, device, req, resp, [], max(64, batch), 1, batch)
        srv = GrpcCopyPathServer(app, batch, uri).start()
        print(f"copy-path server for {name} on {srv.address}, batches of up to {batch}", flush=True)
        try:
            limit = _env("P2P_RPC_SERVER_SECONDS", 0.0)
            t0 = time.time()
            while not limit or time.time() - t0 < limit:
                time.sleep(0.2)
        except KeyboardInterrupt:
            pass
        srv.stop()
        print(srv.times(), flush=True)
        return 0
    if role == "client":
        cli = GrpcClient(uri, req)
        total = _env("P2P_RPC_BENCH_TOTAL_REQUESTS", 1000)
        stats = cli.run_closed_loop(_env("P2P_RPC_N_GEN_THR", 4), total, _env("P2P_RPC_NUM_WARMUP", total // 10))
        print(stats, flush=True)
        cli.close()
        return 0 if stats["errors"] == 0 else 1
    print("usage: python -m splitrpc_b200.utils.grpc_baseline server|client", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
