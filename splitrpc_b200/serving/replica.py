"""Replica main: one app or model on one device behind a batched server, for an ingress in another process.

    python -m splitrpc_b200.serving.replica --app resnet50 --device 1 --path /tmp/replica1.sock
    python -m splitrpc_b200.serving.replica --app echo --device -1 --path /tmp/echo.sock --req-size 4096 --resp-size 1024

The process exports its request ring, response ring and slot control block to the ingress that connects to `--path`
(ALLOC handshake) and serves until it is interrupted (or for `--seconds`).  This is the role of the original's
`gpu_rdma_batched_server` (reference src/splitrpc_rdma_transport/gpu_rdma_batched_server.cc:279-458), with file
descriptors over a Unix socket in place of RDMA region keys.  Prints one JSON line of counters on exit.
"""
from __future__ import annotations

import argparse
import os
import json
import signal
import time

from .. import _C
from .apps import BUILTIN, build_model, make_builtin, sizes

FUNC_ID = 1234


def _env(name: str, default, cast=None):
    """Default of a flag from the original's environment variable of that meaning (reference src/utils/config_utils.h)."""
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return (cast or type(default))(v)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--app", default=os.environ.get("P2P_RPC_APP"), required="P2P_RPC_APP" not in os.environ, help=f"model ({'resnet50, bert_base'}) or built-in app ({', '.join(sorted(BUILTIN))})")
    ap.add_argument("--device", type=int, default=_env("P2P_RPC_CUDA_DEVICE_ID", 0), help="GPU index, -1 = CPU device (built-in apps only)")
    ap.add_argument("--path", required=True, help="Unix socket path of the control channel")
    ap.add_argument("--mode", type=int, default=_env("P2P_RPC_SERVER_MODE", 2), help="worker: 0 fixed batch, 1 stream armed, 2 dynamic batching")
    ap.add_argument("--max-batch", type=int, default=_env("P2P_RPC_ORT_BATCH_SIZE", 64))
    ap.add_argument("--pool", type=int, default=256, help="slots of the request / response rings")
    ap.add_argument("--req-size", type=int, default=_env("P2P_RPC_REQ_SIZE", None, int))
    ap.add_argument("--resp-size", type=int, default=_env("P2P_RPC_RESP_SIZE", None, int))
    ap.add_argument("--mtu", type=int, default=_env("P2P_RPC_MTU", 8192))
    ap.add_argument("--func-id", type=int, default=FUNC_ID)
    ap.add_argument("--seconds", type=float, default=0.0, help="serve this long, 0 = until SIGINT / SIGTERM")
    args = ap.parse_args(argv)
    _C.set_rpc_mtu(args.mtu)
    stop = {"now": False}
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.__setitem__("now", True))
    if args.app in BUILTIN:
        req, resp, _ = sizes(args.app, args.req_size, args.resp_size)
        app = make_builtin(args.app, args.device, req, resp, args.pool, args.max_batch)
        bs = _C.BatchedServer(app, args.path, func_id=args.func_id, server_mode=args.mode, max_batch=args.max_batch)
        node = None
    else:
        from .engine import ModelReplica

        node = ModelReplica(build_model(args.app, args.device, args.max_batch), args.path, device=args.device,
                            max_batch=args.max_batch, server_mode=args.mode, pool_size=args.pool, reserve_sms=12)
        bs = node.batched
    bs.start()
    print(json.dumps({"event": "listening", "path": args.path, "app": args.app, "device": args.device}), flush=True)
    t0 = time.time()
    while not stop["now"] and (args.seconds <= 0 or time.time() - t0 < args.seconds):
        time.sleep(0.05)
    ws = bs.worker_stats()
    out = {"event": "exit", "counters": bs.counters(), "served": ws["num_req"], "batches": ws["num_batches"], "pull": bs.pull_stats()}
    bs.stop()
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
