"""Ingress main: the transport, the receive and shunter threads, flow steering over a local replica and any number of
replicas in other processes.

    # one GPU, kernel-UDP transport
    python -m splitrpc_b200.serving.ingress --app resnet50 --device 0 --port 50051
    # proxy for replicas on other GPUs (started with `python -m splitrpc_b200.serving.replica`), which fetch their
    # requests from this process's shared receive memory themselves
    python -m splitrpc_b200.serving.ingress --app resnet50 --device 0 --port 50051 --replica /tmp/r1.sock --replica /tmp/r2.sock --pull
    # no local replica at all: a pure proxy (the role of the original's SmartNIC proxy)
    python -m splitrpc_b200.serving.ingress --app echo --no-local --port 50051 --replica /tmp/echo.sock

Clients reach it with `python -m splitrpc_b200.utils.client`.  The counterparts in the original are its server main
(reference src/splitrpc_server/splitrpc_server.cc) and its proxies
(reference src/splitrpc_rdma_transport/gpu_dpdk_rdma_proxy_handler.cc:216-296, gpu_socket_rdma_proxy.cc).
Prints one JSON line of counters on exit.
"""
from __future__ import annotations

import argparse
import os
import json
import math
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
    ap.add_argument("--app", default=os.environ.get("P2P_RPC_APP"), required="P2P_RPC_APP" not in os.environ)
    ap.add_argument("--device", type=int, default=_env("P2P_RPC_CUDA_DEVICE_ID", 0), help="device of the local replica and of the gather kernels; -1 = CPU")
    ap.add_argument("--no-local", action="store_true", help="serve no replica in this process (proxy only)")
    ap.add_argument("--ip", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=50051, help="UDP port to listen on (0 = any; the bound port is printed)")
    ap.add_argument("--replica", action="append", default=[], help="control socket of a replica process (repeatable)")
    ap.add_argument("--pull", action="store_true", help="remote replicas fetch their requests themselves")
    ap.add_argument("--mode", type=int, default=_env("P2P_RPC_SERVER_MODE", 2))
    ap.add_argument("--max-batch", type=int, default=_env("P2P_RPC_ORT_BATCH_SIZE", 64))
    ap.add_argument("--pool", type=int, default=256)
    ap.add_argument("--outstanding", type=int, default=None, help="requests in flight to size the arenas for")
    ap.add_argument("--req-size", type=int, default=_env("P2P_RPC_REQ_SIZE", None, int))
    ap.add_argument("--resp-size", type=int, default=_env("P2P_RPC_RESP_SIZE", None, int))
    ap.add_argument("--mtu", type=int, default=_env("P2P_RPC_MTU", 8192))
    ap.add_argument("--steer", type=int, default=1, help="0 round robin in runs of max-batch, 1 least outstanding")
    ap.add_argument("--func-id", type=int, default=FUNC_ID)
    ap.add_argument("--seconds", type=float, default=0.0)
    args = ap.parse_args(argv)
    _C.set_rpc_mtu(args.mtu)
    stop = {"now": False}
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.__setitem__("now", True))
    req, resp, _ = sizes(args.app, args.req_size, args.resp_size)
    n_rep = len(args.replica) + (0 if args.no_local else 1)
    if n_rep == 0:
        raise SystemExit("nothing to serve: give --replica or drop --no-local")
    outstanding = args.outstanding or 3 * args.max_batch * n_rep
    frags = math.ceil(req / args.mtu) + math.ceil(resp / args.mtu)
    # shared (and, with a GPU, pinned) arenas: serving processes store responses into the transmit arena and, in pull
    # mode, read the receive arena
    mem = "shm" if args.device < 0 else "shm_pinned"
    port, bound = _C.make_udp_port(args.ip, args.port, args.mtu, max(1024, 2 * outstanding * frags), mem=mem)
    model_node = None
    if args.app in BUILTIN or args.no_local:
        server = _C.Server(port, req_size=req, resp_size=resp, server_mode=args.mode, max_batch=args.max_batch,
                           rr_pool_size=max(1023, 4 * outstanding), gather_burst=args.max_batch, steer_policy=args.steer)
        if not args.no_local:
            local = make_builtin(args.app, args.device, req, resp, args.pool, args.max_batch)
            server.add_replica(local)
        for path in args.replica:
            server.add_remote_replica(path, func_id=args.func_id, ingress_device=args.device, copy_type=2, pull=args.pull)
    else:
        from .engine import ModelServer

        model_node = ModelServer(build_model(args.app, args.device, args.max_batch), device=args.device, max_batch=args.max_batch,
                                 server_mode=args.mode, outstanding=outstanding, pool_size=args.pool, n_replicas=n_rep,
                                 reserve_sms=12 if (args.pull or not args.replica) else 24, steer_policy=args.steer, port=port)
        server = model_node.server
        for path in args.replica:
            model_node.add_remote(path, pull=args.pull)
    server.start()
    print(json.dumps({"event": "listening", "udp_port": bound, "app": args.app, "replicas": n_rep,
                      "remote": [server.remote_info(i) for i in range(len(args.replica))]}), flush=True)
    t0 = time.time()
    while not stop["now"] and (args.seconds <= 0 or time.time() - t0 < args.seconds):
        time.sleep(0.05)
    st = server.stats()
    server.stop()
    released = server.release_remotes() if args.replica else 0
    print(json.dumps({"event": "exit", "stats": st, "released": released}), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
