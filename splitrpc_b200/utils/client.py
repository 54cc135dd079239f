"""Load generator main (kernel-UDP transport): closed loop with a fixed number of outstanding requests, or open loop
at a request rate with deterministic / exponential / hyper-exponential arrivals.

    python -m splitrpc_b200.utils.client --server-ip 127.0.0.1 --server-port 50051 --app resnet50 --total 5000 --outstanding 64
    python -m splitrpc_b200.utils.client --server-port 50051 --app echo --req-size 4096 --resp-size 1024 --rate 2000 --cov 1

Prints the statistics of the measured requests as one JSON line, with the keys of the original's load generator
(reference src/lib_loadgen/dist_rpc_bench.cc:274-284, stats_factory.h:135-148).
"""
from __future__ import annotations

import argparse
import os
import json
import math

from .. import _C
from ..serving.apps import sizes


def _env(name: str, default, cast=None):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return (cast or type(default))(v)


def main(argv=None) -> int:
    # Defaults come from the original's environment variables (reference src/lib_loadgen/dist_rpc_bench.cc:89-116):
    # P2P_RPC_URI "mac,ip,port,mac,ip,port" (client, then server), P2P_RPC_BENCH_TOTAL_REQUESTS, P2P_RPC_NUM_WARMUP (10 % of
    # the total), P2P_RPC_REQ_GEN_TYPE (0 closed loop, 1 open loop), P2P_RPC_BENCH_ARR_RATE (open loop: requests per
    # second; closed loop: requests in flight), P2P_RPC_ARR_RATE_COV, P2P_RPC_N_GEN_THR, P2P_RPC_CLIENT_TYPE,
    # P2P_RPC_CLIENT_VERIFY_RUN, P2P_RPC_BENCH_EXP_NAME, P2P_RPC_DUMP_RAW_STATS, P2P_RPC_MTU, P2P_RPC_RANDOM_SEED.
    # (P2P_RPC_N_LISTENER_THR is accepted and has no effect: one listener thread reassembles all replies.)
    uri_env = [f.strip() for f in os.environ.get("P2P_RPC_URI", "").split(",")]
    uri_ok = len(uri_env) == 6
    total_d = _env("P2P_RPC_BENCH_TOTAL_REQUESTS", 1000)
    open_loop = _env("P2P_RPC_REQ_GEN_TYPE", 0) == 1
    arr = _env("P2P_RPC_BENCH_ARR_RATE", 1.0)
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--server-ip", default=uri_env[4] if uri_ok else "127.0.0.1")
    ap.add_argument("--server-port", type=int, default=int(uri_env[5]) if uri_ok else None, required=not uri_ok)
    ap.add_argument("--bind-ip", default=uri_env[1] if uri_ok else "0.0.0.0")
    ap.add_argument("--bind-port", type=int, default=int(uri_env[2]) if uri_ok else 0)
    ap.add_argument("--app", default=os.environ.get("P2P_RPC_APP"), required="P2P_RPC_APP" not in os.environ,
                    help="selects request / response sizes and the payload generator")
    ap.add_argument("--req-size", type=int, default=_env("P2P_RPC_REQ_SIZE", None, int))
    ap.add_argument("--resp-size", type=int, default=_env("P2P_RPC_RESP_SIZE", None, int))
    ap.add_argument("--mtu", type=int, default=_env("P2P_RPC_MTU", 8192))
    ap.add_argument("--total", type=int, default=total_d)
    ap.add_argument("--warmup", type=int, default=_env("P2P_RPC_NUM_WARMUP", total_d // 10))
    ap.add_argument("--outstanding", type=int, default=1 if open_loop else max(1, int(arr)), help="closed loop: requests in flight")
    ap.add_argument("--rate", type=float, default=arr if open_loop else 0.0, help="open loop: requests per second (0 = closed loop)")
    ap.add_argument("--cov", type=float, default=_env("P2P_RPC_ARR_RATE_COV", 1.0), help="open loop: coefficient of variation of the inter-arrival times")
    ap.add_argument("--threads", type=int, default=_env("P2P_RPC_N_GEN_THR", 1))
    ap.add_argument("--verify", action="store_true", default=_env("P2P_RPC_CLIENT_VERIFY_RUN", 0) > 0)
    ap.add_argument("--client-type", type=int, default=_env("P2P_RPC_CLIENT_TYPE", 0),
                    help="0: this package's protocol over kernel UDP; 1: the comparison system's gRPC client "
                         "(reference src/lib_loadgen/dist_rpc_bench.cc:89-116)")
    ap.add_argument("--exp-name", default=os.environ.get("P2P_RPC_BENCH_EXP_NAME", "splitrpc"))
    ap.add_argument("--out-dir", default="")
    ap.add_argument("--dump-raw", action="store_true", default=_env("P2P_RPC_DUMP_RAW_STATS", 0) > 0,
                    help="also write raw_<metric>_<experiment>.stat next to the summary")
    args = ap.parse_args(argv)
    _C.set_rpc_mtu(args.mtu)
    req, resp, kind = sizes(args.app, args.req_size, args.resp_size)
    if args.client_type == 1:
        from .grpc_baseline import GrpcClient

        g = GrpcClient(f"{args.server_ip}:{args.server_port}", req)
        st = g.run_closed_loop(max(1, args.outstanding), args.total, args.warmup)
        g.close()
        st["ok"] = st["errors"] == 0 and st["received"] == args.total
        print(json.dumps(st), flush=True)
        return 0 if st["ok"] else 1
    if args.client_type != 0:
        raise SystemExit("client type 2 (raw DPDK) needs a build with SPLITRPC_WITH_DPDK=1 and a NIC")
    frags = math.ceil(req / args.mtu) + math.ceil(resp / args.mtu)
    n_slots = max(1024, 4 * max(args.outstanding, 64) * frags)
    port, bound = _C.make_udp_port(args.bind_ip, args.bind_port, args.mtu, n_slots, args.server_ip, args.server_port)
    my_ip = "127.0.0.1" if args.bind_ip == "0.0.0.0" else args.bind_ip
    uri = f"00:00:00:00:00:01,{my_ip},{bound},00:00:00:00:00:02,{args.server_ip},{args.server_port}"
    cli = _C.Client(port, req_size=req, resp_size=resp, total=args.total + args.warmup, warmup=args.warmup, payload=kind,
                    verify=args.verify, exp_name=args.exp_name, out_dir=args.out_dir or ".", uri=uri)
    ok = cli.run_open_loop(args.rate, args.cov, args.threads) if args.rate > 0 else cli.run_closed_loop(args.outstanding)
    st = dict(cli.post_process())
    if args.out_dir or args.dump_raw:
        cli.save_stats(args.dump_raw)
    st.update({"ok": bool(ok), "received": int(cli.received), "verify_failures": int(cli.verify_failures)})
    print(json.dumps(st), flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
