"""Seeded randomised runs of the whole host path: transports (loopback with wire faults and DMA lanes, kernel UDP), apps
with verified replies, all worker modes, packet sizes from 256 B to 8 KB; and servers stopped while idle, after traffic
and in the middle of a client's run."""
import random
import threading
import time

import pytest


def _one(C, rnd, it):
    mtu = rnd.choice([256, 1024, 4096, 8192])
    transport = rnd.choice(["loop", "loop", "udp"])
    appname = rnd.choice(["echo", "vec_add"])
    req = rnd.randint(1, 30000)
    resp = req if appname == "vec_add" else rnd.randint(1, min(req, 9000))
    mode = rnd.choice([0, 1, 2])
    batch = rnd.choice([1, 2, 4, 8]) if mode != 1 else 1
    # fixed batch sizes (modes 0 and 1) wait for full batches: enough calls in flight, no duplicated requests
    outstanding = max(rnd.randint(1, 16), batch if mode != 2 else 1)
    total = 48
    dupl = rnd.choice([0.0, 0.0, 0.1]) if (mode == 2 or batch == 1) and transport == "loop" else 0.0
    reorder = rnd.choice([0.0, 0.3]) if transport == "loop" else 0.0
    lanes = rnd.choice([1, 2, 4])
    cfg = dict(mtu=mtu, transport=transport, app=appname, req=req, resp=resp, mode=mode, batch=batch, outstanding=outstanding,
               dupl=dupl, reorder=reorder, lanes=lanes)
    C.set_rpc_mtu(mtu)
    nfr = -(-req // mtu) + -(-resp // mtu)
    slots = max(2048, 4 * outstanding * nfr)
    kw = {}
    if transport == "loop":
        sp, cp = C.make_loopback_pair(mtu, slots)
        if lanes > 1:
            C.set_loopback_dma_lanes(cp, lanes)
            C.set_loopback_dma_lanes(sp, lanes)
        if dupl or reorder:
            C.set_loopback_faults(cp, duplicate=dupl, reorder=reorder, seed=it + 1)
    else:
        sp, sport = C.make_udp_port("127.0.0.1", 0, mtu, slots)
        cp, cport = C.make_udp_port("127.0.0.1", 0, mtu, slots, "127.0.0.1", sport)
        kw["uri"] = f"00:00:00:00:00:01,127.0.0.1,{cport},00:00:00:00:00:02,127.0.0.1,{sport}"
    app = C.make_app(appname, -1, req, resp, [], 64, 1, batch)
    srv = C.Server(sp, req_size=req, resp_size=resp, server_mode=mode, max_batch=batch, reassembly_timeout_ns=50_000_000)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=0, payload=appname, verify=True,
                   drain_timeout_ns=10_000_000_000, **kw)
    ok = cli.run_closed_loop(outstanding)
    st = srv.stats()
    srv.stop()
    # a duplicated datagram that is a whole request by itself is served twice; the client drops the second reply
    assert ok and cli.received == total and cli.verify_failures == 0 and (cli.bad_tokens == 0 or dupl > 0), (cfg, cli.received, st)


def test_random_configurations_of_the_host_path(C):
    rnd = random.Random(20241)
    try:
        for it in range(120):
            _one(C, rnd, it)
    finally:
        C.set_rpc_mtu(8192)


def test_servers_stopped_idle_after_traffic_and_mid_run(C):
    rnd = random.Random(3)
    C.set_rpc_mtu(1024)
    try:
        for it in range(60):
            mode = rnd.choice([0, 1, 2])
            batch = rnd.choice([1, 4]) if mode != 1 else 1
            sp, cp = C.make_loopback_pair(1024, 2048)
            app = C.make_app("echo", -1, 3000, 3000, [], 64, 1, batch)
            srv = C.Server(sp, req_size=3000, resp_size=3000, server_mode=mode, max_batch=batch, reassembly_timeout_ns=20_000_000)
            srv.add_replica(app)
            srv.start()
            kind = rnd.choice(["idle", "traffic", "cut"])
            if kind == "traffic":
                cli = C.Client(cp, req_size=3000, resp_size=3000, total=16, warmup=0, payload="echo", verify=True,
                               drain_timeout_ns=5_000_000_000)
                assert cli.run_closed_loop(max(4, batch)) and cli.received == 16
            elif kind == "cut":  # the server goes away under a running client: the client gives up by its drain timeout
                cli = C.Client(cp, req_size=3000, resp_size=3000, total=4000, warmup=0, payload="echo", verify=False,
                               drain_timeout_ns=300_000_000)
                th = threading.Thread(target=lambda: cli.run_closed_loop(max(4, batch)))
                th.start()
                time.sleep(rnd.uniform(0.0, 0.01))
                srv.stop()
                th.join(20)
                assert not th.is_alive(), "client did not give up after the server stopped"
                continue
            t0 = time.time()
            srv.stop()
            assert time.time() - t0 < 5.0, (it, kind, mode)
    finally:
        C.set_rpc_mtu(8192)


def _replica_proc(path, app_name, req, resp, mode, max_batch, mtu, ready, stop):
    from splitrpc_b200 import _C as C

    C.set_rpc_mtu(mtu)
    app = C.make_app(app_name, -1, req, resp, [], 64, 1, max_batch, "cpu")
    srv = C.BatchedServer(app, path, func_id=77, server_mode=mode, max_batch=max_batch)
    srv.start()
    ready.set()
    while not stop.is_set():
        time.sleep(0.005)
    srv.stop()


def test_random_single_ingress_setups_across_processes(C, tmp_path):
    """Replicas in child processes (one or two, any worker mode), fed by push or by pull, with or without a local
    replica beside them, payloads copied or handed over by reference: every call is answered once and correctly."""
    import multiprocessing as mp

    ctx = mp.get_context("spawn")
    rnd = random.Random(11)
    try:
        for it in range(8):
            mtu = rnd.choice([1024, 4096])
            appname = rnd.choice(["echo", "vec_add"])
            req = rnd.randint(1, 20000)
            resp = req if appname == "vec_add" else rnd.randint(1, min(req, 6000))
            mode = rnd.choice([0, 1, 2])
            batch = rnd.choice([1, 2, 4]) if mode == 2 else 1
            pull, n_rep, local = rnd.choice([False, True]), rnd.choice([1, 2]), rnd.choice([False, True])
            outstanding, total = rnd.randint(1, 12), 60
            procs = []
            for r in range(n_rep):
                path = str(tmp_path / f"s{it}_{r}.sock")
                ready, stop = ctx.Event(), ctx.Event()
                p = ctx.Process(target=_replica_proc, args=(path, appname, req, resp, mode, batch, mtu, ready, stop), daemon=True)
                p.start()
                assert ready.wait(60), "replica process did not come up"
                procs.append((p, path, stop))
            try:
                C.set_rpc_mtu(mtu)
                nfr = -(-req // mtu) + -(-resp // mtu)
                sp, cp = C.make_loopback_pair(mtu, max(2048, 4 * outstanding * nfr), "shm")
                srv = C.Server(sp, req_size=req, resp_size=resp, server_mode=2, max_batch=batch, steer_policy=rnd.choice([0, 1]),
                               reassembly_timeout_ns=50_000_000)
                if local:
                    srv.add_replica(C.make_app(appname, -1, req, resp, [], 64, 1, batch, "cpu"))
                for _, path, _ in procs:
                    srv.add_remote_replica(path, func_id=77, ingress_device=-1, pull=pull)
                srv.start()
                cli = C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=0, payload=appname, verify=True,
                               drain_timeout_ns=10_000_000_000, send_by_reference=rnd.choice([False, True]) if pull else False)
                ok = cli.run_closed_loop(outstanding)
                st = srv.stats()
                srv.stop()
                srv.release_remotes()
                cfg = dict(it=it, mtu=mtu, app=appname, req=req, resp=resp, mode=mode, batch=batch, pull=pull, n_rep=n_rep, local=local)
                assert ok and cli.received == total and cli.verify_failures == 0 and cli.bad_tokens == 0 and st["sg_errors"] == 0, (cfg, st)
                del srv
            finally:
                for p, _, stop in procs:
                    stop.set()
                for p, _, _ in procs:
                    p.join(10)
    finally:
        C.set_rpc_mtu(8192)
