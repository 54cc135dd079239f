"""Single ingress, replicas in other processes: the batched-server handshake, remote producers, completion by the
serving side and failure detection, all on the CPU device (host rings in shared memory stand in for GPU rings, the CPU
engine for the ingress GPU's gather kernel).  The protocol and the host code are the same ones the GPUs run."""
import multiprocessing as mp
import os
import time

import numpy as np
import pytest

REQ = 4096
FUNC = 77


def _replica_main(path, app_name, req, resp, mode, max_batch, ready, stop, out):
    """Child process: one app behind a BatchedServer until `stop` is set."""
    from splitrpc_b200 import _C as C

    C.set_rpc_mtu(1024)
    app = C.make_app(app_name, -1, req, resp, [], 64, 1, max_batch, "cpu")
    srv = C.BatchedServer(app, path, func_id=FUNC, server_mode=mode, max_batch=max_batch)
    srv.start()
    ready.set()
    while not stop.is_set():
        time.sleep(0.01)
    out.put((srv.counters(), srv.worker_stats()["num_req"], srv.pull_stats()))
    srv.stop()


def _spawn(tmp_path, name, app_name="echo", req=REQ, resp=REQ, mode=2, max_batch=4):
    ctx = mp.get_context("spawn")
    path = str(tmp_path / f"{name}.sock")
    ready, stop, out = ctx.Event(), ctx.Event(), ctx.Queue()
    p = ctx.Process(target=_replica_main, args=(path, app_name, req, resp, mode, max_batch, ready, stop, out), daemon=True)
    p.start()
    assert ready.wait(60), "replica process did not come up"
    return p, path, stop, out


@pytest.fixture
def mtu1k(C):
    C.set_rpc_mtu(1024)
    yield
    C.set_rpc_mtu(1024)


def _ingress(C, paths, local_app=None, req=REQ, resp=REQ, max_batch=4, steer=0, pull=False):
    sp, cp = C.make_loopback_pair(1024, 2048, "shm")
    srv = C.Server(sp, req_size=req, resp_size=resp, server_mode=2, max_batch=max_batch, steer_policy=steer,
                   reassembly_timeout_ns=50_000_000)
    if local_app is not None:
        srv.add_replica(local_app)
    for p in paths:
        srv.add_remote_replica(p, func_id=FUNC, ingress_device=-1, pull=pull)
    return srv, cp


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_remote_replica_serves_echo_in_every_worker_mode(C, mtu1k, tmp_path, mode):
    proc, path, stop, out = _spawn(tmp_path, f"r{mode}", mode=mode, max_batch=1 if mode < 2 else 4, resp=1024, req=REQ)
    try:
        srv, cp = _ingress(C, [path], resp=1024, max_batch=1 if mode < 2 else 4)
        info = srv.remote_info(0)
        assert info["queue_size"] == 64 and info["req_size"] == REQ and info["resp_size"] == 1024
        assert info["device_id"] == -1 and info["server_mode"] == mode and info["device_completes"] == 1
        srv.start()
        cli = C.Client(cp, req_size=REQ, resp_size=1024, total=120, warmup=0, payload="echo", verify=True)
        assert cli.run_closed_loop(6)
        st = srv.stats()
        ws = srv.worker_stats(0)  # asked from the remote server over the control channel
        lat = srv.device_latency_ns()  # doorbell rung (ingress side) -> response stored (serving side), per request
        srv.stop()
        assert len(lat) == 120 and min(lat) > 0 and max(lat) < 5_000_000_000
        assert cli.received == 120 and cli.verify_failures == 0
        # every response was stored into the ingress transmit arena by the serving process, none was fetched
        assert st["replicas"][0]["pushed"] == 120 and st["sg_errors"] == 0
        assert ws["num_req"] == 120
        assert srv.release_remotes() == 1
    finally:
        stop.set()
        ctr, served, _ = out.get(timeout=20)
        proc.join(20)
    assert ctr["allocs"] == 1 and ctr["releases"] == 1 and ctr["peers_lost"] == 0 and served == 120


@pytest.mark.parametrize("by_reference", [False, True])
@pytest.mark.parametrize("mode", [1, 2])
def test_replica_fetches_described_requests_itself(C, mtu1k, tmp_path, mode, by_reference):
    """Pull mode: the ingress shares its payload regions at ALLOC time and afterwards only writes where a request's
    fragments are; the serving process moves the bytes into its ring, serves and pushes the response.  Fragments lie in
    the receive arena (one descriptor each) or in the sender's by-reference buffer (one descriptor per request)."""
    proc, path, stop, out = _spawn(tmp_path, f"p{mode}{int(by_reference)}", mode=mode, max_batch=1 if mode < 2 else 4, resp=1024)
    try:
        srv, cp = _ingress(C, [path], resp=1024, max_batch=1 if mode < 2 else 4, pull=True)
        assert srv.remote_info(0)["pull"] == 1
        srv.start()
        cli = C.Client(cp, req_size=REQ, resp_size=1024, total=150, warmup=0, payload="echo", verify=True,
                       send_by_reference=by_reference, n_payloads=8)
        assert cli.run_closed_loop(6)
        st = srv.stats()
        lat = srv.device_latency_ns()
        srv.stop()
        assert cli.received == 150 and cli.verify_failures == 0 and st["sg_errors"] == 0
        assert st["replicas"][0]["pushed"] == 150 and len(lat) == 150 and min(lat) > 0
        assert srv.release_remotes() == 1
    finally:
        stop.set()
        ctr, served, pulled = out.get(timeout=20)
        proc.join(20)
    assert served == 150 and pulled["pulled"] == 150 and pulled["errors"] == 0


def test_pull_is_refused_without_shareable_regions(C, mtu1k, tmp_path):
    """A port whose receive arena is private memory cannot be pulled from: the handshake falls back to push."""
    proc, path, stop, out = _spawn(tmp_path, "np", resp=1024)
    try:
        sp, cp = C.make_loopback_pair(1024, 2048)  # malloc arenas: no descriptor to share
        srv = C.Server(sp, req_size=REQ, resp_size=1024, server_mode=2, max_batch=4)
        srv.add_remote_replica(path, func_id=FUNC, ingress_device=-1, pull=True)
        assert srv.remote_info(0)["pull"] == 0
        srv.start()
        cli = C.Client(cp, req_size=REQ, resp_size=1024, total=40, warmup=0, payload="echo", verify=True)
        assert cli.run_closed_loop(4) and cli.received == 40 and cli.verify_failures == 0
        srv.stop()
        srv.release_remotes()
    finally:
        stop.set()
        _, served, pulled = out.get(timeout=20)
        proc.join(20)
    assert served == 40 and pulled["pulled"] == 0


def test_multi_fragment_responses_are_fetched_from_the_remote_ring(C, mtu1k, tmp_path):
    """A 4 KB response is four fragments: the serving side only completes the slot, the ingress reads the response
    ring (the mirror mapping) itself."""
    proc, path, stop, out = _spawn(tmp_path, "mf")
    try:
        srv, cp = _ingress(C, [path])
        srv.start()
        cli = C.Client(cp, req_size=REQ, resp_size=REQ, total=60, warmup=0, payload="echo", verify=True)
        assert cli.run_closed_loop(4)
        st = srv.stats()
        srv.stop()
        srv.release_remotes()
        assert cli.received == 60 and cli.verify_failures == 0 and st["replicas"][0]["pushed"] == 0
    finally:
        stop.set()
        out.get(timeout=20)
        proc.join(20)


def test_local_and_remote_replicas_share_one_ingress(C, mtu1k, tmp_path):
    procs = [_spawn(tmp_path, f"m{i}", app_name="vec_add", req=1024, resp=1024) for i in range(2)]
    try:
        local = C.make_app("vec_add", -1, 1024, 1024, [], 64, 1, 4, "cpu")
        srv, cp = _ingress(C, [p[1] for p in procs], local_app=local, req=1024, resp=1024)
        srv.start()
        cli = C.Client(cp, req_size=1024, resp_size=1024, total=300, warmup=0, payload="vec_add", verify=True)
        assert cli.run_closed_loop(12)
        st = srv.stats()
        srv.stop()
        srv.release_remotes()
        assert cli.received == 300 and cli.verify_failures == 0
        steered = [r["steered"] for r in st["replicas"]]
        assert sum(steered) == 300 and min(steered) >= 60  # round robin in runs of max_batch over three replicas
        assert all(r["pushed"] == r["completed"] for r in st["replicas"])
    finally:
        served = []
        for p, _, stop, out in procs:
            stop.set()
            served.append(out.get(timeout=20)[1])
            p.join(20)
    assert sum(served) + steered[0] == 300


@pytest.mark.parametrize("pull", [False, True])
def test_ingress_skips_a_replica_whose_process_died(C, mtu1k, tmp_path, pull):
    """The replica's process exits between two bursts (no request in flight).  The ingress learns of it on the control
    socket and steers everything to the surviving replica."""
    proc, path, stop, out = _spawn(tmp_path, f"dead{int(pull)}", app_name="echo", req=1024, resp=1024)
    local = C.make_app("echo", -1, 1024, 1024, [], 64, 1, 4, "cpu")
    srv, cp = _ingress(C, [path], local_app=local, req=1024, resp=1024, pull=pull)
    srv.start()
    cli = C.Client(cp, req_size=1024, resp_size=1024, total=80, warmup=0, payload="echo", verify=True)
    assert cli.run_closed_loop(8) and cli.received == 80
    before = srv.stats()
    assert before["replicas"][1]["steered"] > 0
    proc.terminate()  # the process dies without RELEASE
    proc.join(20)
    deadline = time.time() + 5
    while srv.stats()["replicas_lost"] == 0 and time.time() < deadline:
        time.sleep(0.01)
    assert srv.stats()["replicas_lost"] == 1
    cli2 = C.Client(cp, req_size=1024, resp_size=1024, total=80, warmup=0, payload="echo", verify=True, seed=5)
    assert cli2.run_closed_loop(8) and cli2.received == 80 and cli2.verify_failures == 0
    after = srv.stats()
    srv.stop()
    assert after["replicas"][1]["steered"] == before["replicas"][1]["steered"]
    assert after["replicas"][0]["steered"] == before["replicas"][0]["steered"] + 80


def test_batched_server_survives_a_producer_that_vanishes(C, mtu1k, tmp_path):
    """A producer that disconnects without RELEASE is counted as lost; the server stops its worker, forgets the
    producer's arena and accepts the next ALLOC."""
    path = str(tmp_path / "bs.sock")
    app = C.make_app("echo", -1, 1024, 1024, [], 64, 1, 4, "cpu")
    bs = C.BatchedServer(app, path, func_id=FUNC, server_mode=2, max_batch=4)
    bs.start()
    for round_ in range(2):
        srv, cp = _ingress(C, [path], req=1024, resp=1024)
        assert bs.serving
        srv.start()
        cli = C.Client(cp, req_size=1024, resp_size=1024, total=40, warmup=0, payload="echo", verify=True)
        assert cli.run_closed_loop(4) and cli.received == 40 and cli.verify_failures == 0
        srv.stop()
        del cli, srv, cp  # closes the control connection without RELEASE
        deadline = time.time() + 5
        while bs.serving and time.time() < deadline:
            time.sleep(0.01)
        assert not bs.serving and bs.counters()["peers_lost"] == round_ + 1
    # a second producer while one is connected is refused; a wrong function id too
    srv, cp = _ingress(C, [path], req=1024, resp=1024)
    with pytest.raises(RuntimeError):
        _ingress(C, [path], req=1024, resp=1024)
    sp2, _ = C.make_loopback_pair(1024, 256, "shm")
    other = C.Server(sp2, req_size=1024, resp_size=1024, server_mode=2, max_batch=4)
    with pytest.raises(RuntimeError):
        other.add_remote_replica(path, func_id=FUNC + 1, ingress_device=-1, timeout_ms=500)
    assert srv.release_remotes() == 1
    assert bs.counters()["refused"] >= 1 and bs.counters()["releases"] == 1
    bs.stop()
    assert not os.path.exists(path)


def test_host_driven_completion_still_works(C, mtu1k):
    """device_completion=0 keeps the original division of labour: the worker marks slots, the shunter scatters."""
    sp, cp = C.make_loopback_pair(1024, 2048)
    app = C.make_app("echo", -1, 1024, 1024, [], 64, 1, 4, "cpu")
    srv = C.Server(sp, req_size=1024, resp_size=1024, server_mode=2, max_batch=4, device_completion=0)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=1024, resp_size=1024, total=50, warmup=0, payload="echo", verify=True)
    assert cli.run_closed_loop(4) and cli.received == 50 and cli.verify_failures == 0
    st = srv.stats()
    srv.stop()
    assert st["replicas"][0]["pushed"] == 0 and not app.completion_by_device


def test_serving_side_refuses_malformed_descriptors(C, mtu1k, tmp_path):
    """Descriptor blocks are written by another process, so the serving side checks them: an unknown region, a fragment
    past the end of its region, more bytes than a ring slot holds and an empty list are counted as fetch errors and
    nothing is copied; the slot is still handed on, so the ring does not stall."""
    proc, path, stop, out = _spawn(tmp_path, "bad", mode=-1, resp=1024)  # no worker: the test watches the slot states
    try:
        srv, cp = _ingress(C, [path], resp=1024, pull=True)
        assert srv.remote_info(0)["pull"] == 1
        arena = 1024 * 2048  # the receive arena of _ingress (region 0)
        bad = [
            [(3, 0, 1024)],                       # region that was never shared
            [(0, arena - 512, 1024)],             # runs past the end of region 0
            [(0, 0, 4096), (0, 4096, 1024)],      # 5120 bytes into a 4096-byte slot
            [],                                   # nothing at all
        ]
        for slot, frags in enumerate(bad):
            srv.remote_describe_raw(0, slot, frags)
        deadline = time.time() + 5
        while time.time() < deadline and any(srv.remote_slot_state(0, s) != 1 for s in range(len(bad))):
            time.sleep(0.01)
        assert [srv.remote_slot_state(0, s) for s in range(len(bad))] == [1] * len(bad)  # RX_COMPLETE
        # a well-formed list right after them is fetched
        srv.remote_describe_raw(0, len(bad), [(0, 0, 4096)])
        deadline = time.time() + 5
        while time.time() < deadline and srv.remote_slot_state(0, len(bad)) != 1:
            time.sleep(0.01)
        assert srv.remote_slot_state(0, len(bad)) == 1
        srv.release_remotes()
    finally:
        stop.set()
        _, _, pulled = out.get(timeout=20)
        proc.join(20)
    assert pulled["errors"] == len(bad) and pulled["pulled"] == len(bad) + 1
