"""End-to-end tests on CPU: loopback transport, CPU scatter-gather engine, CPU apps,
load generator; failure detection through host-side fault injection."""
import json

import numpy as np
import pytest

from conftest import lenet5_weights


def _serve(C, app_name, req, resp, total, mode, max_batch, payload, outstanding=8, weights=(), zerocopy=0, engine="",
           mtu_slots=8192, faults=None, drain_ns=10_000_000_000, open_rate=None, warmup=10, dma_lanes=1):
    sp, cp = C.make_loopback_pair(mtu_slots, 2048)
    if dma_lanes > 1:
        C.set_loopback_dma_lanes(cp, dma_lanes)
        C.set_loopback_dma_lanes(sp, dma_lanes)
    if faults:
        C.set_loopback_faults(cp, **faults)
    app = C.make_app(app_name, -1, req, resp, list(weights), 256, 1, max_batch, engine)
    srv = C.Server(sp, req_size=req, resp_size=resp, server_mode=mode, max_batch=max_batch, zerocopy=zerocopy,
                   reassembly_timeout_ns=50_000_000)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=warmup, payload=payload, verify=True,
                   drain_timeout_ns=drain_ns)
    ok = cli.run_open_loop(open_rate, 1, 2) if open_rate else cli.run_closed_loop(outstanding)
    stats = cli.post_process()
    sstats = srv.stats()
    wstats = srv.worker_stats(0)
    srv.stop()
    return ok, cli, stats, sstats, wstats


@pytest.mark.parametrize("mode,max_batch", [(0, 1), (0, 4), (2, 8), (1, 1), (1, 4)])
def test_echo_multi_fragment_all_server_modes(C, mtu1k, mode, max_batch):
    ok, cli, st, ss, ws = _serve(C, "echo", 5000, 5000, 400, mode, max_batch, "echo", outstanding=8, mtu_slots=1024)
    assert ok and cli.received == 400 and cli.verify_failures == 0 and cli.bad_tokens == 0
    assert st["incorrect_state_calls"] == 0 and st["recorded"] == 390
    assert ss["rx_pkts"] == 400 * 5 and ss["tx_pkts"] == 400 * 5
    if mode != 2:
        assert set(ws["batch_hist"]) == {max_batch}
    else:
        assert max(ws["batch_hist"]) <= max_batch


def test_emulated_dma_with_several_copy_lanes(C, mtu1k):
    """Bursts of eight fragments or more are written by three threads; duplicates and reordering on the wire on top."""
    ok, cli, st, ss, ws = _serve(C, "echo", 20000, 20000, 300, 2, 4, "echo", outstanding=8, mtu_slots=1024, dma_lanes=3,
                                 faults=dict(duplicate=0.05, reorder=0.1, seed=5))
    assert ok and cli.received == 300 and cli.verify_failures == 0 and cli.bad_tokens == 0
    assert ss["rx_pkts"] >= 300 * 20


def test_vec_add_large_request(C, mtu8k):
    ok, cli, st, ss, ws = _serve(C, "vec_add", 1 << 20, 1 << 20, 40, 2, 4, "vec_add", outstanding=4)
    assert ok and cli.received == 40 and cli.verify_failures == 0
    assert ss["rx_pkts"] == 40 * 128


def test_zero_copy_mode_single_fragment(C, mtu1k):
    ok, cli, st, ss, ws = _serve(C, "vec_add", 1024, 1024, 300, 2, 4, "vec_add", zerocopy=1, engine="zc", mtu_slots=1024)
    assert ok and cli.received == 300 and cli.verify_failures == 0


def test_lenet5_dynamic_batching_matches_oracle(C, mtu8k):
    w = lenet5_weights()
    ok, cli, st, ss, ws = _serve(C, "lenet5", 3136, 40, 600, 2, 32, "uniform", outstanding=48, weights=w)
    assert ok and cli.received == 600
    assert max(ws["batch_hist"]) <= 32 and max(ws["batch_hist"]) > 1
    for i in (0, 7, 599):
        x = np.frombuffer(cli.payload(i % 16), dtype=np.float32)
        ref = C.cpu_lenet5(w, x)[0]
        got = np.frombuffer(cli.response(i), dtype=np.float32)
        np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)
        assert abs(got.sum() - 1.0) < 1e-4


def test_matmul_app(C, mtu8k):
    sp, cp = C.make_loopback_pair(8192, 512)
    app = C.make_app("matmul", -1, 8192, 4096, [], 64, 1, 1)
    srv = C.Server(sp, req_size=8192, resp_size=4096, server_mode=0, max_batch=1)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=8192, resp_size=4096, total=20, warmup=0, payload="uniform", verify=True)
    assert cli.run_closed_loop(2)
    srv.stop()
    req = np.frombuffer(cli.payload(3), dtype=np.float32)
    a, b = req[:1024].reshape(32, 32), req[1024:].reshape(32, 32)
    got = np.frombuffer(cli.response(3), dtype=np.float32).reshape(32, 32)
    np.testing.assert_allclose(got, a @ b, rtol=1e-4, atol=1e-5)


def test_open_loop_poisson_and_stats_file(C, mtu1k, tmp_path):
    sp, cp = C.make_loopback_pair(1024, 2048)
    app = C.make_app("echo", -1, 1024, 1024, [], 256, 1, 8)
    srv = C.Server(sp, req_size=1024, resp_size=1024, server_mode=2, max_batch=8)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=1024, resp_size=1024, total=500, warmup=50, payload="echo", verify=True,
                   exp_name="openloop", out_dir=str(tmp_path))
    assert cli.run_open_loop(5000.0, 1, 2)
    st = cli.post_process()
    fn = cli.save_stats()
    srv.stop()
    data = json.load(open(fn))
    for k in ("n_sojournTime", "min_sojournTime_us", "max_sojournTime_us", "mean_sojournTime_us", "p50_sojournTime_us",
              "p90_sojournTime_us", "p95_sojournTime_us", "p99_sojournTime_us", "p999_sojournTime_us", "throughput_est",
              "n_r_sent", "n_r_recv", "recorded", "warmup_calls", "incorrect_state_calls"):
        assert k in data
    assert data["n_sojournTime"] == 450 and data["warmup_calls"] == 50
    assert 2000 < data["throughput_est"] < 10000


def test_arrival_processes(C):
    det = np.diff([0] + C.arrival_schedule(1000.0, 0, 1000, 1))
    assert np.all(det == 1_000_000)
    exp = np.diff([0] + C.arrival_schedule(1000.0, 1, 20000, 1)).astype(np.float64)
    assert abs(exp.mean() - 1e6) / 1e6 < 0.05 and abs(exp.std() / exp.mean() - 1.0) < 0.05
    hyp = np.diff([0] + C.arrival_schedule(1000.0, 4, 40000, 1)).astype(np.float64)
    assert abs(hyp.mean() - 1e6) / 1e6 < 0.08
    assert abs((hyp.std() / hyp.mean()) ** 2 - 4.0) < 0.6


# ---- failure detection: all faults are injected on the host, in the loopback link

def test_dropped_fragments_expire_and_do_not_leak(C, mtu1k):
    ok, cli, st, ss, ws = _serve(C, "echo", 4096, 4096, 200, 2, 4, "echo", outstanding=4, mtu_slots=1024,
                                 faults=dict(drop=0.05, seed=7), drain_ns=600_000_000, open_rate=4000.0)
    # some requests lose a fragment: the client times out on those, the server reclaims them
    # (open loop: a lost request must not stall the arrivals behind it)
    assert cli.received < 200 and cli.received > 50
    assert cli.verify_failures == 0
    assert ss["expired"] > 0
    assert st["incorrect_state_calls"] > 0


def test_duplicates_and_reordering_are_tolerated(C, mtu1k):
    ok, cli, st, ss, ws = _serve(C, "echo", 4096, 4096, 200, 2, 4, "echo", outstanding=4, mtu_slots=1024,
                                 faults=dict(duplicate=0.1, reorder=0.3, seed=3))
    assert cli.received == 200 and cli.verify_failures == 0
    assert ss["dropped_pkts"] > 0  # the duplicates


def test_zero_token_and_bad_sequence_packets_are_dropped(C, mtu1k):
    for faults in (dict(zero_token=True), dict(force_seq=5000)):
        ok, cli, st, ss, ws = _serve(C, "echo", 1024, 1024, 20, 0, 1, "echo", outstanding=2, mtu_slots=1024,
                                     faults=faults, drain_ns=200_000_000)
        assert cli.received == 0 and ss["dropped_pkts"] == ss["rx_pkts"] > 0 and ss["rx_reqs"] == 0


def test_in_range_sequence_gap_never_reaches_the_engine(C, mtu1k):
    """A single-fragment request stamped with sequence number 3 has all its bytes but leaves indices 0..2 unfilled:
    the server must drop it instead of building a copy list from them (CPU engine only)."""
    ok, cli, st, ss, ws = _serve(C, "echo", 1024, 1024, 20, 0, 1, "echo", outstanding=2, mtu_slots=1024,
                                 faults=dict(force_seq=3), drain_ns=200_000_000)
    assert cli.received == 0 and ss["rx_reqs"] == 0 and ws["num_req"] == 0
    assert ss["dropped_pkts"] == ss["rx_pkts"] > 0


def test_replica_marked_down_is_skipped_by_steering(C, mtu1k):
    sp, cp = C.make_loopback_pair(1024, 2048)
    apps = [C.make_app("echo", -1, 1024, 1024, [], 128, 1, 4) for _ in range(3)]
    srv = C.Server(sp, req_size=1024, resp_size=1024, server_mode=2, max_batch=4)
    for a in apps:
        srv.add_replica(a)
    srv.mark_replica_down(1, True)
    srv.start()
    cli = C.Client(cp, req_size=1024, resp_size=1024, total=600, warmup=0, payload="echo", verify=True)
    assert cli.run_closed_loop(8) and cli.received == 600 and cli.verify_failures == 0
    reps = srv.stats()["replicas"]
    srv.stop()
    assert reps[1]["steered"] == 0 and reps[0]["steered"] > 0 and reps[2]["steered"] > 0
    assert reps[0]["steered"] + reps[2]["steered"] == 600


def test_python_app_callback(C, mtu1k):
    import ctypes

    def run(req, resp, batch, stream, d_stub):
        ctypes.memmove(resp, req, batch * 1024)

    sp, cp = C.make_loopback_pair(1024, 512)
    app = C.make_python_app(run, -1, 1024, 1024, 64, 1, 1)
    srv = C.Server(sp, req_size=1024, resp_size=1024, server_mode=2, max_batch=4)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=1024, resp_size=1024, total=50, warmup=0, payload="echo", verify=True)
    assert cli.run_closed_loop(2) and cli.verify_failures == 0 and cli.received == 50
    srv.stop()


def test_udp_socket_transport(C, mtu1k):
    sp, sport = C.make_udp_port("127.0.0.1", 0, 1024, 512)
    cp, cport = C.make_udp_port("127.0.0.1", 0, 1024, 512, "127.0.0.1", sport)
    app = C.make_app("vec_add", -1, 3000, 3000, [], 64, 1, 2)
    srv = C.Server(sp, req_size=3000, resp_size=3000, server_mode=2, max_batch=2)
    srv.add_replica(app)
    srv.start()
    uri = f"00:00:00:00:00:01,127.0.0.1,{cport},00:00:00:00:00:02,127.0.0.1,{sport}"
    cli = C.Client(cp, req_size=3000, resp_size=3000, total=100, warmup=0, payload="vec_add", verify=True, uri=uri)
    assert cli.run_closed_loop(2) and cli.received == 100 and cli.verify_failures == 0
    srv.stop()


def test_local_bench_cpu(C):
    app = C.make_app("vec_add", -1, 1024, 1024, [], 64, 1, 1)
    ns, outs = C.local_bench(app, 50, 2)
    assert len(ns) == 50 and all(n > 0 for n in ns)


def test_model_files_in_the_original_formats(C, mtu8k, tmp_path):
    """LeNet: four raw fp32 blobs under data/lenet/; LSTM: one Constant_<id>_0.bin per tensor plus a manifest."""
    rng = np.random.default_rng(4)
    shapes = {"data2.dat": (20, 1, 5, 5), "data0.dat": (50, 20, 5, 5), "data1.dat": (10, 1250), "data3.dat": (10,)}
    d = tmp_path / "data" / "lenet"
    d.mkdir(parents=True)
    w = {}
    for name, shape in shapes.items():
        w[name] = (rng.standard_normal(shape) * 0.1).astype(np.float32)
        w[name].tofile(d / name)
    got = C.load_lenet_ref_weights(str(tmp_path))
    for arr, name in zip(got, ("data2.dat", "data0.dat", "data1.dat", "data3.dat")):
        assert np.array_equal(arr, w[name].ravel())
    # the loaded weights serve the reference-format LeNet: uint8 images in, 10 probabilities out
    sp, cp = C.make_loopback_pair(8192, 512)
    app = C.make_app("lenet_ref", -1, 784, 40, got, 64, 1, 4, "cpu")
    srv = C.Server(sp, req_size=784, resp_size=40, server_mode=2, max_batch=4)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=784, resp_size=40, total=12, warmup=0, payload="echo", verify=True)
    assert cli.run_closed_loop(4) and cli.received == 12
    srv.stop()
    assert abs(float(np.frombuffer(cli.response(3), dtype=np.float32).sum()) - 1.0) < 1e-4
    with pytest.raises(RuntimeError):
        C.load_lenet_ref_weights(str(tmp_path / "nowhere"))

    # LSTM: 2 layers, hidden 8 for the test; ids shuffled, matrices stored [in][out] (flag T) as a Dot node wants them
    L, H = 2, 8
    cdir = tmp_path / "Constant"
    cdir.mkdir()
    ids = list(rng.permutation(200)[: L * 12])
    lines, want = ["# layer kind gate id [T]"], []
    k = 0
    for layer in range(L):
        Wm, Um = (rng.standard_normal((4, H, H)).astype(np.float32) for _ in range(2))
        b = rng.standard_normal((4, H)).astype(np.float32)
        for kind, t in (("W", Wm), ("U", Um), ("b", b)):
            for g, gate in enumerate("igfo"):
                cid = int(ids[k]); k += 1
                if kind == "b":
                    t[g].tofile(cdir / f"Constant_{cid}_0.bin")
                    lines.append(f"{layer} {kind} {gate} {cid}")
                else:
                    np.ascontiguousarray(t[g].T).tofile(cdir / f"Constant_{cid}_0.bin")
                    lines.append(f"{layer} {kind} {gate} {cid} T")
        want += [Wm.ravel(), Um.ravel(), b.ravel()]
    (tmp_path / "lstm.manifest").write_text("\n".join(lines) + "\n")
    got = C.load_lstm_constants(str(cdir), str(tmp_path / "lstm.manifest"), L, H)
    assert len(got) == 3 * L and all(np.array_equal(a, b_) for a, b_ in zip(got, want))
    x = rng.standard_normal((3, H)).astype(np.float32)
    y = C.cpu_lstm(got, x, L, 3, H)
    assert y.shape == (H,) and np.all(np.isfinite(y)) and float(np.abs(y).max()) <= 1.0
    (tmp_path / "short.manifest").write_text("\n".join(lines[:5]) + "\n")
    with pytest.raises(RuntimeError):
        C.load_lstm_constants(str(cdir), str(tmp_path / "short.manifest"), L, H)
