"""GPU tests of the scatter-gather kernels, ring memory and the GPU apps behind the server."""
import numpy as np
import pytest

from conftest import lenet5_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


def _random_list(torch, rng, n_items, max_len, align):
    total = n_items * (max_len + 64)
    src = torch.randint(0, 256, (total,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(total, dtype=torch.uint8, device="cuda")
    ref = torch.zeros(total, dtype=torch.uint8, device="cuda")
    items = []
    so = do = 0
    for _ in range(n_items):
        ln = int(rng.integers(1, max_len + 1))
        s_off = so + (int(rng.integers(0, 16)) if not align else 0)
        d_off = do + (int(rng.integers(0, 16)) if not align else 0)
        if align:
            ln = (ln + 15) // 16 * 16
        items.append((src.data_ptr() + s_off, dst.data_ptr() + d_off, ln))
        ref[d_off:d_off + ln] = src[s_off:s_off + ln]
        so = (s_off + ln + 15) // 16 * 16
        do = (d_off + ln + 15) // 16 * 16
    return src, dst, ref, items


@pytest.mark.parametrize("impl", [0, 1])
@pytest.mark.parametrize("align", [True, False])
def test_sg_copy_matches_reference(C, torch_cuda, impl, align):
    torch = torch_cuda
    rng = np.random.default_rng(5 + impl)
    src, dst, ref, items = _random_list(torch, rng, 37, 70000, align)
    C.sg_copy(items, impl)
    torch.cuda.synchronize()
    assert torch.equal(dst, ref)


@pytest.mark.parametrize("n_blocks", [-1, -3, -12, 5])
def test_sg_copy_fat_blocks(C, torch_cuda, n_blocks):
    """Negative block counts run 1024-thread blocks (four chunk groups each); unaligned items take the byte paths."""
    torch = torch_cuda
    rng = np.random.default_rng(11)
    for align in (True, False):
        src, dst, ref, items = _random_list(torch, rng, 53, 90000, align)
        C.sg_copy(items, 0, n_blocks)
        torch.cuda.synchronize()
        assert torch.equal(dst, ref)


def test_persistent_grid_leaves_reserved_sms(C, torch_cuda):
    """gemm_reserve_sms shrinks the persistent grids; results do not change."""
    torch = torch_cuda
    from splitrpc_b200 import ops

    a = (torch.randn(1024, 512, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(768, 512, device="cuda") * 0.3).bfloat16()
    full = C.gemm_grid_sms() + C.gemm_reserved_sms()
    try:
        C.gemm_reserve_sms(12)
        assert C.gemm_grid_sms() == full - 12 and C.gemm_reserved_sms() == 12
        got = ops.gemm(a, b)
    finally:
        C.gemm_reserve_sms(0)
    want = ops.gemm(a, b)
    ops.check_status()
    assert torch.equal(got, want)
    ref = a.float() @ b.float().t()
    assert ((got.float() - ref).norm() / ref.norm()).item() < 1e-2


def test_sg_copy_from_mapped_host_memory(C, torch_cuda):
    torch = torch_cuda
    host = torch.randint(0, 256, (1 << 20,), dtype=torch.uint8).pin_memory()
    dst = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    for impl in (0, 1):
        dst.zero_()
        items = [(host.data_ptr() + i * 8192, dst.data_ptr() + i * 8192, 8192) for i in range(128)]
        C.sg_copy(items, impl)
        torch.cuda.synchronize()
        assert torch.equal(dst.cpu(), host)


def test_sg_cast_bf16(C, torch_cuda):
    torch = torch_cuda
    x = torch.randn(3 * 224 * 224 * 2, device="cuda")
    out = torch.zeros(x.numel(), dtype=torch.bfloat16, device="cuda")
    half = x.numel() // 2
    items = [(x.data_ptr(), out.data_ptr(), half * 4), (x.data_ptr() + half * 4, out.data_ptr() + half * 2, half * 4)]
    C.sg_cast_bf16(items, 0.5, 0.25)
    torch.cuda.synchronize()
    ref = ((x - 0.25) * 0.5).to(torch.bfloat16)
    assert torch.equal(out, ref)


def test_device_caps(C, torch_cuda):
    caps = C.device_caps(0)
    assert caps["sm"] >= 100 and caps["vmm"] == 1 and caps["num_sms"] > 100


def test_ring_is_double_mapped(C, torch_cuda):
    import ctypes

    torch = torch_cuda
    app = C.make_app("echo", 0, 3000, 3000, [], 64, 1, 1)
    base, cap, dbl = app.req_ring
    assert dbl and cap >= 64 * 3000
    # bytes written through the first mapping are visible through the second
    src = torch.arange(256, dtype=torch.uint8, device="cuda")
    C.sg_copy([(src.data_ptr(), base + cap - 128, 256)], 0)  # runs across the end of the ring
    back = torch.zeros(256, dtype=torch.uint8, device="cuda")
    C.sg_copy([(base + cap - 128, back.data_ptr(), 128), (base, back.data_ptr() + 128, 128)], 0)
    torch.cuda.synchronize()
    assert torch.equal(back, src)


def _serve_gpu(C, app_name, req, resp, total, mode, max_batch, payload, copy_type, launch_type=1, weights=(),
               outstanding=8, slot=8192):
    sp, cp = C.make_loopback_pair(slot, 2048, "pinned")
    app = C.make_app(app_name, 0, req, resp, list(weights), 256, launch_type, max_batch, "gpu", copy_type)
    assert app.init_ok
    srv = C.Server(sp, req_size=req, resp_size=resp, server_mode=mode, max_batch=max_batch)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=5, payload=payload, verify=True)
    ok = cli.run_closed_loop(outstanding)
    st = cli.post_process()
    ss = srv.stats()
    ws = srv.worker_stats(0)
    sg = app.sg_counters
    srv.stop()
    return ok, cli, st, ss, ws, sg


@pytest.mark.parametrize("copy_type", [0, 1, 2, 3])
def test_gpu_echo_all_copy_types(C, torch_cuda, mtu8k, copy_type):
    ok, cli, st, ss, ws, sg = _serve_gpu(C, "echo", 40000, 40000, 120, 2, 8, "echo", copy_type)
    assert ok and cli.received == 120 and cli.verify_failures == 0
    assert ss["sg_errors"] == 0 and sg["timeouts"] == 0 and sg["engine"] == "gpu"


@pytest.mark.parametrize("launch_type", [1, 3, 4])
def test_gpu_vec_add_launch_types(C, torch_cuda, mtu8k, launch_type):
    ok, cli, st, ss, ws, sg = _serve_gpu(C, "vec_add", 16384, 16384, 100, 2, 4, "vec_add", 2, launch_type)
    assert (ok, cli.received, cli.verify_failures, ws["wait_timeouts"], ss["sg_errors"]) == (True, 100, 0, 0, 0), (ws["batch_hist"], ss)


def test_gpu_async_stream_armed_mode(C, torch_cuda, mtu8k):
    ok, cli, st, ss, ws, sg = _serve_gpu(C, "vec_add", 8192, 8192, 200, 1, 4, "vec_add", 2, outstanding=8)
    assert ok and cli.received == 200 and cli.verify_failures == 0
    assert set(ws["batch_hist"]) == {4}


@pytest.mark.parametrize("launch_type", [1, 3, 4])
def test_gpu_lenet5_matches_cpu_oracle(C, torch_cuda, mtu8k, launch_type):
    """Kernel launch per batch, resident kernel behind the doorbell (launch type 3), CUDA graph."""
    w = lenet5_weights()
    ok, cli, st, ss, ws, sg = _serve_gpu(C, "lenet5", 3136, 40, 400, 2, 32, "uniform", 2, launch_type, weights=w, outstanding=64)
    assert ok and cli.received == 400 and ws["wait_timeouts"] == 0
    for i in (0, 100, 399):
        x = np.frombuffer(cli.payload(i % 16), dtype=np.float32)
        ref = C.cpu_lenet5(w, x)[0]
        got = np.frombuffer(cli.response(i), dtype=np.float32)
        np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("launch_type", [1, 3])
def test_gpu_matmul(C, torch_cuda, mtu8k, launch_type):
    sp, cp = C.make_loopback_pair(8192, 1024, "pinned")
    app = C.make_app("matmul", 0, 32768, 16384, [], 64, launch_type, 2, "gpu", 2)
    assert app.init_ok
    srv = C.Server(sp, req_size=32768, resp_size=16384, server_mode=2, max_batch=2)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=32768, resp_size=16384, total=20, warmup=0, payload="uniform", verify=True)
    assert cli.run_closed_loop(2)
    srv.stop()
    req = np.frombuffer(cli.payload(5), dtype=np.float32)
    a, b = req[:4096].reshape(64, 64), req[4096:].reshape(64, 64)
    got = np.frombuffer(cli.response(5), dtype=np.float32).reshape(64, 64)
    np.testing.assert_allclose(got, a @ b, rtol=1e-4, atol=1e-4)


def test_resident_launch_type_is_refused_where_it_does_not_exist(C, torch_cuda):
    """Launch type 3 exists for vec_add, matmul and lenet5; asking for it elsewhere fails the app's init instead of
    silently running something else."""
    app = C.make_app("echo", 0, 1024, 1024, [], 64, 3, 1, "gpu", 2)
    assert not app.init_ok


def test_local_bench_gpu(C, torch_cuda):
    app = C.make_app("vec_add", 0, 1024, 1024, [], 64, 1, 1, "gpu", 2)
    ns, outs = C.local_bench(app, 200, 1)
    assert len(ns) == 200


def test_gpu_header_swap_matches_host(C, torch_cuda):
    torch = torch_cuda
    uri = "b8:ce:f6:cc:6a:53,192.168.25.2,50052,b8:ce:f6:cc:6a:52,192.168.25.1,50051"
    tmpl = C.client_conn_template(uri)
    hdrs = [C.build_fragments(tmpl, 1000 + i, bytes(100 + i), 1024)[0][0] for i in range(300)]
    dev = torch.tensor(np.frombuffer(b"".join(hdrs), dtype=np.uint8).copy(), device="cuda")
    C.swap_hdrs(0, dev.data_ptr(), 300, False, 0)
    torch.cuda.synchronize()
    got = dev.cpu().numpy().tobytes()
    for i in (0, 77, 299):
        assert got[i * 64:(i + 1) * 64] == C.swap_header(hdrs[i])


@pytest.mark.parametrize("launch_type", [1, 2])
def test_gpu_header_processor_api(C, torch_cuda, launch_type, monkeypatch):
    """setup_g_pp / do_g_pp / stop_g_pp: per-burst launches and the resident kernel, which leaves after its idle limit
    and is started again by the next burst."""
    import time

    torch = torch_cuda
    monkeypatch.setenv("P2P_RPC_G_PP_IDLE_MS", "5")
    uri = "b8:ce:f6:cc:6a:53,192.168.25.2,50052,b8:ce:f6:cc:6a:52,192.168.25.1,50051"
    tmpl = C.client_conn_template(uri)
    h = C.g_pp_setup(0, launch_type)
    try:
        for burst in range(3):
            n = (5, 300, 1024)[burst]
            hdrs = [C.build_fragments(tmpl, 5000 + 7 * burst + i, bytes(64 + (i % 50)), 1024)[0][0] for i in range(n)]
            dev = torch.tensor(np.frombuffer(b"".join(hdrs), dtype=np.uint8).copy(), device="cuda")
            addrs = [dev.data_ptr() + 64 * i for i in range(n)]
            assert C.g_pp_do(h, addrs, burst == 1) == 0
            torch.cuda.synchronize()
            got = dev.cpu().numpy().tobytes()
            for i in (0, n // 2, n - 1):
                want = C.swap_header(hdrs[i])
                if burst == 1:  # the sockperf word's low half is cleared: compare the routing part only
                    assert got[i * 64:i * 64 + 42] == want[:42]
                else:
                    assert got[i * 64:(i + 1) * 64] == want
            time.sleep(0.05)  # longer than the idle limit: the resident kernel leaves
        ctr = C.g_pp_counters(h)
        assert ctr["bursts"] == 3 and ctr["timeouts"] == 0 and ctr["launch_type"] == launch_type
        if launch_type == 2:
            assert ctr["rearmed"] >= 1
    finally:
        C.g_pp_stop(h)


def test_resident_copy_engine_leaves_when_idle_and_is_rearmed(C, torch_cuda, mtu8k, monkeypatch):
    """Copy type 1: the resident copy kernel leaves after P2P_RPC_SG_IDLE_MS without work; the next gather starts it
    again and is served correctly."""
    import time

    monkeypatch.setenv("P2P_RPC_SG_IDLE_MS", "5")
    sp, cp = C.make_loopback_pair(8192, 2048, "pinned")
    app = C.make_app("echo", 0, 40000, 40000, [], 256, 1, 8, "gpu", 1)
    srv = C.Server(sp, req_size=40000, resp_size=40000, server_mode=2, max_batch=8)
    srv.add_replica(app)
    srv.start()
    try:
        for rnd in range(3):
            cli = C.Client(cp, req_size=40000, resp_size=40000, total=24, warmup=0, payload="echo", verify=True, seed=rnd + 1)
            assert cli.run_closed_loop(4) and cli.received == 24 and cli.verify_failures == 0
            time.sleep(0.06)  # idle for much longer than the limit
        assert app.sg_counters["timeouts"] == 0 and srv.stats()["sg_errors"] == 0
    finally:
        srv.stop()


def test_gpu_lenet_ref_and_lstm_match_cpu_oracles(C, torch_cuda, mtu8k):
    rng = np.random.default_rng(3)
    w = [(rng.standard_normal(s) * 0.1).astype(np.float32) for s in [(20, 1, 5, 5), (50, 20, 5, 5), (10, 1250), (10,)]]
    outs = {}
    for dev in (-1, 0):
        sp, cp = C.make_loopback_pair(8192, 512, "pinned" if dev >= 0 else "malloc")
        app = C.make_app("lenet_ref", dev, 784, 40, w, 64, 1, 4)
        srv = C.Server(sp, req_size=784, resp_size=40, server_mode=2, max_batch=4)
        srv.add_replica(app)
        srv.start()
        cli = C.Client(cp, req_size=784, resp_size=40, total=40, warmup=0, payload="echo", verify=True)
        assert cli.run_closed_loop(4) and cli.received == 40
        srv.stop()
        outs[dev] = np.frombuffer(cli.response(7), dtype=np.float32).copy()
    np.testing.assert_allclose(outs[0], outs[-1], rtol=1e-3, atol=1e-5)
    H = 256
    lw = []
    for _ in range(8):
        lw += [(rng.standard_normal((4, H, H)) * 0.05).astype(np.float32), (rng.standard_normal((4, H, H)) * 0.05).astype(np.float32),
               (rng.standard_normal((4, H)) * 0.1).astype(np.float32)]
    sp, cp = C.make_loopback_pair(8192, 512, "pinned")
    app = C.make_app("lstm", 0, 8192, 1024, lw, 64, 1, 4)
    srv = C.Server(sp, req_size=8192, resp_size=1024, server_mode=2, max_batch=4)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=8192, resp_size=1024, total=24, warmup=0, payload="uniform", verify=True)
    assert cli.run_closed_loop(4) and cli.received == 24
    srv.stop()
    x = np.frombuffer(cli.payload(3), dtype=np.float32)
    ref = C.cpu_lstm(lw, x, 8, 8, H)
    got = np.frombuffer(cli.response(3), dtype=np.float32)
    np.testing.assert_allclose(got, ref, rtol=1e-3, atol=1e-4)
