"""The comparison system on a GPU app: requests through gRPC and the copy path (a copy to the device and back per
request) against the same app behind this package's server, same request size and number of outstanding requests."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
grpc = pytest.importorskip("grpc")


def test_copy_path_against_split_path_on_gpu(C):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from splitrpc_b200.utils.grpc_baseline import GrpcClient, GrpcCopyPathServer

    size, outstanding, total = 8192, 8, 600
    app = C.make_app("echo", 0, size, size, [], 64, 1, 8)
    with GrpcCopyPathServer(app, 8) as srv:
        cli = GrpcClient(srv.address, size)
        copy = cli.run_closed_loop(outstanding, total, warmup=100, keep=8)
        assert copy["received"] == total and copy["errors"] == 0
        for guid, out in cli.responses.items():
            assert out == cli.payloads[guid % len(cli.payloads)]
        cli.close()
        t = srv.times()
    per_req = {k: t[k] / t["requests"] / 1e3 for k in ("h2d_ns", "run_ns", "d2h_ns")}

    C.set_rpc_mtu(8192)
    sp, cp = C.make_loopback_pair(8192, 1024, "pinned")
    app2 = C.make_app("echo", 0, size, size, [], 256, 1, 8, "gpu")
    s = C.Server(sp, req_size=size, resp_size=size, server_mode=2, max_batch=8)
    s.add_replica(app2)
    s.start()
    c2 = C.Client(cp, req_size=size, resp_size=size, total=total + 100, warmup=100, payload="echo", verify=True)
    assert c2.run_closed_loop(outstanding) and c2.received == total + 100
    s.stop()
    st = c2.post_process()
    print(f"echo {size} B, {outstanding} outstanding: gRPC + copy path {copy['req_per_s']:.0f} req/s, p50 {copy['p50_us']:.0f} us, "
          f"p99 {copy['p99_us']:.0f} us (per request: copy in {per_req['h2d_ns']:.1f} us, run {per_req['run_ns']:.1f} us, "
          f"copy out {per_req['d2h_ns']:.1f} us; mean batch {t['requests'] / t['batches']:.1f}); this package's server over "
          f"the loopback port {st['throughput_est']:.0f} req/s, p50 {st['p50_sojournTime_us']:.0f} us, p99 {st['p99_sojournTime_us']:.0f} us")
