"""Failure detection on the GPU without faulting it: a bounded device-side wait runs out on purpose (nothing ever sets
the flag it waits for), the kernel returns an error status that the host reads, and the context stays usable."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


def test_tp_flag_wait_runs_out_and_reports(C, torch_cuda):
    torch = torch_cuda
    from splitrpc_b200 import ops

    ops.check_status()
    C.tp_set_wait_ns(2_000_000)  # 2 ms instead of 2 s
    try:
        flags = torch.zeros(4, dtype=torch.int32, device="cuda")  # nobody will ever raise these
        base = torch.zeros(1, dtype=torch.int32, device="cuda")
        t0 = time.perf_counter()
        C.tp_wait(flags.data_ptr(), 4, 7, base.data_ptr(), ops.status_word().data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        took = time.perf_counter() - t0
        assert took < 1.0, f"the bounded wait took {took:.3f} s"
        with pytest.raises(RuntimeError, match="status 4"):
            ops.check_status()
        ops.check_status()  # the status word was cleared
        # the context is intact: a tensor-core GEMM right after gives the right answer
        a = torch.randn(256, 128, device="cuda").bfloat16()
        b = torch.randn(192, 128, device="cuda").bfloat16()
        out = ops.gemm(a, b)
        ref = a.float() @ b.float().t()
        assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
        # a wait whose flags are already there returns at once and reports nothing
        flags.fill_(9)
        C.tp_wait(flags.data_ptr(), 4, 7, base.data_ptr(), ops.status_word().data_ptr(), torch.cuda.current_stream().cuda_stream)
        ops.check_status()
    finally:
        C.tp_set_wait_ns(2_000_000_000)


def test_stream_armed_worker_shuts_down_while_armed(C, torch_cuda):
    """Mode 1 parks the work stream on a slot doorbell before any request exists.  Stopping the server in that state must
    release the stream and return promptly."""
    C.set_rpc_mtu(8192)
    sp, cp = C.make_loopback_pair(8192, 512, "pinned")
    app = C.make_app("vec_add", 0, 8192, 8192, [], 64, 1, 4, "gpu", 2)
    srv = C.Server(sp, req_size=8192, resp_size=8192, server_mode=1, max_batch=4)
    srv.add_replica(app)
    srv.start()
    time.sleep(0.05)  # the worker has armed the stream by now
    t0 = time.perf_counter()
    srv.stop()
    assert time.perf_counter() - t0 < 3.0
    # and the same app serves requests afterwards
    srv2 = C.Server(sp, req_size=8192, resp_size=8192, server_mode=1, max_batch=4)
    srv2.add_replica(app)
    srv2.start()
    cli = C.Client(cp, req_size=8192, resp_size=8192, total=40, warmup=0, payload="vec_add", verify=True)
    assert cli.run_closed_loop(8) and cli.received == 40 and cli.verify_failures == 0
    srv2.stop()
