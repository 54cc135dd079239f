"""The reference-format LeNet app against the ORIGINAL LeNet: the original's code (compiled unmodified into
baseline/_ref by baseline/build_ref.py) reads weights in its own .dat format and classifies images, this package loads
the same files and answers the same images from its one-kernel GPU app and from its CPU oracle.  Skipped where the
original's build is not present."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "baseline", "_ref", "libsplitrpc_ref_lenet.so")


def test_lenet_app_matches_the_original(C, tmp_path):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.exists(LIB):
        pytest.skip("the original's LeNet has not been built (python baseline/build_ref.py)")
    rng = np.random.default_rng(11)
    shapes = {"data2.dat": (20, 1, 5, 5), "data0.dat": (50, 20, 5, 5), "data1.dat": (10, 1250), "data3.dat": (10,)}
    d = tmp_path / "data" / "lenet"
    d.mkdir(parents=True)
    for name, shape in shapes.items():
        (rng.standard_normal(shape) * (0.2 if len(shape) > 1 else 0.1)).astype(np.float32).tofile(d / name)
    lib = ctypes.CDLL(LIB)
    lib.ref_lenet_init.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.ref_lenet_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.ref_lenet_time.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.ref_lenet_time.restype = ctypes.c_float
    assert lib.ref_lenet_init(str(tmp_path).encode(), 0) == 0
    w = C.load_lenet_ref_weights(str(tmp_path))
    C.set_rpc_mtu(8192)
    sp, cp = C.make_loopback_pair(8192, 512, "pinned")
    app = C.make_app("lenet_ref", 0, 784, 40, w, 64, 1, 4)
    srv = C.Server(sp, req_size=784, resp_size=40, server_mode=2, max_batch=4)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=784, resp_size=40, total=32, warmup=0, payload="echo", verify=True, n_payloads=8)
    assert cli.run_closed_loop(4) and cli.received == 32
    srv.stop()
    worst = 0.0
    for k in range(8):
        img = np.frombuffer(cli.payload(k), dtype=np.uint8).copy()
        ref = np.zeros(10, dtype=np.float32)
        assert lib.ref_lenet_forward(img.ctypes.data, ref.ctypes.data) == 0
        assert np.isfinite(ref).all() and abs(float(ref.sum()) - 1.0) < 1e-3  # the original produced probabilities
        gpu = np.frombuffer(cli.response(k), dtype=np.float32)
        np.testing.assert_allclose(gpu, ref, rtol=2e-3, atol=2e-5)
        worst = max(worst, float(np.abs(gpu - ref).max()))
    ms = lib.ref_lenet_time(5, 100)
    ns, _ = C.local_bench(app, 60, 1)
    ns4, _ = C.local_bench(app, 60, 4)

    def device_us(batch, n=100):
        st = torch.cuda.ExternalStream(app.work_stream, device=torch.device("cuda", 0))
        app.queue_runs(batch, 5)
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        app.queue_runs(batch, n)
        e1.record(st)
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    d1, d4, d32 = device_us(1), device_us(4), device_us(32)
    print(f"original LeNet: {ms * 1e3:.1f} us per inference (12 launches, device time, back to back); this package's app, "
          f"device time, back to back: {d1:.1f} us for 1 request, {d4:.1f} us for 4, {d32:.1f} us for 32; launch + sync on the "
          f"host clock: {float(np.median(ns[10:])) / 1e3:.1f} us for 1 request, {float(np.median(ns4[10:])) / 1e3:.1f} us for 4; "
          f"max |difference| {worst:.2e}")
    assert ms > 0
