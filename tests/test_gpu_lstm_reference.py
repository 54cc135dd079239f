"""The LSTM app against the ORIGINAL's generated model: the original's runtime (compiled unmodified into
baseline/_ref by baseline/build_ref.py) runs its own weights on a request, this package loads the same per-constant
weight files through the default manifest and answers the same request from its GPU app and from its CPU oracle.
Skipped where the original's build is not present."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "baseline", "_ref", "libsplitrpc_ref_lstm.so")
LSTM_DIR = os.path.join(ROOT, "baseline", "_ref", "lstm")
MANIFEST = os.path.join(ROOT, "splitrpc_b200", "data", "nnfusion_lstm.manifest")


def test_lstm_app_matches_the_originals_generated_model(C):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not (os.path.exists(LIB) and os.path.isdir(os.path.join(LSTM_DIR, "Constant"))):
        pytest.skip("the original's LSTM runtime has not been built (python baseline/build_ref.py)")
    lib = ctypes.CDLL(LIB)
    lib.ref_lstm_init.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.ref_lstm_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.ref_lstm_time.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.ref_lstm_time.restype = ctypes.c_float
    assert lib.ref_lstm_init(LSTM_DIR.encode(), 0) == 0
    H, L, T = 256, 8, 8
    w = C.load_lstm_constants(os.path.join(LSTM_DIR, "Constant"), MANIFEST, L, H)
    C.set_rpc_mtu(8192)
    sp, cp = C.make_loopback_pair(8192, 512, "pinned")
    app = C.make_app("lstm", 0, T * H * 4, H * 4, w, 64, 1, 4)
    srv = C.Server(sp, req_size=T * H * 4, resp_size=H * 4, server_mode=2, max_batch=4)
    srv.add_replica(app)
    srv.start()
    cli = C.Client(cp, req_size=T * H * 4, resp_size=H * 4, total=16, warmup=0, payload="uniform", verify=True, n_payloads=4)
    assert cli.run_closed_loop(4) and cli.received == 16
    srv.stop()
    worst = 0.0
    for k in range(4):
        x = np.frombuffer(cli.payload(k), dtype=np.float32).copy()
        ref = np.zeros(H, dtype=np.float32)
        assert lib.ref_lstm_forward(x.ctypes.data, ref.ctypes.data) == 0
        assert np.isfinite(ref).all() and np.abs(ref).max() > 1e-4  # the original produced a real answer
        cpu = C.cpu_lstm(w, x, L, T, H)
        gpu = np.frombuffer(cli.response(k), dtype=np.float32)
        np.testing.assert_allclose(cpu, ref, rtol=2e-3, atol=2e-4)
        np.testing.assert_allclose(gpu, ref, rtol=2e-3, atol=2e-4)
        worst = max(worst, float(np.abs(gpu - ref).max()))
    ms = lib.ref_lstm_time(5, 50)
    ours = {}
    for batch in (1, 4):
        ns, _ = C.local_bench(app, 60, batch)
        ours[batch] = float(np.median(ns[10:])) / 1e3
    st = torch.cuda.ExternalStream(app.work_stream, device=torch.device("cuda", 0))
    dev = {}
    for batch in (1, 4):
        app.queue_runs(batch, 5)
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        app.queue_runs(batch, 50)
        e1.record(st)
        e1.synchronize()
        dev[batch] = e0.elapsed_time(e1) * 1e3 / 50
    print(f"original LSTM runtime: {ms * 1e3:.1f} us per inference (device time, back-to-back launches); this package's app, "
          f"device time, back to back: {dev[1]:.1f} us for 1 request, {dev[4]:.1f} us for 4; launch + sync per batch on the "
          f"host clock: {ours[1]:.1f} us for 1 request, {ours[4]:.1f} us for 4; "
          f"max |difference| between the two models' outputs {worst:.2e}")
    assert ms > 0
