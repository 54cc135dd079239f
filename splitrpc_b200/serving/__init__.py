"""Serving layer: wires transports, apps and the native server together from Python."""
from __future__ import annotations

import numpy as np

from .. import _C
from .engine import ModelReplica, ModelServer  # noqa: F401


def __getattr__(name):
    if name == "TensorParallelServer":  # needs torch.distributed; imported on first use
        from .tp_server import TensorParallelServer

        return TensorParallelServer
    raise AttributeError(name)


def lenet5_random_weights(seed: int = 0) -> list[np.ndarray]:
    """Random-init LeNet-5 parameters in the order the native apps expect."""
    rng = np.random.default_rng(seed)
    shapes = [(6, 1, 5, 5), (6,), (16, 6, 5, 5), (16,), (120, 400), (120,), (84, 120), (84,), (10, 84), (10,)]
    return [(rng.standard_normal(s) * 0.1).astype(np.float32) for s in shapes]


def smoke_test(device: int = 0) -> dict:
    """Serves a few LeNet-5 requests end to end on ``device`` through the loopback transport and
    checks them against the CPU oracle; then runs one tensor-core GEMM."""
    import torch

    if not _C.cuda_available():
        raise RuntimeError("smoke test needs a CUDA device")
    _C.set_rpc_mtu(8192)
    w = lenet5_random_weights()
    sp, cp = _C.make_loopback_pair(8192, 256, "pinned")
    app = _C.make_app("lenet5", device, 3136, 40, w, 128, 1, 8, "gpu", 2)
    srv = _C.Server(sp, req_size=3136, resp_size=40, server_mode=2, max_batch=8)
    srv.add_replica(app)
    srv.start()
    cli = _C.Client(cp, req_size=3136, resp_size=40, total=64, warmup=0, payload="uniform", verify=True)
    ok = cli.run_closed_loop(8)
    srv.stop()
    if not ok or cli.received != 64:
        raise RuntimeError(f"smoke: served {cli.received}/64 requests")
    x = np.frombuffer(cli.payload(5), dtype=np.float32)
    ref = _C.cpu_lenet5(w, x)[0]
    got = np.frombuffer(cli.response(5), dtype=np.float32)
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)

    from .. import ops

    torch.cuda.set_device(device)
    a = torch.randn(256, 256, device="cuda").bfloat16()
    b = torch.randn(256, 256, device="cuda").bfloat16()
    out = ops.gemm(a, b)
    ops.check_status()
    err = ((out.float() - a.float() @ b.float().t()).norm() / (a.float() @ b.float().t()).norm()).item()
    if err > 1e-2:
        raise RuntimeError(f"smoke: gemm relative error {err}")
    # one small forward of the flagship model (ResNet-50, batch 2) through the same kernels the server's graph replays
    from ..models import ResNet50

    model = ResNet50(device=device, max_batch=2)
    x = torch.randn(2, 3, 224, 224, device="cuda")
    probs = torch.empty(2, 1000, device="cuda")
    model.forward(2, x=x, out=probs)
    torch.cuda.synchronize()
    ops.check_status()
    ref = model.reference_forward(x)
    if not torch.allclose(probs.sum(-1), torch.ones(2, device="cuda"), atol=1e-3) or not torch.equal(probs.argmax(-1), ref.argmax(-1)):
        raise RuntimeError("smoke: ResNet-50 forward disagrees with the PyTorch evaluation of the same weights")
    return {"served": int(cli.received), "gemm_rel_err": err, "resnet50_top1_match": True}
