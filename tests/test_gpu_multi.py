"""Multi-GPU checks (fused tensor-parallel kernels, cross-GPU scatter-gather, single-ingress serving across
processes); skipped with fewer than 2 GPUs.  The world size follows the number of GPUs (largest power of two, at most 8)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def _world():
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    w = 2
    while w * 2 <= min(n, 8):
        w *= 2
    return w


def _torchrun(script, world, port):
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi_gpu", script)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), path]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)


def test_tensor_parallel_and_cross_gpu_paths():
    r = _torchrun("tp_check.py", _world(), 29533)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tensor_parallel_group_of_one():
    """The same checks with a single rank (needs one GPU): every "peer" is the rank itself, the fused kernels run
    without copiers and store their partial tiles into their own slot, the serving front end fans out to itself."""
    import torch

    if torch.cuda.device_count() < 1:
        pytest.skip("needs a GPU")
    r = _torchrun("tp_check.py", 1, 29535)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_single_ingress_serving_across_gpus():
    r = _torchrun("ingress_check.py", _world(), 29534)
    assert r.returncode == 0 and "INGRESS_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
