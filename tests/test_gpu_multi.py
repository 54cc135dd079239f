"""Multi-GPU checks (fused tensor-parallel kernels, cross-GPU scatter-gather); skipped with fewer than 2 GPUs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_tensor_parallel_and_cross_gpu_paths():
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi_gpu", "tp_check.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29533", script]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
