"""Tensor-parallel fused kernels with the ranks emulated on one GPU.

Each "rank" is a set of buffers on the same device and its kernel is launched on its own, after every flag it waits
for has been set (by the host or by an earlier launch), so no launch ever waits on a later one.  This checks the data
paths of the copier blocks, the per-row-block flags, the rotated tile order and the peer-store epilogue; the real
multi-GPU run is tests/test_gpu_multi.py.
"""
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    torch.manual_seed(3)
    from splitrpc_b200 import _C, ops

    return torch, _C, ops


# Rows per rank that are a multiple of 256 run on CTA pairs (256-row tiles, 128 / 192 / 256 columns wide), the others
# on the one-SM kernel.
@pytest.mark.parametrize("T,K,N,tp", [(512, 256, 384, 2), (1024, 1024, 512, 4), (2048, 512, 2048, 2), (768, 256, 384, 2),
                                      (6144, 1024, 1536, 2), (6144, 1024, 512, 8), (2048, 512, 640, 4)])
def test_all_gather_gemm_emulated_ranks(env, T, K, N, tp):
    torch, C, ops = env
    rows = T // tp
    x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
    shards = [x[r * rows:(r + 1) * rows].contiguous() for r in range(tp)]
    status = ops.status_word()
    for r in range(tp):
        w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
        bias = torch.randn(N, device="cuda")
        gathered = torch.zeros(T, K, dtype=torch.bfloat16, device="cuda")
        gathered[r * rows:(r + 1) * rows] = shards[r]
        out = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
        ready = torch.full((8,), 5, dtype=torch.int32, device="cuda")       # every peer has published step 5
        mblock = torch.zeros(T // 128, dtype=torch.int32, device="cuda")
        C.gemm_tp(gathered.data_ptr(), K, w.data_ptr(), K, T, N, K, out.data_ptr(), N, bias.data_ptr(), ops.ACT["gelu"], tp, r, 5,
                  mblock.data_ptr(), 6, [s.data_ptr() for s in shards], gathered.data_ptr(), ready.data_ptr(), 0, [], [], 0,
                  status.data_ptr(), torch.cuda.current_stream().cuda_stream, 0)
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(gathered, x)
        ref = torch.nn.functional.gelu(x.float() @ w.float().t() + bias)
        assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
        remote = [m for m in range(T // 128) if m // (rows // 128) != r]
        assert all(int(mblock[m]) == 5 for m in remote)


@pytest.mark.parametrize("T,Kl,N,tp", [(512, 256, 384, 2), (1024, 512, 1024, 4), (2048, 2048, 1024, 2), (768, 256, 384, 2),
                                       (6144, 512, 1024, 2), (6144, 128, 1024, 8), (2048, 256, 640, 4)])
def test_gemm_reduce_scatter_emulated_ranks(env, T, Kl, N, tp):
    torch, C, ops = env
    rows = T // tp
    status = ops.status_word()
    slots = torch.zeros(tp, tp, rows, N, dtype=torch.bfloat16, device="cuda")   # [owner][source]
    flags = torch.zeros(tp, 8, dtype=torch.int32, device="cuda")                # [owner][source]
    total = torch.zeros(T, N, device="cuda")
    for r in range(tp):
        a = (torch.randn(T, Kl, device="cuda") * 0.3).bfloat16()
        w = (torch.randn(N, Kl, device="cuda") * 0.1).bfloat16()
        total += (a.float() @ w.float().t()).bfloat16().float()
        count = torch.zeros(8, dtype=torch.int32, device="cuda")
        dst = [slots[o, r].data_ptr() for o in range(tp)]
        dflag = [flags[o, r:].data_ptr() for o in range(tp)]
        C.gemm_tp(a.data_ptr(), Kl, w.data_ptr(), Kl, T, N, Kl, slots[r].data_ptr(), N, 0, 0, tp, r, 9, 0, 0, [], 0, 0, 1, dst,
                  dflag, count.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream, 0)
        torch.cuda.synchronize()
        ops.check_status()
        assert int(count.abs().sum()) == 0          # the last tile of every owner reset its counter
    assert bool((flags[:, :tp] == 9).all())
    got = slots.float().sum(1).reshape(T, N)
    assert ((got - total).norm() / total.norm()).item() < 1e-2


@pytest.mark.parametrize("rows,hidden,tp", [(3072, 1024, 2), (768, 1024, 8), (384, 320, 2)])
def test_reduce_layernorm_emulated_ranks(env, rows, hidden, tp):
    """Sum of the source ranks' partial rows + bias + residual, then LayerNorm, with the flags of every source already
    published; the kernel's last block publishes the step number to the peers' words."""
    torch, C, ops = env
    status = ops.status_word()
    slots = (torch.randn(tp, rows, hidden, device="cuda") * 0.5).bfloat16()
    residual = torch.randn(rows, hidden, device="cuda").bfloat16()
    bias, gamma, beta = torch.randn(hidden, device="cuda"), torch.rand(hidden, device="cuda") + 0.5, torch.randn(hidden, device="cuda")
    flags = torch.full((8,), 3, dtype=torch.int32, device="cuda")
    out = torch.zeros(rows, hidden, dtype=torch.bfloat16, device="cuda")
    peer_words = torch.zeros(tp, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.layernorm_reduce([slots[r].data_ptr() for r in range(tp)], flags.data_ptr(), 3, bias.data_ptr(), residual.data_ptr(),
                       gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), rows, hidden, 1e-12, status.data_ptr(),
                       torch.cuda.current_stream().cuda_stream, 0, [peer_words[p:].data_ptr() for p in range(tp)], 7, done.data_ptr())
    torch.cuda.synchronize()
    ops.check_status()
    z = slots.float().sum(0) + bias + residual.float()
    ref = torch.nn.functional.layer_norm(z, (hidden,), gamma, beta, 1e-12)
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
    assert bool((peer_words == 7).all()) and int(done) == 0
