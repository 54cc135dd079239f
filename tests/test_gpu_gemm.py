"""Numerics of the tcgen05 GEMM and implicit-GEMM convolution against plain PyTorch fp32."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    from splitrpc_b200 import ops

    return torch, ops


def _rel_err(torch, got, ref):
    return ((got.float() - ref).norm() / ref.norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 512), (256, 384, 1024), (8192, 768, 768),
                                   (100, 200, 72), (4096, 3072, 768), (64, 10, 2048), (3136, 64, 64)])
def test_gemm_plain(env, M, N, K):
    torch, ops = env
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    out = ops.gemm(a, b)
    ops.check_status()
    ref = a.float() @ b.float().t()
    assert _rel_err(torch, out, ref) < 1e-2


@pytest.mark.parametrize("act", [None, "relu", "gelu"])
def test_gemm_epilogue(env, act):
    torch, ops = env
    M, N, K = 512, 320, 256
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    out = ops.gemm(a, b, bias=bias, residual=res, act=act)
    ops.check_status()
    ref = a.float() @ b.float().t() + bias + res.float()
    if act == "relu":
        ref = torch.relu(ref)
    elif act == "gelu":
        ref = torch.nn.functional.gelu(ref)
    assert _rel_err(torch, out, ref) < 1e-2
    out32 = ops.gemm(a, b, bias=bias, out_dtype=torch.float32)
    ref32 = a.float() @ b.float().t() + bias
    assert _rel_err(torch, out32, ref32) < 2e-3


@pytest.mark.parametrize("M,N,K", [(4096, 768, 3072), (4096, 1536, 768), (1000, 576, 1024)])
def test_gemm_wide_tiles_with_epilogue(env, M, N, K):
    """Shapes that select the 192-column tile (N a multiple of 192); long K keeps the residual on plain loads."""
    torch, ops = env
    a = (torch.randn(M, K, device="cuda") * 0.2).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.2).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    out = ops.gemm(a, b, bias=bias, residual=res, act="gelu")
    ops.check_status()
    ref = torch.nn.functional.gelu(a.float() @ b.float().t() + bias + res.float())
    assert _rel_err(torch, out, ref) < 1e-2


def test_gelu_epilogue_matches_erf_definition(env):
    """The epilogue's rational erfc approximation against torch's exact GELU over a wide range of inputs."""
    torch, ops = env
    x = torch.linspace(-8, 8, 128 * 256, device="cuda").view(128, 256)
    eye = torch.eye(256, device="cuda").bfloat16()
    out = ops.gemm(x.bfloat16(), eye, act="gelu", out_dtype=torch.float32)
    ops.check_status()
    ref = torch.nn.functional.gelu(x.bfloat16().float())
    assert (out - ref).abs().max().item() < 2e-6


@pytest.mark.parametrize("n,oh,c1,h2,c2,cout,stride2", [(2, 56, 64, 56, 64, 256, 1), (3, 28, 128, 56, 256, 512, 2),
                                                        (2, 14, 256, 28, 512, 1024, 2), (5, 7, 512, 14, 1024, 2048, 2)])
def test_two_input_pointwise_conv(env, n, oh, c1, h2, c2, cout, stride2):
    """Last bottleneck convolution + projection shortcut as one kernel vs the two convolutions in fp32."""
    torch, ops = env
    x1 = (torch.randn(n, oh, oh, c1, device="cuda") * 0.5).bfloat16()
    x2 = (torch.randn(n, h2, h2, c2, device="cuda") * 0.5).bfloat16()
    w1 = (torch.randn(cout, c1, device="cuda") * 0.1).bfloat16()
    w2 = (torch.randn(cout, c2, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(cout, device="cuda")
    out = ops.conv1x1_dual(x1, x2, torch.cat([w1, w2], dim=1).contiguous(), bias=bias, stride2=stride2, act="relu")
    ops.check_status()
    ref = x1.float() @ w1.float().t() + x2[:, ::stride2, ::stride2].float() @ w2.float().t() + bias
    assert out.shape == ref.shape
    assert _rel_err(torch, out, torch.relu(ref)) < 1e-2


@pytest.mark.parametrize("n,h,cin,cout,r,stride,pad", [(2, 56, 64, 64, 3, 1, 1), (4, 28, 128, 128, 3, 1, 1),
                                                       (2, 56, 256, 128, 1, 2, 0), (3, 14, 256, 256, 3, 1, 1),
                                                       (2, 7, 512, 512, 3, 1, 1), (2, 56, 64, 256, 1, 1, 0),
                                                       (2, 28, 128, 128, 3, 2, 1)])
def test_conv_implicit_gemm(env, n, h, cin, cout, r, stride, pad):
    torch, ops = env
    x = (torch.randn(n, h, h, cin, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(cout, r, r, cin, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(cout, device="cuda")
    out = ops.conv2d_nhwc(x, w, bias=bias, stride=stride, pad=pad, act="relu")
    ops.check_status()
    ref = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float().permute(0, 3, 1, 2), bias, stride, pad)
    ref = torch.relu(ref).permute(0, 2, 3, 1)
    assert out.shape == ref.shape
    assert _rel_err(torch, out, ref) < 1e-2
    res = torch.randn_like(out)
    out2 = ops.conv2d_nhwc(x, w, bias=bias, residual=res, stride=stride, pad=pad, act="relu")
    ref2 = torch.relu(torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float().permute(0, 3, 1, 2), bias, stride,
                                                 pad).permute(0, 2, 3, 1) + res.float())
    assert _rel_err(torch, out2, ref2) < 1e-2
