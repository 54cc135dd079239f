"""Model numerics against plain PyTorch fp32 and end-to-end serving of the models."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch

    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch


def test_nn_layers_match_pytorch(torch_cuda):
    torch = torch_cuda
    from splitrpc_b200 import ops

    F = torch.nn.functional
    x = torch.randn(3, 56, 56, 64, device="cuda").bfloat16()
    ref = F.max_pool2d(x.float().permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    assert torch.equal(ops.maxpool3x3s2(x).float(), ref)
    y = torch.randn(4, 7, 7, 2048, device="cuda").bfloat16()
    torch.testing.assert_close(ops.global_avgpool(y).float(), y.float().mean((1, 2)), rtol=1e-2, atol=1e-2)
    x = torch.randn(2, 13, 9, 72, device="cuda").bfloat16()  # odd sizes: clamped windows on every border
    ref = F.max_pool2d(x.float().permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    assert torch.equal(ops.maxpool3x3s2(x).float(), ref)
    y = torch.randn(3, 5, 5, 640, device="cuda").bfloat16()
    torch.testing.assert_close(ops.global_avgpool(y).float(), y.float().mean((1, 2)), rtol=1e-2, atol=1e-2)
    for m_rows, n_cols, k in ((64, 1000, 2048), (5, 10, 512), (130, 77, 256), (70, 100, 1024)):
        a = torch.randn(m_rows, k, device="cuda").bfloat16()
        w = (torch.randn(n_cols, k, device="cuda") * 0.05).bfloat16()
        bias = torch.randn(n_cols, device="cuda")
        torch.testing.assert_close(ops.fc_skinny(a, w, bias=bias), a.float() @ w.float().t() + bias, rtol=1e-3, atol=1e-3)
    h = torch.randn(300, 768, device="cuda").bfloat16()
    r = torch.randn(300, 768, device="cuda").bfloat16()
    g, b = torch.randn(768, device="cuda"), torch.randn(768, device="cuda")
    ln = ops.layernorm(h, g, b, residual=r)
    torch.testing.assert_close(ln.float(), F.layer_norm(h.float() + r.float(), (768,), g, b, 1e-12), rtol=2e-2, atol=2e-2)
    logits = torch.randn(5, 1000, device="cuda")
    out = torch.zeros(5, 1001, device="cuda")
    ops.softmax_response(logits, 5, out=out, resp_stride=1001 * 4, write_argmax=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(out[:, :1000], torch.softmax(logits, -1), rtol=1e-4, atol=1e-6)
    assert torch.equal(out[:, 1000].view(torch.int32), logits.argmax(-1).int())
    img = torch.randn(2, 3, 224, 224, device="cuda")
    col = torch.zeros(2 * 112 * 112, 192, dtype=torch.bfloat16, device="cuda")
    ops.stem_im2col(col, 2, x=img, mean=(0.1, 0.2, 0.3), inv_std=(2.0, 3.0, 4.0))
    m = torch.tensor([0.1, 0.2, 0.3], device="cuda").view(1, 3, 1, 1)
    s = torch.tensor([2.0, 3.0, 4.0], device="cuda").view(1, 3, 1, 1)
    unf = F.unfold((img - m) * s, 7, padding=3, stride=2).transpose(1, 2).reshape(-1, 3, 7, 7)  # [pix, c, ky, kx]
    got = col[:, :168].float().view(-1, 7, 3, 8)  # [pix, ky, c, kx8]
    torch.testing.assert_close(got[..., :7], unf.permute(0, 2, 1, 3).bfloat16().float(), rtol=0, atol=0)
    assert got[..., 7].abs().max() == 0 and col[:, 168:].abs().max() == 0


def test_space_to_depth_stem_matches_conv2d(torch_cuda):
    """stem_s2d + stem_conv (4x1 taps over overlapping 64-channel windows) against an fp32 7x7/2 convolution."""
    torch = torch_cuda
    import torch.nn.functional as F
    from splitrpc_b200 import ops

    nb = 3
    img = torch.randn(nb, 3, 224, 224, device="cuda")
    w = torch.randn(64, 3, 7, 7, device="cuda") * 0.1
    bias = torch.randn(64, device="cuda")
    mean, inv = (0.1, 0.2, 0.3), (2.0, 3.0, 4.0)
    s2d = torch.full((nb, 115, 115, 16), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.stem_s2d(s2d, nb, x=img, mean=mean, inv_std=inv)
    m = torch.tensor(mean, device="cuda").view(1, 3, 1, 1)
    s = torch.tensor(inv, device="cuda").view(1, 3, 1, 1)
    xn = ((img - m) * s).bfloat16().float()
    pad = F.pad(xn, (3, 3, 3, 3))  # [nb, 3, 230, 230]
    want = torch.zeros(nb, 115, 115, 16, device="cuda")
    for dy in range(2):
        for dx in range(2):
            for c in range(3):
                want[..., dy * 8 + dx * 3 + c] = pad[:, c, dy::2, dx::2]
    torch.testing.assert_close(s2d.float(), want, rtol=0, atol=0)
    out = ops.stem_conv(s2d, ops.stem_weight_s2d(w), nb, bias=bias, act="relu")
    ops.check_status()
    ref = F.relu(F.conv2d(xn, w.bfloat16().float(), bias, 2, 3)).permute(0, 2, 3, 1)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=3e-2)


@pytest.mark.parametrize("seq,heads", [(128, 12), (384, 16)])
def test_attention_matches_pytorch(torch_cuda, seq, heads):
    torch = torch_cuda
    from splitrpc_b200 import ops

    B, H = 2, heads * 64
    qkv = (torch.randn(B * seq, 3 * H, device="cuda") * 0.5).bfloat16()
    out = ops.attention_d64(qkv, B, seq, heads)
    q, k, v = (t.float().view(B, seq, heads, 64).transpose(1, 2) for t in qkv.split(H, dim=1))
    ref = (torch.softmax(q @ k.transpose(-1, -2) / 8.0, -1) @ v).transpose(1, 2).reshape(B * seq, H)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("seq,heads", [(128, 12), (384, 16)])
def test_tensor_core_attention_with_v_in_place(torch_cuda, seq, heads):
    """V read in place from the fused Q|K|V buffer (MN-major operand of the second product)."""
    torch = torch_cuda
    from splitrpc_b200 import ops

    B, H = 3, heads * 64
    qkv = (torch.randn(B * seq, 3 * H, device="cuda") * 0.6).bfloat16()
    out = ops.attention_tc_qkv(qkv, B, seq, heads)
    torch.cuda.synchronize()
    ops.check_status()
    q, k, v = (t.float().view(B, seq, heads, 64).transpose(1, 2) for t in qkv.split(H, dim=1))
    ref = (torch.softmax(q @ k.transpose(-1, -2) / 8.0, -1) @ v).transpose(1, 2).reshape(B * seq, H)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("seq,heads", [(128, 12), (384, 16)])
def test_tensor_core_attention_matches_pytorch(torch_cuda, seq, heads):
    torch = torch_cuda
    from splitrpc_b200 import ops

    B, H = 3, heads * 64
    qk = (torch.randn(B * seq, 2 * H, device="cuda") * 0.7).bfloat16()
    v = (torch.randn(B * seq, H, device="cuda") * 0.5).bfloat16()
    vb = torch.randn(H, device="cuda")
    out = ops.attention_tc(qk, v.t().contiguous(), B, seq, heads, v_bias=vb)
    ops.check_status()
    q, k = (t.float().view(B, seq, heads, 64).transpose(1, 2) for t in qk.split(H, dim=1))
    vv = v.float().view(B, seq, heads, 64).transpose(1, 2)
    ref = (torch.softmax(q @ k.transpose(-1, -2) / 8.0, -1) @ vv).transpose(1, 2).reshape(B * seq, H) + vb
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("fuse_shortcut", [True, False])
def test_resnet50_matches_fp32_reference(torch_cuda, fuse_shortcut):
    torch = torch_cuda
    from splitrpc_b200 import ops
    from splitrpc_b200.models import ResNet50

    n = 16
    m = ResNet50(device=0, max_batch=n, fuse_shortcut=fuse_shortcut)
    x = torch.randn(n, 3, 224, 224, device="cuda")
    out = torch.zeros(n, 1000, device="cuda")
    m.forward(n, x=x, out=out)
    ops.check_status()
    # the oracle in true fp32: no TF32 in cuDNN or cuBLAS
    tf32 = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = m.reference_forward(x)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = tf32
    assert torch.isfinite(out).all() and (out.sum(1) - 1.0).abs().max().item() < 1e-3
    # bf16 activations through 53 layers: compare the probability rows as vectors
    cos = torch.nn.functional.cosine_similarity(out, ref, dim=1)
    rel = ((out - ref).norm(dim=1) / ref.norm(dim=1)).max().item()
    agree = (out.argmax(1) == ref.argmax(1)).float().mean().item()
    print(f"resnet50 fuse={fuse_shortcut}: min cos {cos.min().item():.5f}, max rel err {rel:.4f}, argmax agreement {agree:.3f}")
    assert cos.min().item() > 0.999, cos  # measured: 0.99999
    assert rel < 0.05, rel                # measured: 0.006 - 0.007
    assert agree >= 15 / 16, agree        # measured: 16 of 16
    # where the oracle is decisive (its best class leads the runner-up by more than the bf16 noise), the classes agree
    top2 = ref.topk(2, dim=1).values
    decisive = (top2[:, 0] - top2[:, 1]) > 0.1 * top2[:, 0]
    assert bool((out.argmax(1) == ref.argmax(1))[decisive].all())


def test_bert_matches_fp32_reference(torch_cuda):
    torch = torch_cuda
    from splitrpc_b200 import ops
    from splitrpc_b200.models import BertClassifier, BERT_BASE

    m = BertClassifier(BERT_BASE, seq=128, device=0, max_batch=4)
    ids = torch.randint(0, 30522, (3, 128), device="cuda", dtype=torch.int32)
    out = torch.zeros(3, 2, device="cuda")
    m.forward(3, ids=ids, out=out)
    ops.check_status()
    ref = m.reference_forward(ids)
    torch.testing.assert_close(out, ref, rtol=5e-2, atol=3e-2)


def test_fused_gather_deserialise_matches_stem_s2d(torch_cuda):
    """The gather that writes normalised space-to-depth tensors into ring slots against stem_s2d on the raw bytes;
    fragments are given out of order and split at odd (4-byte aligned) places."""
    torch = torch_cuda
    from splitrpc_b200 import _C, ops

    n, req = 3, 3 * 224 * 224 * 4
    slot_bytes = req
    img = torch.randn(n, 3, 224, 224, device="cuda")
    raw = img.view(torch.uint8).reshape(n, req)
    ring = torch.zeros(8 * slot_bytes, dtype=torch.uint8, device="cuda")
    mean, inv = (0.1, 0.2, 0.3), (2.0, 3.0, 4.0)
    items = []
    cuts = [0, 8192, 8192 + 4, 100000, 100000 + 16388, 300004, req]
    for r in range(n):
        slot = 2 + r  # the batch sits in slots 2..4
        for a, b in reversed(list(zip(cuts[:-1], cuts[1:]))):
            items.append((raw[r].data_ptr() + a, ring.data_ptr() + slot * slot_bytes + a, b - a))
    h = _C.sg_list_create(items)
    _C.sg_list_launch_stem_s2d(h, ring.data_ptr(), slot_bytes, list(mean), list(inv), -2, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    _C.sg_list_destroy(h)
    want = torch.zeros(n, 115, 115, 16, dtype=torch.bfloat16, device="cuda")
    ops.stem_s2d(want, n, x=img, mean=mean, inv_std=inv)
    torch.cuda.synchronize()
    got = torch.stack([ring[(2 + r) * slot_bytes:(2 + r) * slot_bytes + 115 * 115 * 32].view(torch.bfloat16).view(115, 115, 16)
                       for r in range(n)])
    assert torch.equal(got, want)
    assert int(ring[:2 * slot_bytes].max()) == 0 and int(ring[5 * slot_bytes:].max()) == 0


@pytest.mark.parametrize("fused_ingress", [True, False])
def test_model_server_end_to_end_resnet(torch_cuda, fused_ingress):
    torch = torch_cuda
    from splitrpc_b200.models import ResNet50
    from splitrpc_b200.serving import ModelServer

    m = ResNet50(device=0, max_batch=8)
    srv = ModelServer(m, device=0, max_batch=8, outstanding=16, fused_ingress=fused_ingress)
    assert srv.fused_ingress == fused_ingress
    with srv:
        cli = srv.client(total=48, warmup=0, payload="normal", verify=True, n_payloads=4)
        assert cli.run_closed_loop(16)
        assert cli.received == 48
        stats = srv.server.stats()
        ws = srv.server.worker_stats(0)
    assert stats["sg_errors"] == 0 and ws["wait_timeouts"] == 0
    x = torch.from_numpy(np.frombuffer(cli.payload(1), dtype=np.float32).copy()).view(1, 3, 224, 224).cuda()
    direct = torch.zeros(1, 1000, device="cuda")
    m.forward(1, x=x, out=direct)
    torch.cuda.synchronize()
    got = torch.from_numpy(np.frombuffer(cli.response(5), dtype=np.float32).copy())  # request 5 used payload 5 % 4 == 1
    torch.testing.assert_close(got, direct[0].cpu(), rtol=1e-3, atol=1e-5)
