"""PyTorch-facing wrappers of the hand-written sm_100a kernels.

Each function takes ``torch`` CUDA tensors, checks layout, allocates the output
(or uses ``out=``) and launches the kernel on the current stream through the
native library.  There is no fallback path: calling these without the native
library or without a GPU raises.
"""
from __future__ import annotations

import torch

from .. import _C

ACT = {None: _C.ACT_NONE, "none": _C.ACT_NONE, "relu": _C.ACT_RELU, "gelu": _C.ACT_GELU, "tanh": _C.ACT_TANH}


# 2 = persistent kernels (TMA-store epilogue, TMA tap-shift convolution); 1 = one tile per block, gathered convolution.
GEMM_IMPL = int(__import__("os").environ.get("SPLITRPC_GEMM_IMPL", "2"))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels write an error code into when a bounded wait runs out."""
    dev = torch.cuda.current_device() if device is None else device
    if dev not in _status_words:
        _status_words[dev] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
    return _status_words[dev]


def check_status() -> None:
    """Raises if any kernel launched so far on this device reported a timed-out wait (synchronises)."""
    code = int(status_word().item())
    if code != 0:
        status_word().zero_()
        raise RuntimeError(f"kernel reported error status {code} (a bounded device-side wait ran out)")


def gemm(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         act: str | None = None, out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``act(a @ b.T + bias + residual)`` with a ``[M,K]`` and b ``[N,K]`` bf16 (row-major, K contiguous).

    bias is fp32 ``[N]``; residual is bf16 ``[M,N]``; the result is bf16 or fp32 ``[M,N]``.
    """
    assert a.is_cuda and b.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    assert a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
    _C.gemm_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), M, N, K, out.data_ptr(), out.stride(0),
                 out.dtype == torch.float32, _ptr(bias), _ptr(residual), residual.stride(0) if residual is not None else 0,
                 ACT[act], status_word().data_ptr(), _stream(), GEMM_IMPL)
    return out


def fc_skinny(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a @ w.T + bias`` in fp32 for a handful of rows (``a`` ``[M,K]``, ``w`` ``[N,K]`` bf16): the classifier head of a
    batch, where a 128-row tensor-core tile would leave most SMs without work."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    assert out.dtype == torch.float32 and out.shape == (M, N) and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _C.fc_skinny(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), M, N, K, _stream())
    return out


def conv2d_nhwc(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                stride: int = 1, pad: int = 0, act: str | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Convolution of an NHWC bf16 tensor with ``[Cout, R, S, Cin]`` bf16 filters (Cin a multiple of 64)."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    n, h, wd, cin = x.shape
    cout, r, s, cin2 = w.shape
    assert cin == cin2 and cin % 64 == 0 and cout % 8 == 0
    oh, ow = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - s) // stride + 1
    if out is None:
        out = torch.empty((n, oh, ow, cout), dtype=torch.bfloat16, device=x.device)
    assert out.is_contiguous() and out.shape == (n, oh, ow, cout)
    if residual is not None:
        assert residual.shape == out.shape and residual.is_contiguous() and residual.dtype == torch.bfloat16
    _C.conv_bf16(x.data_ptr(), w.data_ptr(), n, h, wd, cin, cout, r, s, stride, pad, out.data_ptr(), _ptr(bias),
                 _ptr(residual), ACT[act], status_word().data_ptr(), _stream(), GEMM_IMPL)
    return out


def conv1x1_dual(x1: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, stride2: int = 1,
                 act: str | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``act(W1 . x1 + W2 . x2[:, ::stride2, ::stride2] + bias)`` in one kernel: two 1x1 convolutions that share their
    output pixels (a bottleneck's last convolution and its projection shortcut).  ``w`` is ``[Cout, C1 + C2]``."""
    assert x1.is_cuda and x1.dtype == x2.dtype == w.dtype == torch.bfloat16
    assert x1.is_contiguous() and x2.is_contiguous() and w.is_contiguous()
    n, oh, ow, c1 = x1.shape
    n2, h2, w2, c2 = x2.shape
    cout = w.shape[0]
    assert n == n2 and w.numel() == cout * (c1 + c2) and c1 % 64 == 0 and c2 % 64 == 0 and cout % 8 == 0
    assert (h2 - 1) // stride2 + 1 == oh and (w2 - 1) // stride2 + 1 == ow
    if out is None:
        out = torch.empty((n, oh, ow, cout), dtype=torch.bfloat16, device=x1.device)
    assert out.is_contiguous() and out.shape == (n, oh, ow, cout)
    _C.conv_bf16(x1.data_ptr(), w.data_ptr(), n, oh, ow, c1, cout, 1, 1, 1, 0, out.data_ptr(), _ptr(bias), 0, ACT[act],
                 status_word().data_ptr(), _stream(), 2, in2=x2.data_ptr(), h2=h2, w2=w2, cin2=c2, stride2=stride2)
    return out


def sg_copy(items, impl: int = 0, n_blocks: int = 0) -> None:
    """Runs a copy list ``[(src_addr, dst_addr, nbytes)]`` on the current stream and waits for it."""
    _C.sg_copy(list(items), impl, n_blocks, _stream())


IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_INV_STD = (1 / 0.229, 1 / 0.224, 1 / 0.225)


def stem_im2col(out: torch.Tensor, batch: int, x: torch.Tensor | None = None, d_stub: int = 0,
                mean=(0.0, 0.0, 0.0), inv_std=(1.0, 1.0, 1.0)) -> torch.Tensor:
    """im2col of the 7x7/2 stem over fp32 CHW images (given directly or through a device stub), fused with
    normalisation and the bf16 cast.  ``out`` is ``[batch*112*112, 192]`` bf16."""
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() >= batch * 112 * 112 * 192
    if x is not None:
        assert x.dtype == torch.float32 and x.is_contiguous() and x.numel() >= batch * 3 * 224 * 224
    _C.stem_im2col(d_stub, _ptr(x), batch, out.data_ptr(), list(mean), list(inv_std), _stream())
    return out


def stem_s2d(out: torch.Tensor, batch: int, x: torch.Tensor | None = None, d_stub: int = 0,
             mean=(0.0, 0.0, 0.0), inv_std=(1.0, 1.0, 1.0)) -> torch.Tensor:
    """Normalised bf16 space-to-depth form of fp32 CHW 224x224 images: ``out[batch, 115, 115, 16]`` with channel
    ``dy*8 + dx*3 + c`` = pixel ``(2Y+dy-3, 2X+dx-3)`` of channel ``c`` (zero outside the image)."""
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() >= batch * 115 * 115 * 16
    if x is not None:
        assert x.dtype == torch.float32 and x.is_contiguous() and x.numel() >= batch * 3 * 224 * 224
    _C.stem_s2d(d_stub, _ptr(x), batch, out.data_ptr(), list(mean), list(inv_std), _stream())
    return out


def stem_weight_s2d(w: torch.Tensor) -> torch.Tensor:
    """Re-orders ``[64, 3, 7, 7]`` stem filters into the ``[64, 4, 1, 64]`` bf16 filters that ``stem_conv`` expects:
    tap row ``ky' = ky // 2``, channel ``kx'*16 + dy*8 + dx*3 + c`` with ``ky = 2ky'+dy``, ``kx = 2kx'+dx``."""
    cout = w.shape[0]
    w8 = torch.zeros((cout, 3, 8, 8), dtype=torch.float32, device=w.device)
    w8[:, :, :7, :7] = w.float()
    w8 = w8.view(cout, 3, 4, 2, 4, 2)  # [o, c, ky', dy, kx', dx]
    w2 = torch.zeros((cout, 4, 4, 16), dtype=torch.float32, device=w.device)
    for dy in range(2):
        for dx in range(2):
            for c in range(3):
                w2[:, :, :, dy * 8 + dx * 3 + c] = w8[:, c, :, dy, :, dx]
    return w2.view(cout, 4, 1, 64).to(torch.bfloat16).contiguous()


def stem_conv(s2d: torch.Tensor | None, w2: torch.Tensor, batch: int, bias: torch.Tensor | None = None, act: str | None = "relu",
              out: torch.Tensor | None = None, ring: tuple[int, int, int] | None = None, d_stub: int = 0) -> torch.Tensor:
    """The 7x7/2 stem as a 4x1-tap convolution over overlapping 64-channel windows of ``stem_s2d``'s output.

    With ``ring=(base, slots, slot_bytes)`` and ``d_stub`` the space-to-depth tensors are read out of a request ring
    instead (one per slot, written by the fused gather ``sg_list_launch_stem_s2d``); the batch starts at the slot
    that the stub's request pointer names when the kernel runs."""
    cout = w2.shape[0]
    if ring is not None:
        base, slots, slot_bytes = ring
        assert d_stub and slot_bytes % 16 == 0 and slot_bytes >= 115 * 115 * 16 * 2
        assert tuple(w2.shape) == (cout, 4, 1, 64) and w2.dtype == torch.bfloat16 and w2.is_contiguous()
        assert out is not None and out.is_contiguous() and out.numel() >= batch * 112 * 112 * cout
        _C.conv_bf16(base, w2.data_ptr(), batch, 115, 112, 64, cout, 4, 1, 1, 0, out.data_ptr(), _ptr(bias), 0, ACT[act],
                     status_word().data_ptr(), _stream(), 2, 16, 115 * 16, slot_bytes // 2, d_stub, slots, slot_bytes)
        return out
    assert s2d.dtype == torch.bfloat16 and s2d.is_contiguous() and s2d.numel() >= batch * 115 * 115 * 16
    assert tuple(w2.shape) == (cout, 4, 1, 64) and w2.dtype == torch.bfloat16 and w2.is_contiguous()
    if out is None:
        out = torch.empty((batch, 112, 112, cout), dtype=torch.bfloat16, device=s2d.device)
    assert out.is_contiguous() and out.numel() >= batch * 112 * 112 * cout
    _C.conv_bf16(s2d.data_ptr(), w2.data_ptr(), batch, 115, 112, 64, cout, 4, 1, 1, 0, out.data_ptr(), _ptr(bias), 0,
                 ACT[act], status_word().data_ptr(), _stream(), 2, 16, 115 * 16, 115 * 115 * 16)
    return out


def maxpool3x3s2(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    n, h, w, c = x.shape
    oh, ow = (h - 1) // 2 + 1, (w - 1) // 2 + 1
    if out is None:
        out = torch.empty((n, oh, ow, c), dtype=torch.bfloat16, device=x.device)
    _C.maxpool3x3s2(x.data_ptr(), out.data_ptr(), n, h, w, c, _stream())
    return out


def global_avgpool(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    n, h, w, c = x.shape
    if out is None:
        out = torch.empty((n, c), dtype=torch.bfloat16, device=x.device)
    _C.global_avgpool(x.data_ptr(), out.data_ptr(), n, h * w, c, _stream())
    return out


def softmax_response(logits: torch.Tensor, rows: int, out: torch.Tensor | None = None, d_stub: int = 0,
                     resp_stride: int | None = None, write_argmax: bool = False, counter: torch.Tensor | None = None,
                     flag_ptr: int = 0, flag_value: int = 0, d_push: int = 0) -> None:
    """Row softmax of fp32 logits written as fp32 into response slots (``out`` or the stub's response window).

    ``d_push``: device address of the app's response-push block (``App.d_push``).  When the server has enabled
    completion by the serving side, every row is stored where the ingress asked for it (its transmit arena) and the
    row's slot is marked complete by this kernel; otherwise the block is inert and the row goes to the response ring."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    n = logits.shape[1]
    if resp_stride is None:
        resp_stride = (n + (1 if write_argmax else 0)) * 4
    _C.softmax_response(logits.data_ptr(), rows, n, logits.stride(0), d_stub, _ptr(out), resp_stride, write_argmax,
                        _ptr(counter), flag_ptr, flag_value, _stream(), d_push)


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, residual: torch.Tensor | None = None,
              out: torch.Tensor | None = None, eps: float = 1e-12) -> torch.Tensor:
    """``LN(x + residual) * gamma + beta`` over the last dimension (bf16 in/out, fp32 parameters)."""
    rows, hidden = x.shape
    if out is None:
        out = torch.empty_like(x)
    _C.layernorm(x.data_ptr(), _ptr(residual), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), rows, hidden, eps, _stream())
    return out


def bert_embed_ln(out: torch.Tensor, batch: int, seq: int, word: torch.Tensor, pos: torch.Tensor, typ: torch.Tensor,
                  gamma: torch.Tensor, beta: torch.Tensor, ids: torch.Tensor | None = None, d_stub: int = 0,
                  req_stride: int | None = None, eps: float = 1e-12) -> torch.Tensor:
    """Embedding gather (word + position + type 0) + LayerNorm, reading int32 ids directly or through a stub."""
    vocab, hidden = word.shape
    if req_stride is None:
        req_stride = seq * 4
    _C.bert_embed_ln(d_stub, _ptr(ids), req_stride, batch, seq, word.data_ptr(), pos.data_ptr(), typ.data_ptr(),
                     gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), hidden, vocab, eps, _stream())
    return out


def attention_d64(qkv: torch.Tensor, batch: int, seq: int, heads: int, out: torch.Tensor | None = None,
                  offsets: tuple[int, int, int] | None = None) -> torch.Tensor:
    """Multi-head attention with head dim 64 over ``qkv = [tokens, q|k|v]`` (all-ones mask)."""
    hidden = heads * 64
    if offsets is None:
        offsets = (0, hidden, 2 * hidden)
    if out is None:
        out = torch.empty((batch * seq, hidden), dtype=torch.bfloat16, device=qkv.device)
    _C.attention_d64(qkv.data_ptr(), out.data_ptr(), batch, seq, heads, qkv.stride(0), offsets[0], offsets[1], offsets[2],
                     out.stride(0), _stream())
    return out


def attention_tc_qkv(qkv: torch.Tensor, batch: int, seq: int, heads: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core attention (head dim 64, all-ones mask) straight from the fused projection ``[tokens, 3*hidden]``
    (Q | K | V, biases included): V is used in place as an MN-major operand, no transposed copy.  Returns
    ``[tokens, hidden]`` bf16."""
    hidden = heads * 64
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape == (batch * seq, 3 * hidden)
    if out is None:
        out = torch.empty((batch * seq, hidden), dtype=torch.bfloat16, device=qkv.device)
    _C.attention_tc(qkv.data_ptr(), qkv.stride(0), 0, 0, out.data_ptr(), out.stride(0), 0, batch, seq, heads,
                    status_word().data_ptr(), _stream())
    return out


def attention_tc(qk: torch.Tensor, vt: torch.Tensor, batch: int, seq: int, heads: int, v_bias: torch.Tensor | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core attention (head dim 64, all-ones mask).

    ``qk`` is ``[tokens, 2*hidden]`` (Q | K), ``vt`` is ``[hidden, tokens]`` (V transposed, without its bias);
    ``v_bias`` (fp32 ``[hidden]``) is added to the output.  Returns ``[tokens, hidden]`` bf16.
    """
    hidden = heads * 64
    assert qk.dtype == torch.bfloat16 and vt.dtype == torch.bfloat16 and qk.stride(1) == 1 and vt.stride(1) == 1
    assert qk.shape == (batch * seq, 2 * hidden) and vt.shape == (hidden, batch * seq)
    if out is None:
        out = torch.empty((batch * seq, hidden), dtype=torch.bfloat16, device=qk.device)
    _C.attention_tc(qk.data_ptr(), qk.stride(0), vt.data_ptr(), vt.stride(0), out.data_ptr(), out.stride(0), _ptr(v_bias),
                    batch, seq, heads, status_word().data_ptr(), _stream())
    return out
