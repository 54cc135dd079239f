"""The allocation-free scatter-gather entry point, called through its exported C symbol.

Some embedders cannot let a library call cudaMalloc on their threads (it stalls
every stream of the device, and they budget GPU memory up front), so the library
offers ``srpc_sg_copy_noalloc``: the copy list lives in a device array built into
the library instead of an allocated buffer.  This checks it against the regular
entry point on two calls in a row (the second reuses and overwrites the built-in
list) and checks that an over-long list is refused.  It is collected last on
purpose: a run that stops at the first failure has then already run every other
test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(lib, items, stream=0):
    n = len(items)
    arr = lambda k: (ctypes.c_uint64 * max(n, 1))(*[it[k] for it in items])
    return lib.srpc_sg_copy_noalloc(arr(0), arr(1), arr(2), ctypes.c_uint32(n), ctypes.c_void_p(stream))


def test_no_alloc_copy_matches_regular_entry_point(C):
    import torch

    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    lib = ctypes.CDLL(C.__file__)
    lib.srpc_sg_copy_noalloc.restype = ctypes.c_int
    lib.srpc_sg_copy_noalloc.argtypes = [ctypes.POINTER(ctypes.c_uint64)] * 3 + [ctypes.c_uint32, ctypes.c_void_p]
    rng = np.random.default_rng(11)
    for call, (n_items, max_len) in enumerate([(37, 50000), (5, 300000)]):
        total = n_items * (max_len + 64)
        src = torch.randint(0, 256, (total,), dtype=torch.uint8, device="cuda")
        ref = torch.zeros(total, dtype=torch.uint8, device="cuda")
        got = torch.zeros(total, dtype=torch.uint8, device="cuda")
        items_ref, items_new, off = [], [], 0
        for _ in range(n_items):
            ln = int(rng.integers(1, max_len + 1))
            so, do = off + int(rng.integers(0, 16)), off + int(rng.integers(0, 16))
            items_ref.append((src.data_ptr() + so, ref.data_ptr() + do, ln))
            items_new.append((src.data_ptr() + so, got.data_ptr() + do, ln))
            off = (max(so, do) + ln + 15) // 16 * 16
        C.sg_copy(items_ref, 0)                 # regular entry point (allocates its device list)
        rc = _call(lib, items_new)              # allocation-free entry point, default stream
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        assert torch.equal(got, ref), f"call {call}: outputs differ"
    # a list longer than the built-in array is refused and nothing runs
    too_many = [(src.data_ptr(), got.data_ptr(), 16)] * 1025
    assert _call(lib, too_many) == -1
    assert _call(lib, []) == 0
    # malformed lists: a zero-length item, null arrays
    assert _call(lib, [(src.data_ptr(), got.data_ptr(), 0)]) == -2
    null = ctypes.POINTER(ctypes.c_uint64)()
    assert lib.srpc_sg_copy_noalloc(null, null, null, ctypes.c_uint32(3), ctypes.c_void_p(0)) == -2
    # exactly the largest list, on a stream of the caller's
    n = 1024
    src2 = torch.randint(0, 256, (n * 48,), dtype=torch.uint8, device="cuda")
    ref2, got2 = torch.zeros_like(src2), torch.zeros_like(src2)
    full_ref = [(src2.data_ptr() + 48 * i, ref2.data_ptr() + 48 * i, 33 + i % 15) for i in range(n)]
    full_new = [(s_, got2.data_ptr() + (d_ - ref2.data_ptr()), l_) for s_, d_, l_ in full_ref]
    C.sg_copy(full_ref[:512], 0)
    C.sg_copy(full_ref[512:], 0)
    user = torch.cuda.Stream()
    user.wait_stream(torch.cuda.current_stream())
    assert _call(lib, full_new, user.cuda_stream) == 0
    user.synchronize()
    torch.cuda.synchronize()
    assert torch.equal(got2, ref2)
    # a stream that is being captured is refused, and the capture stays usable
    cap_stream = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=cap_stream):
        assert _call(lib, full_new[:4], cap_stream.cuda_stream) == -5
        got2.add_(0)
    g.replay()
    torch.cuda.synchronize()
