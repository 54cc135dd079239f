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
