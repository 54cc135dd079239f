"""Property tests (hypothesis) of the host core: reassembly under arbitrary interleavings of the fragments of several
requests with duplicates, the copy-list builder against a byte-level model, and the comparison system's wire codec."""
import struct

import numpy as np
import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, Phase, given, settings
from hypothesis import strategies as st

CLIENT_URI = "b8:ce:f6:cc:6a:53,192.168.25.2,50052,b8:ce:f6:cc:6a:52,192.168.25.1,50051"
COMMON = dict(deadline=None, derandomize=True, database=None,
              suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])  # the same examples on every run


@settings(max_examples=60, **COMMON)
@given(size=st.integers(1, 9000), mtu=st.sampled_from([256, 1024, 4096]), n_req=st.integers(1, 4), dup=st.integers(0, 6),
       seed=st.integers(0, 2**32 - 1))
def test_reassembly_under_any_interleaving(C, size, mtu, n_req, dup, seed):
    """Whatever the arrival order of the fragments of several requests, with duplicates thrown in: every request
    completes with its own bytes (a second time only when every one of its fragments arrived again after the first
    completion, which the protocol cannot tell from a retransmission), and nothing stays partial after the sweep."""
    rng = np.random.default_rng(seed)
    ctmpl = C.client_conn_template(CLIENT_URI)
    payloads = {1000 + k: bytes(rng.integers(0, 256, size, dtype=np.uint8)) for k in range(n_req)}
    stream = []
    for tok, p in payloads.items():
        stream += [(tok, h, b) for h, b in C.build_fragments(ctmpl, tok, p, mtu)]
    n_frag = len(stream) // n_req
    assert n_frag == -(-size // mtu)
    extra = [stream[i] for i in rng.integers(0, len(stream), dup)]
    order = rng.permutation(len(stream) + len(extra))
    allp = stream + extra
    r = C.Reassembler(size)
    done = {}
    for i in order:
        tok, h, b = allp[i]
        out = r.feed(h, b)
        if out is not None:
            assert out[1] == payloads[out[0]]
            done[out[0]] = done.get(out[0], 0) + 1
    # a duplicate that arrives after its request completed starts a new partial record: sweep those
    r.expire(0)
    assert set(done) == set(payloads)
    assert r.partial == 0 and r.counters["rx_ready"] == sum(done.values())
    if n_frag > 1 and dup < n_frag:
        assert all(v == 1 for v in done.values())  # too few duplicates to rebuild a whole request


@settings(max_examples=80, **COMMON)
@given(lens=st.lists(st.integers(1, 8192), min_size=1, max_size=40), gaps=st.lists(st.integers(0, 3), min_size=40, max_size=40))
def test_copy_list_equals_byte_model(C, lens, gaps):
    """The gather list (adjacent source fragments merged) moves exactly the bytes that copying fragment by fragment would."""
    base, dst = 1 << 20, 1 << 30
    frags, at = [], base
    for ln, g in zip(lens, gaps):
        at += g * 64  # 0: adjacent to the previous fragment
        frags.append((at, ln))
        at += ln
    items = C.gather_list(frags, dst)
    assert sum(n for _, _, n in items) == sum(lens) and len(items) <= len(frags)
    # byte-level model: destination offset -> source address
    want = {}
    off = 0
    for a, ln in frags:
        for k in range(0, ln, 997):  # sample
            want[off + k] = a + k
        off += ln
    got_runs = sorted((d - dst, s, n) for s, d, n in items)
    pos = 0
    for d0, s0, n in got_runs:
        assert d0 == pos  # destination runs tile [0, total) without gaps
        pos += n
    for doff, src in want.items():
        run = next(r for r in got_runs if r[0] <= doff < r[0] + r[2])
        assert run[1] + (doff - run[0]) == src


@settings(max_examples=200, **COMMON)
@given(guid=st.integers(0, 2**64 - 1), funcid=st.integers(0, 2**32 - 1), payload=st.binary(max_size=3000),
       junk=st.binary(max_size=12))
def test_grpc_wire_codec_roundtrip_and_robustness(guid, funcid, payload, junk):
    from splitrpc_b200.utils.grpc_baseline import decode_message, encode_message

    enc = encode_message(guid, funcid, payload)
    assert decode_message(enc) == (guid, funcid, payload, len(payload))
    # arbitrary trailing bytes either decode (unknown fields) or raise ValueError, never anything else
    try:
        g, f, p, s = decode_message(enc + junk)
        assert isinstance(p, bytes)
    except ValueError:
        pass
    # every strict prefix that cuts the payload field is refused or decodes to a shorter, well-formed message
    if payload:
        cut = enc[: len(enc) - 1 - len(struct.pack("<B", 0))]
        try:
            decode_message(cut)
        except ValueError:
            pass


@settings(max_examples=12, phases=[Phase.explicit, Phase.generate], **COMMON)  # a server per example: no shrinking
@given(req=st.integers(1, 20000), resp=st.integers(1, 6000), mode=st.sampled_from([0, 1, 2]), batch=st.sampled_from([1, 3, 8]),
       outstanding=st.integers(1, 12), dupl=st.sampled_from([0.0, 0.1]), reorder=st.sampled_from([0.0, 0.3]), lanes=st.sampled_from([1, 3]),
       seed=st.integers(1, 1000))
def test_echo_server_any_sizes_modes_and_wire_faults(C, req, resp, mode, batch, outstanding, dupl, reorder, lanes, seed):
    """Every worker mode, any request / response size (responses are the first bytes of the request), duplicates and
    reordering on the wire, one or several DMA lanes: every call is answered once and correctly."""
    if mode != 2 and batch > 1:
        # a fixed batch size waits for full batches: no extra (duplicated) requests, enough calls in flight to fill one,
        # and a total that is a whole number of batches (48 = 16 x 3 = 6 x 8)
        dupl = 0.0
        outstanding = max(outstanding, batch)
    old = 8192
    C.set_rpc_mtu(1024)
    try:
        sp, cp = C.make_loopback_pair(1024, 4096)
        if lanes > 1:
            C.set_loopback_dma_lanes(cp, lanes)
        if dupl or reorder:
            C.set_loopback_faults(cp, duplicate=dupl, reorder=reorder, seed=seed)
        app = C.make_app("echo", -1, req, resp, [], 64, 1, batch if mode != 1 else 1)
        srv = C.Server(sp, req_size=req, resp_size=resp, server_mode=mode, max_batch=batch if mode != 1 else 1,
                       reassembly_timeout_ns=50_000_000)
        srv.add_replica(app)
        srv.start()
        total = 48
        cli = C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=0, payload="echo", verify=False,
                       drain_timeout_ns=20_000_000_000)
        ok = cli.run_closed_loop(outstanding)
        st_ = srv.stats()
        srv.stop()
        assert ok and cli.received == total
        # a duplicated datagram that is a whole request by itself is served twice; the client drops the second reply
        assert cli.bad_tokens == 0 or dupl > 0
        assert st_["tx_resps"] >= total
    finally:
        C.set_rpc_mtu(old)
