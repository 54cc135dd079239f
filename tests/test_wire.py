"""Golden tests of the on-wire format: header offsets, fragmenting, checksum, header swap."""
import struct

import numpy as np

CLIENT_URI = "b8:ce:f6:cc:6a:53,192.168.25.2,50052,b8:ce:f6:cc:6a:52,192.168.25.1,50051"
SERVER_URI = "b8:ce:f6:cc:6a:52,192.168.25.1,50051"


def test_header_is_64_bytes_with_fixed_offsets(C):
    assert C.RPC_HEADER_LEN == 64 and C.UDP_HEADER_LEN == 42 and C.RPC_HEADER_TAIL_LEN == 22
    tmpl = C.client_conn_template(CLIENT_URI)
    frags = C.build_fragments(tmpl, 0x1122334455667788, b"x" * 10, 1024)
    hdr, payload = frags[0]
    assert len(hdr) == 64 and payload == b"x" * 10
    # token @42 (host order), sockperf @50, seq @58
    assert struct.unpack_from("<Q", hdr, 42)[0] == 0x1122334455667788
    assert struct.unpack_from("<H", hdr, 58)[0] == 0
    # ethernet: dst mac first, then src mac, then type 0x0800 big endian
    assert hdr[0:6] == bytes.fromhex("b8cef6cc6a52")
    assert hdr[6:12] == bytes.fromhex("b8cef6cc6a53")
    assert hdr[12:14] == b"\x08\x00"
    # ipv4: version/ihl byte 0x45, ttl 128, proto 17, addresses big endian
    assert hdr[14] == 0x45 and hdr[22] == 128 and hdr[23] == 17
    assert hdr[26:30] == bytes([192, 168, 25, 2]) and hdr[30:34] == bytes([192, 168, 25, 1])
    # udp ports big endian
    assert struct.unpack_from(">HH", hdr, 34) == (50052, 50051)
    # lengths cover the 22-byte RPC tail + payload
    assert struct.unpack_from(">H", hdr, 16)[0] == 20 + 8 + 22 + 10
    assert struct.unpack_from(">H", hdr, 38)[0] == 8 + 22 + 10


def test_fragmenting_rule(C):
    tmpl = C.client_conn_template(CLIENT_URI)
    payload = bytes(np.random.default_rng(1).integers(0, 256, 602112, dtype=np.uint8))
    frags = C.build_fragments(tmpl, 77, payload, 8192)
    assert len(frags) == 74 == C.num_fragments(602112, 8192)
    assert [C.parse_header(h)["seq_num"] for h, _ in frags] == list(range(74))
    assert all(C.parse_header(h)["req_token"] == 77 for h, _ in frags)
    assert all(len(p) == 8192 for _, p in frags[:-1]) and len(frags[-1][1]) == 602112 - 73 * 8192
    assert b"".join(p for _, p in frags) == payload


def test_pseudo_header_checksum_matches_manual_sum(C):
    tmpl = C.client_conn_template(CLIENT_URI)
    hdr, _ = C.build_fragments(tmpl, 5, b"abcd", 1024)[0]
    d = C.parse_header(hdr)
    # one's complement sum over {src ip, dst ip, 0, proto, len} read as little-endian 16-bit words
    l4 = d["ip_tot_len"] - 16
    pseudo = hdr[26:34] + bytes([0, 17]) + struct.pack(">H", l4)
    s = sum(struct.unpack("<6H", pseudo))
    s = (s & 0xFFFF) + (s >> 16)
    s = (s & 0xFFFF) + (s >> 16)
    assert d["udp_check"] == s == C.ipv4_pseudo_csum(hdr)


def test_reply_header_and_swap(C):
    ctmpl = C.client_conn_template(CLIENT_URI)
    stmpl = C.server_conn_template(SERVER_URI)
    req_hdr, _ = C.build_fragments(ctmpl, 99, b"hello", 1024)[0]
    rtmpl = C.reply_template(stmpl, req_hdr)
    rep_hdr, _ = C.build_fragments(rtmpl, 99, b"world!", 1024, True)[0]
    q, r = C.parse_header(req_hdr), C.parse_header(rep_hdr)
    assert (r["dst_mac"], r["dst_ip"], r["dst_port"]) == (q["src_mac"], q["src_ip"], q["src_port"])
    assert (r["src_mac"], r["src_ip"], r["src_port"]) == (q["dst_mac"], q["dst_ip"], q["dst_port"])
    assert r["req_token"] == 99 and (r["sock_perf_header"] & 0xFFFFFFFF) == 0
    sw = C.parse_header(C.swap_header(req_hdr))
    for k in ("mac", "ip", "port"):
        assert sw["src_" + k] == q["dst_" + k] and sw["dst_" + k] == q["src_" + k]


def test_reassembly_out_of_order_duplicates_and_bad_packets(C):
    ctmpl = C.client_conn_template(CLIENT_URI)
    payload = bytes(np.random.default_rng(2).integers(0, 256, 5000, dtype=np.uint8))
    frags = C.build_fragments(ctmpl, 1234, payload, 1024)
    r = C.Reassembler(5000)
    order = [3, 0, 4, 1, 1, 2]  # out of order with one duplicate
    out = None
    for i in order:
        res = r.feed(*frags[i])
        if res is not None:
            out = res
    tok, data, runs = out
    assert tok == 1234 and data == payload
    assert r.counters["dropped_dup"] == 1
    # token 0 and out-of-range sequence numbers are dropped
    z = C.build_fragments(ctmpl, 0, b"zz", 1024)[0]
    assert r.feed(*z) is None and r.counters["dropped_zero_token"] == 1
    bad = bytearray(frags[0][0])
    struct.pack_into("<H", bad, 58, 2000)
    assert r.feed(bytes(bad), frags[0][1]) is None and r.counters["dropped_bad_seq"] == 1
    # a request that lost a fragment is reclaimed by the timeout sweep
    for i in (0, 1, 2):
        r.feed(*C.build_fragments(ctmpl, 555, payload, 1024)[i])
    assert r.partial == 1
    assert r.expire(0) == 1 and r.partial == 0


def test_reassembly_needs_every_sequence_number(C):
    """The byte count alone does not complete a request: sequence numbers must fill 0..n-1 without a hole."""
    ctmpl = C.client_conn_template(CLIENT_URI)
    payload = bytes(np.random.default_rng(3).integers(0, 256, 4096, dtype=np.uint8))
    # one fragment that carries all 4096 bytes but claims sequence number 3: indices 0..2 were never filled
    hdr, body = C.build_fragments(ctmpl, 77, payload, 4096)[0]
    bad = bytearray(hdr)
    struct.pack_into("<H", bad, 58, 3)
    r = C.Reassembler(4096)
    assert r.feed(bytes(bad), body) is None and r.partial == 1
    assert r.expire(0) == 1
    # sequence numbers 0, 2, 3 whose sizes add up to the request size (the middle one is oversized)
    r = C.Reassembler(4096)
    f = C.build_fragments(ctmpl, 78, payload, 1024)

    def with_seq(h, seq):
        b = bytearray(h)
        struct.pack_into("<H", b, 58, seq)
        return bytes(b)

    assert r.feed(f[0][0], payload[:1024]) is None
    assert r.feed(with_seq(f[2][0], 2), payload[1024:3072]) is None
    assert r.feed(with_seq(f[3][0], 3), payload[3072:]) is None  # 4096 bytes are in, index 1 is a hole
    assert r.partial == 1 and r.counters["rx_ready"] == 0
    # an empty fragment of a non-empty request is refused
    assert r.feed(with_seq(f[1][0], 1), b"") is None and r.counters["dropped_dup"] >= 1
    # a well-formed request on the same pool still completes after the malformed ones
    for h, b in C.build_fragments(ctmpl, 79, payload, 1024):
        out = r.feed(h, b)
    assert out is not None and out[1] == payload


def test_copy_list_coalesces_adjacent_fragments(C):
    base = 1 << 20
    frags = [(base, 8192), (base + 8192, 8192), (base + 3 * 8192, 8192), (base + 4 * 8192, 100)]
    g = C.gather_list(frags, 1 << 30)
    assert g == [(base, 1 << 30, 16384), (base + 3 * 8192, (1 << 30) + 16384, 8292)]
    s = C.scatter_list(frags, 1 << 30)
    assert s == [(1 << 30, base, 16384), ((1 << 30) + 16384, base + 3 * 8192, 8292)]


def test_tring_wraps(C):
    t = C.P2pRpcTring(4096, 1000)
    addrs = [t.get_next(300) for _ in range(5)]
    assert addrs == [4096, 4396, 4696, 4996, 4296]


def test_percentile_rule(C):
    v = list(range(1, 102))  # 101 samples
    assert C.percentile(v, 0.5) == 51 and C.percentile(v, 0.99) == 100 and C.percentile(v, 0.999) == 101
    assert C.percentile([], 0.5) == 0.0
    assert abs(C.mean([1, 2, 3, 4]) - 2.5) < 1e-12


def test_multi_tensor_pack_list(C):
    """BERT-SQuAD style request: 4 tensors (8 B + 3 x 2048 B) in 1 KB fragments, packed into per-tensor batch buffers."""
    import ctypes

    sizes = [8, 2048, 2048, 2048]
    req = np.arange(sum(sizes), dtype=np.uint32).astype(np.uint8)  # 6152 bytes with a recognisable pattern
    frag_bufs = [np.ascontiguousarray(req[o:o + 1024]) for o in range(0, len(req), 1024)]
    frags = [(b.ctypes.data, len(b)) for b in frag_bufs]
    batch = 3
    outs = [np.zeros(batch * s, dtype=np.uint8) for s in sizes]
    tensors = [(o.ctypes.data, s) for o, s in zip(outs, sizes)]
    for bi in range(batch):
        lst = C.pack_list(frags, tensors, bi)
        assert len(lst) <= len(frags) + len(sizes)
        for src, dst, ln in lst:
            ctypes.memmove(dst, src, ln)
    off = 0
    for o, s in zip(outs, sizes):
        for bi in range(batch):
            assert np.array_equal(o[bi * s:(bi + 1) * s], req[off:off + s])
        off += s


def test_older_public_types(C):
    """BufItemPool, the first-generation record and pool, UdpRr / UdpRrPool keep the original's names and behaviour."""
    res = C.compat_selftest(-1)
    assert res and all(res.values()), res
