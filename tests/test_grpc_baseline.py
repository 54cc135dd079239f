"""The comparison system (gRPC front end + copy path, reference src/grpc_bench): wire format against the protobuf
runtime, and the per-request and batched servers around CPU apps over 127.0.0.1."""
import numpy as np
import pytest

grpc = pytest.importorskip("grpc")

from splitrpc_b200.utils.grpc_baseline import GrpcClient, GrpcCopyPathServer, decode_message, encode_message


def _proto_class():
    """ScheduleRequest of the original's infer.proto, built at run time from a descriptor."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

    f = descriptor_pb2.FileDescriptorProto(name="infer_test.proto", package="doinference_test", syntax="proto3")
    m = f.message_type.add(name="ScheduleRequest")
    T = descriptor_pb2.FieldDescriptorProto
    for name, num, typ in (("guid", 1, T.TYPE_UINT64), ("funcid", 2, T.TYPE_UINT32), ("payload", 3, T.TYPE_BYTES),
                           ("size", 4, T.TYPE_UINT32)):
        m.field.add(name=name, number=num, type=typ, label=T.LABEL_OPTIONAL)
    pool = descriptor_pool.DescriptorPool()
    pool.Add(f)
    return message_factory.GetMessageClass(pool.FindMessageTypeByName("doinference_test.ScheduleRequest"))


def test_wire_format_matches_protobuf():
    cls = _proto_class()
    rng = np.random.default_rng(3)
    for guid, funcid, n in ((1, 1, 0), (0, 0, 5), (2**40 + 7, 9, 784), (2**64 - 1, 2**32 - 1, 70000)):
        payload = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        ours = encode_message(guid, funcid, payload)
        theirs = cls(guid=guid, funcid=funcid, payload=payload, size=n)
        assert ours == theirs.SerializeToString()
        back = cls.FromString(ours)
        assert (back.guid, back.funcid, back.payload, back.size) == (guid, funcid, payload, n)
        assert decode_message(theirs.SerializeToString()) == (guid, funcid, payload, n)
    # unknown fields are skipped, truncation is an error
    assert decode_message(encode_message(5, 6, b"abc") + b"\x28\x01" + b"\x32\x02hi") == (5, 6, b"abc", 3)
    with pytest.raises(ValueError):
        decode_message(encode_message(5, 6, b"abcdef")[:-4])


@pytest.mark.parametrize("max_batch", [1, 4])
def test_copy_path_server_echo(C, max_batch):
    app = C.make_app("echo", -1, 256, 256, [], 64, 1, max_batch)
    with GrpcCopyPathServer(app, max_batch) as srv:
        cli = GrpcClient(srv.address, 256)
        stats = cli.run_closed_loop(outstanding=4, total=120, warmup=20, keep=8)
        assert stats["received"] == 120 and stats["errors"] == 0 and stats["req_per_s"] > 0
        for guid, out in cli.responses.items():
            assert out == cli.payloads[guid % len(cli.payloads)]
        # a short request is zero-padded to the app's request size, a long one is cut
        assert cli.one(1000, b"xyz") == b"xyz" + bytes(253)
        assert cli.one(1001, bytes(range(256)) + b"tail") == bytes(range(256))
        cli.close()
        t = srv.times()
    assert t["requests"] == 142 and 1 <= t["batches"] <= 142
    if max_batch == 1:
        assert t["batches"] == 142
    assert srv.calls == 142 and srv.errors == 0


def test_copy_path_server_lenet_matches_oracle(C):
    rng = np.random.default_rng(5)
    shapes = [(20, 1, 5, 5), (50, 20, 5, 5), (10, 1250), (10,)]
    w = [(rng.standard_normal(s) * 0.2).astype(np.float32) for s in shapes]
    app = C.make_app("lenet_ref", -1, 784, 40, w, 64, 1, 4)
    with GrpcCopyPathServer(app, 4) as srv:
        cli = GrpcClient(srv.address, 784)
        stats = cli.run_closed_loop(outstanding=4, total=16, warmup=0, keep=4)
        assert stats["received"] == 16 and stats["errors"] == 0
        for guid, out in cli.responses.items():
            probs = np.frombuffer(out, dtype=np.float32)
            assert probs.shape == (10,) and abs(float(probs.sum()) - 1.0) < 1e-4
        # the same image twice gives the same answer, whatever batch it travelled in
        a, b = cli.one(77, cli.payloads[0]), cli.one(78, cli.payloads[0])
        assert a == b
        cli.close()


def test_load_generator_client_type_1(C, capsys):
    import json

    from splitrpc_b200.utils import client

    app = C.make_app("echo", -1, 1024, 1024, [], 64, 1, 2)
    with GrpcCopyPathServer(app, 2) as srv:
        host, port = srv.address.rsplit(":", 1)
        rc = client.main(["--server-ip", host, "--server-port", port, "--app", "echo", "--req-size", "1024", "--resp-size", "1024",
                          "--total", "40", "--warmup", "10", "--outstanding", "2", "--client-type", "1"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["ok"] and out["received"] == 40


def test_load_generator_main_reads_the_original_environment(C, capsys, monkeypatch):
    """No flags at all: server address, sizes, counts, loop type and client type come from the P2P_RPC_* variables."""
    import json

    from splitrpc_b200.utils import client

    app = C.make_app("echo", -1, 512, 512, [], 64, 1, 2)
    with GrpcCopyPathServer(app, 2) as srv:
        host, port = srv.address.rsplit(":", 1)
        env = {"P2P_RPC_URI": f"00:00:00:00:00:01,127.0.0.1,0,00:00:00:00:00:02,{host},{port}", "P2P_RPC_APP": "echo",
               "P2P_RPC_REQ_SIZE": "512", "P2P_RPC_RESP_SIZE": "512", "P2P_RPC_BENCH_TOTAL_REQUESTS": "30", "P2P_RPC_REQ_GEN_TYPE": "0",
               "P2P_RPC_BENCH_ARR_RATE": "3", "P2P_RPC_CLIENT_TYPE": "1", "P2P_RPC_CLIENT_VERIFY_RUN": "1"}
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        monkeypatch.delenv("P2P_RPC_NUM_WARMUP", raising=False)
        rc = client.main([])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["ok"] and out["received"] == 30  # 3 warm-up calls (10 %) come on top
    assert srv.calls == 33
