"""Run under torchrun on 2+ GPUs: one ingress (rank 0) feeding replicas on every GPU.

Rank 0 owns the loopback transport and the native server, serves one replica on GPU 0 and produces into the request
rings of the replicas that the other ranks serve behind batched servers: its gather kernel stores the payload into
the peer GPU's ring over NVLink and rings the slot doorbells; the serving GPU's kernels store the responses into rank
0's transmit arena and complete the slots.  Checks: echo replies are byte-exact, every replica served its share, every
response was pushed by the serving side; ResNet-50 responses equal the single-GPU forward of the same weights.
Prints ``INGRESS_OK`` on rank 0."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import numpy as np
import torch
import torch.distributed as dist

from splitrpc_b200 import _C, ops
from splitrpc_b200.models import ResNet50
from splitrpc_b200.serving import ModelReplica, ModelServer

FUNC = 1234


def sock_path(tag, rank):
    return os.path.join(tempfile.gettempdir(), f"srpc_{os.environ.get('MASTER_PORT', '0')}_{tag}_{rank}.sock")


def check_echo(rank, world, pull=False):
    """Generic app (no fused response writer): the push kernel behind the app stores the responses.  With ``pull`` the
    ingress only describes the requests and every serving GPU fetches the fragments from the shared host memory."""
    req = 3 * 8192 + 512  # four fragments, the last one short
    resp = 4096           # one fragment: pushed by the serving GPU
    _C.set_rpc_mtu(8192)
    app = _C.make_app("echo", rank, req, resp, [], 128, 1, 8, "gpu", 2)
    if rank == 0:
        sp, cp = _C.make_loopback_pair(8192, 4096, "shm_pinned")
        srv = _C.Server(sp, req_size=req, resp_size=resp, server_mode=2, max_batch=8, gather_burst=8)
        srv.add_replica(app)
        dist.barrier()  # the batched servers are listening
        for r in range(1, world):
            srv.add_remote_replica(sock_path("echo", r), func_id=FUNC, ingress_device=0, copy_type=2, pull=pull)
            info = srv.remote_info(r - 1)
            assert info["device_id"] == r and info["device_completes"] == 1 and bool(info["pull"]) == pull, info
        srv.start()
        total = 200 * world
        # pulled requests come both ways: copied into the receive arena (one descriptor per fragment) and handed over
        # by reference (one descriptor per request, in a region announced after the handshake)
        cli = _C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=0, payload="echo", verify=True)
        ok = cli.run_closed_loop(8 * world)
        if pull:
            cli2 = _C.Client(cp, req_size=req, resp_size=resp, total=total, warmup=0, payload="echo", verify=True,
                             send_by_reference=True, n_payloads=8, seed=3)
            ok = ok and cli2.run_closed_loop(8 * world) and cli2.received == total and cli2.verify_failures == 0
        lat = srv.device_latency_ns()
        assert lat and 0 < min(lat) and max(lat) < 2_000_000_000, (min(lat), max(lat))
        st = srv.stats()
        srv.stop()
        released = srv.release_remotes()
        assert ok and cli.received == total and cli.verify_failures == 0, (cli.received, cli.verify_failures, st)
        assert st["sg_errors"] == 0 and released == world - 1, st
        for i, rs in enumerate(st["replicas"]):
            assert rs["steered"] >= total // (2 * world) and rs["pushed"] == rs["completed"] == rs["steered"], (i, st)
        dist.barrier()
    else:
        bs = _C.BatchedServer(app, sock_path("echo", rank), func_id=FUNC, server_mode=2, max_batch=8)
        bs.start()
        dist.barrier()
        dist.barrier()  # rank 0 has released
        ctr = bs.counters()
        served = bs.worker_stats()["num_req"]
        pulled = bs.pull_stats()
        bs.stop()
        assert ctr["allocs"] == 1 and ctr["releases"] == 1 and ctr["peers_lost"] == 0 and served > 0, (ctr, served)
        assert pulled["errors"] == 0 and pulled["pulled"] == (served if pull else 0), (pulled, served)
    ops.check_status()


def check_resnet(rank, world, pull=False):
    """Fused ingress (gather + deserialise, over NVLink or by the serving GPU itself) and fused response (softmax +
    store into the ingress arena)."""
    nb = 8
    model = ResNet50(device=rank, max_batch=nb)
    if rank == 0:
        srv = ModelServer(model, device=0, max_batch=nb, outstanding=3 * nb * world, n_replicas=world)
        dist.barrier()
        for r in range(1, world):
            srv.add_remote(sock_path("resnet", r), pull=pull)
        n_pay = 4
        total = 6 * nb * world
        with srv:
            cli = srv.client(total=total, warmup=0, payload="normal", verify=True, n_payloads=n_pay, send_by_reference=pull)
            ok = cli.run_closed_loop(2 * nb * world)
            st = srv.server.stats()
        assert ok and cli.received == total and st["sg_errors"] == 0, (cli.received, st)
        for i, rs in enumerate(st["replicas"]):
            assert rs["steered"] > 0 and rs["pushed"] == rs["completed"] == rs["steered"], (i, st)
        # every response equals the direct forward of its payload on GPU 0, whichever GPU served it
        direct = torch.zeros(n_pay, 1000, device="cuda:0")
        x = torch.stack([torch.from_numpy(np.frombuffer(cli.payload(i), dtype=np.float32).copy()).view(3, 224, 224)
                         for i in range(n_pay)]).cuda(0)
        model.forward(n_pay, x=x, out=direct)
        torch.cuda.synchronize()
        for i in range(total):
            got = torch.from_numpy(np.frombuffer(cli.response(i), dtype=np.float32).copy())
            torch.testing.assert_close(got, direct[i % n_pay].cpu(), rtol=1e-3, atol=1e-5)
        dist.barrier()
    else:
        rep = ModelReplica(model, sock_path("resnet", rank), device=rank, max_batch=nb)
        rep.start()
        dist.barrier()
        dist.barrier()
        served = rep.batched.worker_stats()["num_req"]
        rep.stop()
        assert served > 0
    ops.check_status()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")
    for pull in (False, True):
        check_echo(rank, world, pull)
        dist.barrier()
        check_resnet(rank, world, pull)
        dist.barrier()
    if rank == 0:
        print("INGRESS_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
