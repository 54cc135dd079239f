"""The command-line mains as separate processes on the CPU device: a replica behind a batched server, an ingress that
is a pure proxy over kernel UDP, and the load generator."""
import json
import os
import signal
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(mod, *args):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), PYTHONUNBUFFERED="1")
    return subprocess.Popen([sys.executable, "-m", mod, *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                            text=True, env=env, cwd=ROOT)


def _first_json(proc, timeout=90):
    t0 = time.time()
    while time.time() - t0 < timeout:
        line = proc.stdout.readline()
        if line.startswith("{"):
            return json.loads(line)
        if not line and proc.poll() is not None:
            break
    raise AssertionError("no JSON line from the process: " + proc.stderr.read()[-2000:])


def _finish(proc):
    proc.send_signal(signal.SIGTERM)
    out, err = proc.communicate(timeout=60)
    lines = [json.loads(l) for l in out.splitlines() if l.startswith("{")]
    assert proc.returncode == 0, err[-2000:]
    return lines[-1]


@pytest.mark.parametrize("pull", [False, True])
def test_replica_ingress_and_client_mains(tmp_path, pull):
    sock = str(tmp_path / "echo.sock")
    common = ("--app", "echo", "--req-size", 3000, "--resp-size", 1000, "--mtu", 1024, "--max-batch", 4)
    rep = _spawn("splitrpc_b200.serving.replica", *common, "--device", -1, "--path", sock, "--pool", 64)
    ing = None
    try:
        assert _first_json(rep)["event"] == "listening"
        extra = ("--pull",) if pull else ()
        ing = _spawn("splitrpc_b200.serving.ingress", *common, "--device", -1, "--no-local", "--ip", "127.0.0.1", "--port", 0,
                     "--replica", sock, "--pool", 64, *extra)
        hello = _first_json(ing)
        assert hello["event"] == "listening" and hello["replicas"] == 1 and bool(hello["remote"][0]["pull"]) == pull
        cli = _spawn("splitrpc_b200.utils.client", "--server-port", hello["udp_port"], "--app", "echo", "--req-size", 3000,
                     "--resp-size", 1000, "--mtu", 1024, "--total", 200, "--warmup", 20, "--outstanding", 4, "--verify")
        out, err = cli.communicate(timeout=120)
        st = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
        assert cli.returncode == 0 and st["ok"] and st["received"] == 220 and st["verify_failures"] == 0, (st, err[-1000:])
        assert st["n_sojournTime"] == 200 and st["p99_sojournTime_us"] >= st["p50_sojournTime_us"] > 0
        bye = _finish(ing)
        ing = None
        assert bye["stats"]["replicas"][0]["completed"] == 220 and bye["released"] == 1
        served = _finish(rep)
        rep = None
        assert served["served"] == 220 and served["counters"]["releases"] == 1
        assert served["pull"]["pulled"] == (220 if pull else 0)
    finally:
        for p in (ing, rep):
            if p is not None and p.poll() is None:
                p.kill()
