"""The host core under ThreadSanitizer and AddressSanitizer/UBSan: a stand-alone program (no Python, no CUDA) runs the
server threads, the CPU engine and apps, the load generator with fault injection and a replica behind a batched server,
and must finish without a single report."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "splitrpc_b200", "csrc", "host", "selftest_main.cpp")


@pytest.mark.parametrize("flags,name", [("-fsanitize=thread", "tsan"), ("-fsanitize=address,undefined", "asan")])
def test_host_core_is_clean_under_sanitizers(tmp_path, flags, name):
    exe = tmp_path / f"selftest_{name}"
    # the system compiler first (it ships the sanitizer runtimes), then whatever CXX names
    compilers = [c for c in dict.fromkeys([shutil.which("g++"), shutil.which(os.environ.get("CXX", "g++")), shutil.which("clang++")]) if c]
    if not compilers:
        pytest.skip("no C++ compiler")
    b = None
    for cxx in compilers:
        cmd = [cxx, "-std=c++17", "-O1", "-g", *flags.split(), "-fno-omit-frame-pointer", "-pthread", "-I",
               os.path.join(ROOT, "splitrpc_b200", "csrc"), SRC, "-o", str(exe), "-lrt"]
        b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        if b.returncode == 0:
            break
    if b.returncode != 0 and any(m in b.stderr for m in ("cannot find -ltsan", "cannot find -lasan", "cannot find -lubsan", "libtsan", "libasan")):
        pytest.skip("no compiler here ships the sanitizer runtime")
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=67",
               UBSAN_OPTIONS="print_stacktrace=1 halt_on_error=0")
    r = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=600, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "SELFTEST OK" in out, out[-4000:]
    assert "ThreadSanitizer" not in out and "AddressSanitizer" not in out and "runtime error" not in out, out[-4000:]


def test_host_core_builds_and_reports_in_profile_mode(tmp_path):
    """-DPROFILE_MODE compiles the per-stage timers (and NVTX ranges where the header is present) into the host core;
    the engines print their [N, Mean, p90, p95, p99, min, max] lines at teardown."""
    cxx = shutil.which("g++") or shutil.which(os.environ.get("CXX", "g++"))
    if not cxx:
        pytest.skip("no C++ compiler")
    exe = tmp_path / "selftest_prof"
    cmd = [cxx, "-std=c++17", "-O1", "-DPROFILE_MODE", "-pthread", "-I", os.path.join(ROOT, "splitrpc_b200", "csrc"), SRC, "-o",
           str(exe), "-lrt"]
    cuda_inc = "/usr/local/cuda/include"
    if os.path.isdir(cuda_inc):
        cmd[1:1] = ["-I", cuda_inc]  # nvtx3 headers, when present
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "SELFTEST OK" in out, out[-3000:]
    lines = [l for l in out.splitlines() if l.startswith("Gather stats(ns) [N, Mean, p90, p95, p99, min, max]:")]
    assert lines and any(int(l.split(":")[1].split(",")[0]) > 0 for l in lines), out[-3000:]
