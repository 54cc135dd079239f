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
