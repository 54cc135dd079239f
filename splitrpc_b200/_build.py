"""In-tree build of the native library ``splitrpc_b200/_C*.so``.

One shared object holds the C++ host core, every CUDA kernel (compiled for
sm_100a only) and the pybind11 bindings.  Objects are cached under
``splitrpc_b200/build/`` keyed by a hash of the source, its headers and the
flags, so a rebuild only recompiles what changed.  ``nvcc`` cross-compiles
without a GPU; the CUDA runtime is linked statically and driver entry points are
resolved at run time, so the library imports on a machine without a driver.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
TARGET = PKG / f"_C{EXT_SUFFIX}"

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = GENCODE + [
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-O3,-Wall,-Wno-unused-function",
    "-Xcudafe", "--diag_suppress=177",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-fvisibility=hidden", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the native library cannot be built")


def _includes() -> list[str]:
    import pybind11

    cuda_home = Path(_nvcc()).resolve().parent.parent
    return [f"-I{CSRC}", f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_home}/include"]


def sources() -> list[Path]:
    out = sorted(CSRC.glob("*.cpp")) + sorted((CSRC / "cuda").glob("*.cu"))
    return out


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _obj_for(src: Path, hdr_digest: str, verbose_ptxas: bool) -> tuple[Path, list[str]]:
    is_cu = src.suffix == ".cu"
    # SPLITRPC_NVCC_EXTRA: extra nvcc flags for a one-off build, e.g. -DSRPC_GEMM_TRACE (phase time stamps in the GEMM)
    extra = os.environ.get("SPLITRPC_NVCC_EXTRA", "").split()
    # SPLITRPC_PROFILE=1: per-stage host timers and NVTX ranges on the server threads (-DPROFILE_MODE)
    prof = ["-DPROFILE_MODE"] if os.environ.get("SPLITRPC_PROFILE") == "1" else []
    prof += _dpdk_flags()[0]
    flags = (NVCC_FLAGS + extra + prof + (["-Xptxas", "-v"] if verbose_ptxas else [])) if is_cu else CXX_FLAGS + prof
    key = hashlib.sha256((src.read_text() + hdr_digest + " ".join(flags)).encode()).hexdigest()[:16]
    obj = BUILD / f"{src.stem}.{key}.o"
    if is_cu:
        cmd = [_nvcc(), "-c", str(src), "-o", str(obj)] + flags + _includes()
    else:
        cmd = [os.environ.get("CXX", "g++"), "-c", str(src), "-o", str(obj)] + flags + _includes()
    return obj, cmd


def _dpdk_flags() -> tuple[list[str], list[str]]:
    """SPLITRPC_WITH_DPDK=1: compile the DPDK port (csrc/host/dpdk_port.h) against the libdpdk that pkg-config finds."""
    if os.environ.get("SPLITRPC_WITH_DPDK") != "1":
        return [], []
    try:
        cflags = subprocess.run(["pkg-config", "--cflags", "libdpdk"], capture_output=True, text=True, check=True).stdout.split()
        libs = subprocess.run(["pkg-config", "--libs", "libdpdk"], capture_output=True, text=True, check=True).stdout.split()
    except (OSError, subprocess.CalledProcessError) as e:
        raise RuntimeError("SPLITRPC_WITH_DPDK=1 but pkg-config does not know libdpdk") from e
    # nvcc takes host-compiler options through -Xcompiler; keep only what both compilers understand
    cflags = [f for f in cflags if f.startswith(("-I", "-D"))]
    return ["-DSPLITRPC_WITH_DPDK"] + cflags, libs


def build(force: bool = False, verbose: bool = False, verbose_ptxas: bool = False) -> Path:
    """Compiles what changed and links ``_C``; returns the path of the library.

    Safe to call from several processes at once (one rank per GPU importing the package at the same time): a file lock
    serialises them, the winner builds, the others find the result up to date; the library is linked under a temporary
    name and moved into place atomically, so no process ever maps a half-written file."""
    import fcntl

    BUILD.mkdir(exist_ok=True)
    with open(BUILD / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not verbose_ptxas and up_to_date():
                return TARGET
            return _build_locked(force, verbose, verbose_ptxas)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool, verbose_ptxas: bool) -> Path:
    hdr = _headers_digest()
    jobs = [_obj_for(s, hdr, verbose_ptxas) for s in sources()]
    todo = [(o, c) for o, c in jobs if force or not o.exists()]

    def run(job):
        obj, cmd = job
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        if (verbose or verbose_ptxas) and (r.stdout or r.stderr):
            print(r.stdout + r.stderr, flush=True)
        return obj

    if todo:
        with ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(run, todo))
    objs = [o for o, _ in jobs]
    stamp = BUILD / "link.stamp"
    link_key = hashlib.sha256(" ".join(o.name for o in objs).encode()).hexdigest()  # names, not paths: the tree may move
    if force or todo or not TARGET.exists() or not stamp.exists() or stamp.read_text() != link_key:
        tmp = TARGET.with_name(TARGET.name + f".tmp{os.getpid()}")
        cmd = [_nvcc(), "-shared", "-o", str(tmp)] + [str(o) for o in objs] + GENCODE + ["-cudart", "static", "-lpthread", "-ldl", "-lrt"] + _dpdk_flags()[1]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, TARGET)
        stamp.write_text(link_key)
        # drop objects of older source versions
        keep = {o.name for o in objs}
        for p in BUILD.glob("*.o"):
            if p.name not in keep:
                p.unlink()
    return TARGET


def up_to_date() -> bool:
    """True when the library exists and was linked from the objects of the current sources, headers and flags."""
    if not TARGET.exists():
        return False
    hdr = _headers_digest()
    objs = [_obj_for(s, hdr, False)[0] for s in sources()]
    if not all(o.exists() for o in objs):
        return False
    stamp = BUILD / "link.stamp"
    return stamp.exists() and stamp.read_text() == hashlib.sha256(" ".join(o.name for o in objs).encode()).hexdigest()


if __name__ == "__main__":
    t = build(force="--force" in sys.argv, verbose="-v" in sys.argv, verbose_ptxas="--ptxas" in sys.argv)
    print(t)
